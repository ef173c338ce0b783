"""ctypes binding of libpimb200.so — the only way Python code in this package reaches the kernels.

There is no fall-back: if the shared library is missing or a symbol declared in
``include/pimb200.h`` is absent, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
LIB_PATH = os.path.join(PKG_DIR, "libpimb200.so")
HEADER_PATHS = [os.path.join(ROOT, "include", "pimb200.h"), os.path.join(ROOT, "include", "pimb200_rnnt.h")]

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_TIMEOUT, ERR_NOT_INIT, ERR_NO_MEMORY = range(7)
ACT_NONE, ACT_RELU = 0, 1
LSTM_AUTO, LSTM_STREAMED, LSTM_PERSISTENT, LSTM_PERSISTENT_TAGGED = 0, 1, 2, 3

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t

# name -> (restype, argtypes); must list every function declared in include/pimb200.h
class GemmProblem(C.Structure):
    """pimb200_gemm_problem of include/pimb200.h."""
    _fields_ = [("W", C.c_void_p), ("X", C.c_void_p), ("bias", C.c_void_p), ("Y", C.c_void_p), ("N", C.c_int), ("K", C.c_int),
                ("J", C.c_int), ("ldx", C.c_int), ("ldy", C.c_int), ("act", C.c_int), ("y_is_f32", C.c_int)]


SIGNATURES = {
    "pimb200_status_string": (C.c_char_p, [_i]),
    "pimb200_init": (_i, [_i]),
    "pimb200_shutdown": (_i, [_i]),
    "pimb200_gemv_mv": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pimb200_gemv_vm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pimb200_gemv_vm_static": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pimb200_dot_vv": (_i, [_vp, _vp, _vp, _i, _vp]),
    "pimb200_bmm_row": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "pimb200_gemm_wx": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "pimb200_gemm_last_status": (_i, []),
    "pimb200_gemm_force_simt": (_i, [_i]),
    "pimb200_add_f16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "pimb200_copy_2d": (_i, [_vp, _sz, _vp, _sz, _sz, _sz, _vp]),
    "pimb200_cat": (_i, [_vp, C.POINTER(_vp), C.POINTER(_sz), _i, _sz, _vp]),
    "pimb200_softmax_rows": (_i, [_vp, _vp, C.c_long, C.c_long, _i, _vp]),
    "pimb200_argmax_rows": (_i, [_vp, _vp, C.c_long, C.c_long, _vp]),
    "pimb200_layer_norm_rows": (_i, [_vp, _vp, _vp, _vp, C.c_long, C.c_long, C.c_float, _vp]),
    "pimb200_tanh_f16": (_i, [_vp, _vp, _sz, _vp]),
    "pimb200_attention_row": (_i, [_vp, _vp, _vp, _vp, C.c_long, C.c_long, _vp, _i, _i, C.c_long, C.c_float, _vp]),
    "pimb200_gemm_wx_grouped": (_i, [_vp, _i, _vp]),
    "pimb200_attention_rows": (_i, [_vp, _vp, _vp, _vp, C.c_long, C.c_long, C.c_long, _vp, _i, _i, _i, C.c_long, C.c_long,
                                    C.c_long, C.c_long, C.c_float, _vp]),
    "pimb200_attention_block": (_i, [_vp, _vp, _vp, _vp, _vp, _i, C.c_long, _i, _i, C.c_long, C.c_long, C.c_long, C.c_long,
                                     C.c_float, _vp]),
    "pimb200_add_layer_norm_rows": (_i, [_vp, _vp, _vp, _vp, _vp, C.c_long, C.c_long, C.c_float, _vp]),
    "pimb200_additive_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, C.c_long, _i, C.c_long, C.c_long,
                                        C.c_long, _vp]),
    "pimb200_gather_rows": (_i, [_vp, _vp, _vp, C.c_long, _sz, C.c_long, _vp]),
    "pimb200_scatter_rows": (_i, [_vp, _vp, _vp, C.c_long, _sz, C.c_long, _vp]),
    "pimb200_masked_fill_f16": (_i, [_vp, _vp, C.c_float, _vp, _sz, _sz, _vp]),
    "pimb200_topk_rows": (_i, [_vp, _vp, _vp, C.c_long, C.c_long, _i, _i, _vp]),
    "pimb200_lstm_create": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "pimb200_lstm_destroy": (_i, [_vp]),
    "pimb200_lstm_set_variant": (_i, [_vp, _i]),
    "pimb200_lstm_set_packed_lockstep": (_i, [_vp, _i]),
    "pimb200_lstm_set_wavefront": (_i, [_vp, _i]),
    "pimb200_rnnt_set_wavefront": (_i, [_vp, _i]),
    "pimb200_lstm_forward_step": (_i, [_vp, _vp, C.c_long, _i, _vp, _vp, _vp, C.c_long, _vp, _vp, _vp, C.c_long, _vp]),
    "pimb200_lstm_forward": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "pimb200_lstm_forward_packed": (_i, [_vp, _vp, C.POINTER(C.c_int64), _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "pimb200_lstm_last_status": (_i, [_vp]),
    "pimb200_lstm_profile_enable": (_i, [_vp, _i]),
    "pimb200_lstm_profile_read": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_long), C.POINTER(C.c_double)]),
    "pimb200_lstm_set_poll_limit": (_i, [_vp, _i]),
    "pimb200_lstm_set_use_tc": (_i, [_vp, _i]),
    "pimb200_lstm_set_bulk_wide": (_i, [_vp, _i]),
    "pimb200_lstm_set_pipe_group_size": (_i, [_vp, _i]),
    "pimb200_rnnt_profile_enable": (_i, [_vp, _i]),
    "pimb200_rnnt_profile_read": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_long), C.POINTER(C.c_double)]),
    "pimb200_rnnt_create": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "pimb200_rnnt_destroy": (_i, [_vp]),
    "pimb200_rnnt_decode": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp]),
    "pimb200_rnnt_set_encoder_batch": (_i, [_vp, _i]),
    "pimb200_rnnt_set_greedy_multi": (_i, [_vp, _i]),
    "pimb200_rnnt_info": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_sz)]),
    "pimb200_rnnt_last_status": (_i, [_vp]),
    "pimb200_rnnt_set_poll_limit": (_i, [_vp, _i]),
    "pimb200_rnnt_set_trace": (_i, [_vp, _vp]),
    "pimb200_lstm_set_exchange_copies": (_i, [_vp, _i]),
    "pimb200_lstm_set_exchange_stride": (_i, [_vp, _i]),
    "pimb200_lstm_set_trace": (_i, [_vp, _vp]),
}


class RnntConfigC(C.Structure):
    """struct pimb200_rnnt_config (include/pimb200_rnnt.h)."""
    _fields_ = [(n, _i) for n in ("feat_dim", "enc_hidden", "pre_layers", "post_layers", "stack_factor",
                                  "pred_hidden", "pred_layers", "joint_hidden", "vocab", "blank", "max_symbols")]


class RnntWeightsC(C.Structure):
    """struct pimb200_rnnt_weights (include/pimb200_rnnt.h)."""
    _fields_ = [("pre_params", C.POINTER(_vp)), ("n_pre", _i), ("post_params", C.POINTER(_vp)), ("n_post", _i),
                ("embedding", _vp), ("pred_params", C.POINTER(_vp)), ("n_pred", _i),
                ("joint_w1", _vp), ("joint_b1", _vp), ("joint_w2", _vp), ("joint_b2", _vp)]

_lib = None


def declared_symbols() -> list[str]:
    """Function names declared in include/*.h (parsed from the header text)."""
    names = set()
    for path in HEADER_PATHS:
        with open(path) as f:
            text = f.read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(pimb200_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def lib() -> C.CDLL:
    """Load libpimb200.so once and attach argument types.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m pimaicompiler_b200.build` "
            "(there is no CPU or PyTorch fall-back for these ops)")
    handle = C.CDLL(LIB_PATH)
    for name in declared_symbols():
        if not hasattr(handle, name):
            raise RuntimeError(f"libpimb200.so does not export {name}, which include/*.h declares")
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib


class Pimb200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().pimb200_status_string(status).decode()
        super().__init__(f"{where}: status {status} ({msg})")


def check(status: int, where: str) -> None:
    if status != OK:
        raise Pimb200Error(status, where)
