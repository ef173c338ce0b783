"""Thin tensor-level wrappers over the C ABI (``include/pimb200.h``).

torch is used for device memory and streams only: every function passes raw ``data_ptr()``
values and sizes through ctypes into libpimb200.so.  Nothing here computes on the host and
nothing falls back to a PyTorch op.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import (ACT_NONE, ACT_RELU, LSTM_AUTO, LSTM_PERSISTENT, LSTM_PERSISTENT_TAGGED,  # noqa: F401
                   LSTM_STREAMED, check)

_initialised: set[int] = set()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _req_half_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.float16:
            raise TypeError("expected a CUDA fp16 tensor")
        if not t.is_contiguous():
            raise ValueError("expected a contiguous tensor")


def _req_half_cuda_rows(*ts: Optional[torch.Tensor]) -> None:
    """fp16 CUDA views whose last dimension is contiguous (rows may be strided: slices of a wider buffer)."""
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.float16:
            raise TypeError("expected a CUDA fp16 tensor")
        if t.dim() and t.stride(-1) != 1:
            raise ValueError("expected a contiguous last dimension")


def init(device: Optional[int] = None) -> None:
    """pimb200_init for ``device`` (default: the current device); idempotent."""
    dev = torch.cuda.current_device() if device is None else int(device)
    if dev in _initialised:
        return
    check(_lib.lib().pimb200_init(dev), "pimb200_init")
    _initialised.add(dev)


def shutdown(device: Optional[int] = None) -> None:
    dev = torch.cuda.current_device() if device is None else int(device)
    check(_lib.lib().pimb200_shutdown(dev), "pimb200_shutdown")
    _initialised.discard(dev)


def gemv_mv(W: torch.Tensor, x: torch.Tensor, bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[N] = act(W[N,K] @ x[K] + bias)."""
    _req_half_cuda(W, x, bias)
    N, K = W.shape
    assert x.numel() == K
    y = out if out is not None else torch.empty(N, dtype=torch.float16, device=W.device)
    check(_lib.lib().pimb200_gemv_mv(_ptr(W), _ptr(x), _ptr(bias), _ptr(y), N, K, act, _stream()), "gemv_mv")
    return y


def gemv_vm(x: torch.Tensor, A: torch.Tensor, bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[N] = act(x[K] @ A[K,N] + bias)."""
    _req_half_cuda(A, x, bias)
    init(A.device.index)
    K, N = A.shape
    assert x.numel() == K
    y = out if out is not None else torch.empty(N, dtype=torch.float16, device=A.device)
    check(_lib.lib().pimb200_gemv_vm(_ptr(x), _ptr(A), _ptr(bias), _ptr(y), K, N, act, _stream()), "gemv_vm")
    return y


def dot_vv(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    _req_half_cuda(a, b)
    assert a.numel() == b.numel()
    y = torch.empty(1, dtype=torch.float16, device=a.device)
    check(_lib.lib().pimb200_dot_vv(_ptr(a), _ptr(b), _ptr(y), a.numel(), _stream()), "dot_vv")
    return y


def bmm_row(x: torch.Tensor, A: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[n] = x[k] @ A[k,n] (single-row batched matmul of the GNMT attention context)."""
    _req_half_cuda(x, A)
    k, n = A.shape[-2], A.shape[-1]
    assert x.numel() == k
    y = out if out is not None else torch.empty(n, dtype=torch.float16, device=A.device)
    check(_lib.lib().pimb200_bmm_row(_ptr(x), _ptr(A), _ptr(y), k, n, _stream()), "bmm_row")
    return y


def gemm_wx(W: torch.Tensor, X: torch.Tensor, bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
            out_f32: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y[J,N] = act(X[J,K] @ W[N,K]^T + bias).  Rows of X and of `out` may be strided (column slices of wider buffers)."""
    _req_half_cuda(W, bias)
    _req_half_cuda_rows(X)
    N, K = W.shape
    J = X.shape[0]
    assert X.shape[1] == K and X.stride(1) == 1
    if out is None:
        out = torch.empty(J, N, dtype=torch.float32 if out_f32 else torch.float16, device=W.device)
    check(_lib.lib().pimb200_gemm_wx(_ptr(W), _ptr(X), _ptr(bias), _ptr(out), N, K, J, X.stride(0), out.stride(0), act,
                                     1 if out.dtype == torch.float32 else 0, _stream()), "gemm_wx")
    return out


def gemm_wx_grouped(problems: Sequence[tuple], act: int = ACT_NONE) -> list:
    """[(W [N,K], X [J,K], bias or None), ...] -> [Y [J,N], ...]: independent products in one launch when their shapes allow
    it (the branches of a MULTISTREAM node), else one launch each."""
    n = len(problems)
    arr = (_lib.GemmProblem * n)()
    outs = []
    for i, (W, X, b) in enumerate(problems):
        _req_half_cuda(W, b)
        _req_half_cuda_rows(X)
        N, K = W.shape
        J = X.shape[0]
        Y = torch.empty(J, N, dtype=torch.float16, device=W.device)
        outs.append(Y)
        arr[i] = _lib.GemmProblem(W.data_ptr(), X.data_ptr(), _ptr(b), Y.data_ptr(), N, K, J, X.stride(0), N, act, 0)
    check(_lib.lib().pimb200_gemm_wx_grouped(C.cast(arr, C.c_void_p), n, _stream()), "gemm_wx_grouped")
    return outs


def add_f16(A: torch.Tensor, B: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A + B, same shape, or B a single row broadcast over the rows of A."""
    _req_half_cuda(A, B)
    n = A.shape[-1]
    m = A.numel() // n
    bcast = 0 if B.numel() == A.numel() else 1
    if bcast and B.numel() != n:
        raise ValueError("B must match A or be one row of it")
    C_ = out if out is not None else torch.empty_like(A)
    check(_lib.lib().pimb200_add_f16(_ptr(A), _ptr(B), _ptr(C_), m, n, bcast, _stream()), "add_f16")
    return C_


def copy_2d(dst: torch.Tensor, dst_off_bytes: int, dst_pitch: int, src: torch.Tensor, src_off_bytes: int,
            src_pitch: int, row_bytes: int, rows: int) -> None:
    check(_lib.lib().pimb200_copy_2d(dst.data_ptr() + dst_off_bytes, dst_pitch, src.data_ptr() + src_off_bytes,
                                     src_pitch, row_bytes, rows, _stream()), "copy_2d")


def cat(tensors: Sequence[torch.Tensor], dim: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """aten::cat for contiguous CUDA tensors of one dtype, via strided device copies."""
    nonempty = [t for t in tensors if t.numel() > 0]
    ref = nonempty[0] if nonempty else tensors[0]
    nd = ref.dim()
    dim = dim % nd
    shape = list(ref.shape)
    shape[dim] = sum(t.shape[dim] for t in nonempty)
    if out is None:
        out = torch.empty(shape, dtype=ref.dtype, device=ref.device)
    if not nonempty or out.numel() == 0:
        return out
    outer = 1
    for s in shape[:dim]:
        outer *= s
    es = ref.element_size()
    n = len(nonempty)
    srcs = (C.c_void_p * n)(*[t.data_ptr() for t in nonempty])
    inner = (C.c_size_t * n)(*[(t.numel() // max(outer, 1)) * es for t in nonempty])
    for t in nonempty:
        if not t.is_contiguous() or t.dtype != ref.dtype:
            raise ValueError("cat operands must be contiguous and share a dtype")
    check(_lib.lib().pimb200_cat(out.data_ptr(), srcs, inner, n, outer, _stream()), "cat")
    return out


def softmax(x: torch.Tensor, log: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax / log_softmax over the last dimension of a contiguous CUDA fp16 tensor."""
    _req_half_cuda(x)
    cols = x.shape[-1] if x.dim() else 1
    rows = x.numel() // max(cols, 1)
    y = out if out is not None else torch.empty_like(x)
    check(_lib.lib().pimb200_softmax_rows(_ptr(x), _ptr(y), rows, cols, 1 if log else 0, _stream()), "softmax_rows")
    return y


def argmax(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest element along the last dimension (lowest index on ties), int64."""
    _req_half_cuda(x)
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    idx = out if out is not None else torch.empty(x.shape[:-1], dtype=torch.int64, device=x.device)
    if idx.dtype != torch.int64 or not idx.is_cuda or idx.numel() != rows:
        raise TypeError("expected a CUDA int64 tensor with one element per row")
    check(_lib.lib().pimb200_argmax_rows(_ptr(x), idx.data_ptr(), rows, cols, _stream()), "argmax_rows")
    return idx


def topk(x: torch.Tensor, k: int, largest: bool = True):
    """(values, int64 indices) of the k largest / smallest elements along the last dimension, in order."""
    _req_half_cuda(x)
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    vals = torch.empty(*x.shape[:-1], k, dtype=torch.float16, device=x.device)
    idx = torch.empty(*x.shape[:-1], k, dtype=torch.int64, device=x.device)
    check(_lib.lib().pimb200_topk_rows(_ptr(x), _ptr(vals), idx.data_ptr(), rows, cols, k, 1 if largest else 0, _stream()),
          "topk_rows")
    return vals, idx


def layer_norm(x: torch.Tensor, gamma: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
               eps: float = 1e-5) -> torch.Tensor:
    """Layer normalisation over the last dimension."""
    _req_half_cuda(x, gamma, beta)
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    y = torch.empty_like(x)
    check(_lib.lib().pimb200_layer_norm_rows(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), rows, cols, float(eps),
                                             _stream()), "layer_norm_rows")
    return y


def gather_rows(table: torch.Tensor, idx: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """table[idx] for a device-resident int64 index tensor (embedding lookup without a host round trip)."""
    if not table.is_cuda or not table.is_contiguous() or table.dim() != 2:
        raise TypeError("expected a contiguous 2-D CUDA table")
    if idx.dtype != torch.int64 or not idx.is_cuda or not idx.is_contiguous():
        raise TypeError("expected a contiguous CUDA int64 index tensor")
    y = out if out is not None else torch.empty(*idx.shape, table.shape[1], dtype=table.dtype, device=table.device)
    check(_lib.lib().pimb200_gather_rows(table.data_ptr(), idx.data_ptr(), y.data_ptr(), idx.numel(),
                                         table.shape[1] * table.element_size(), table.shape[0], _stream()),
          "gather_rows")
    return y


def scatter_rows(table: torch.Tensor, idx: torch.Tensor, src: torch.Tensor) -> None:
    """table[idx] = src for a device-resident int64 index tensor (in-place KV-cache append at a device-side position)."""
    if not table.is_cuda or not table.is_contiguous() or table.dim() != 2:
        raise TypeError("expected a contiguous 2-D CUDA table")
    if idx.dtype != torch.int64 or not idx.is_cuda or not idx.is_contiguous():
        raise TypeError("expected a contiguous CUDA int64 index tensor")
    if src.dtype != table.dtype or not src.is_cuda or not src.is_contiguous() or src.numel() != idx.numel() * table.shape[1]:
        raise TypeError("src must hold one row of the table's width and dtype per index")
    check(_lib.lib().pimb200_scatter_rows(table.data_ptr(), idx.data_ptr(), src.data_ptr(), idx.numel(),
                                          table.shape[1] * table.element_size(), table.shape[0], _stream()),
          "scatter_rows")


def attention_row(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, heads: int, length: Optional[int] = None,
                  length_dev: Optional[torch.Tensor] = None, length_add: int = 0, scale: Optional[float] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-query multi-head attention over the first L rows of the caches K, V [S, d]: L = `length`, or
    `length_dev` (int64 on the device) + `length_add`."""
    _req_half_cuda(q, K, V)
    d = q.numel()
    hd = d // heads
    if K.shape != V.shape or K.shape[1] != d:
        raise ValueError("K and V must be [S, heads * head_dim]")
    if length_dev is not None and (length_dev.dtype != torch.int64 or not length_dev.is_cuda):
        raise TypeError("length_dev must be a CUDA int64 tensor")
    y = out if out is not None else torch.empty(d, dtype=torch.float16, device=q.device)
    add = length_add if length_dev is not None else (K.shape[0] if length is None else int(length))
    check(_lib.lib().pimb200_attention_row(_ptr(q), _ptr(K), _ptr(V), None if length_dev is None else length_dev.data_ptr(),
                                           add, K.shape[0], _ptr(y), heads, hd, K.stride(0),
                                           float(scale if scale is not None else hd ** -0.5), _stream()),
          "attention_row")
    return y


def attention_rows(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, heads: int, len_dev: Optional[torch.Tensor] = None,
                   len_inc: int = 0, len_add: int = 0, max_len: Optional[int] = None, scale: Optional[float] = None,
                   out: Optional[torch.Tensor] = None, time_major: bool = False) -> torch.Tensor:
    """Single-query multi-head attention for n sequences in lock step: q [n, heads*hd] (rows may be strided); K, V
    [n, S_max, heads*hd] views (one cache per sequence; [S_max, n, heads*hd] with time_major), last dimension contiguous;
    lengths from the int64 device tensor `len_dev` (element j*len_inc for sequence j) plus len_add."""
    _req_half_cuda_rows(q, K, V)
    n, d = q.shape
    hd = d // heads
    seq_dim, t_dim = (1, 0) if time_major else (0, 1)
    S = K.shape[t_dim] if max_len is None else max_len
    if K.stride() != V.stride() or K.stride(2) != 1 or q.stride(1) != 1:
        raise ValueError("K and V must share their strides; the last dimension must be contiguous")
    if out is None:
        out = torch.empty(n, d, dtype=torch.float16, device=q.device)
    check(_lib.lib().pimb200_attention_rows(_ptr(q), _ptr(K), _ptr(V), _ptr(len_dev), len_inc, len_add, S, _ptr(out), n,
                                            heads, hd, K.stride(t_dim), K.stride(seq_dim), q.stride(0), out.stride(0),
                                            scale if scale is not None else 1.0 / math.sqrt(hd), _stream()), "attention_rows")
    return out


def attention_block(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, lengths: Optional[torch.Tensor],
                    out: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Self-attention over all positions of n padded sequences: q, k, v [n, S, heads*hd] views with equal strides (e.g.
    column slices of one fused projection), lengths int64 [n] on the device."""
    _req_half_cuda_rows(q, k, v)
    n, S, d = q.shape
    hd = d // heads
    if not (q.stride() == k.stride() == v.stride()) or q.stride(2) != 1:
        raise ValueError("q, k, v must share their strides; the last dimension must be contiguous")
    if out is None:
        out = torch.empty(n, S, d, dtype=torch.float16, device=q.device)
    check(_lib.lib().pimb200_attention_block(_ptr(q), _ptr(k), _ptr(v), _ptr(lengths), _ptr(out), n, S, heads, hd,
                                             q.stride(1), q.stride(0), out.stride(1), out.stride(0),
                                             scale if scale is not None else 1.0 / math.sqrt(hd), _stream()), "attention_block")
    return out


def add_layer_norm(x: torch.Tensor, r: torch.Tensor, gamma: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
                   eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """layer_norm(x + r) over the last dimension."""
    _req_half_cuda(x, r, gamma, beta)
    cols = x.shape[-1]
    rows = x.numel() // max(cols, 1)
    y = out if out is not None else torch.empty_like(x)
    check(_lib.lib().pimb200_add_layer_norm_rows(_ptr(x), _ptr(r), _ptr(gamma), _ptr(beta), _ptr(y), rows, cols, float(eps),
                                                 _stream()), "add_layer_norm_rows")
    return y


def additive_attention(q: torch.Tensor, keys_proj: torch.Tensor, values: torch.Tensor, lengths: Optional[torch.Tensor],
                       v: torch.Tensor, bias: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
                       scores: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Normalised Bahdanau attention for n sentences: q [n, H]; keys_proj / values time-major [S, n, H] (contiguous);
    lengths int64 [n] on the device; v, bias [H].  `out` may be a column slice of a wider [n, *] buffer."""
    _req_half_cuda(q, v, bias)
    _req_half_cuda_rows(keys_proj, values)
    S, n, H = keys_proj.shape
    if out is None:
        out = torch.empty(n, H, dtype=torch.float16, device=q.device)
    if scores is None:
        scores = torch.empty(n, S, dtype=torch.float32, device=q.device)
    check(_lib.lib().pimb200_additive_attention(_ptr(q), _ptr(keys_proj), _ptr(values), _ptr(lengths), _ptr(v), _ptr(bias),
                                                _ptr(out), _ptr(scores), n, S, H, keys_proj.stride(0), keys_proj.stride(1),
                                                out.stride(0), _stream()), "additive_attention")
    return out


def tanh(x: torch.Tensor) -> torch.Tensor:
    _req_half_cuda(x)
    y = torch.empty_like(x)
    check(_lib.lib().pimb200_tanh_f16(_ptr(x), _ptr(y), x.numel(), _stream()), "tanh_f16")
    return y


def masked_fill(x: torch.Tensor, mask: torch.Tensor, value: float) -> torch.Tensor:
    """x with `value` where mask is set; mask (bool) has x's shape or is one row broadcast over the rows of x."""
    _req_half_cuda(x)
    if mask.dtype != torch.bool or not mask.is_cuda or not mask.is_contiguous():
        raise TypeError("expected a contiguous CUDA bool mask")
    if mask.numel() not in (x.numel(), x.shape[-1]):
        raise ValueError("mask must match x or be one row of it")
    y = torch.empty_like(x)
    check(_lib.lib().pimb200_masked_fill_f16(_ptr(x), mask.data_ptr(), float(value), _ptr(y), x.numel(), mask.numel(),
                                             _stream()), "masked_fill_f16")
    return y


class Lstm:
    """Packed-weight handle of one aten::lstm node (``pimb200_lstm_create`` ... ``_destroy``)."""

    def __init__(self, params: Sequence[torch.Tensor], num_layers: int, bidirectional: bool, input_size: int,
                 hidden_size: int, has_biases: bool = True):
        for p in params:
            _req_half_cuda(p)
        self.L, self.D = num_layers, 2 if bidirectional else 1
        self.I, self.H = input_size, hidden_size
        self.device = params[0].device
        arr = (C.c_void_p * len(params))(*[p.data_ptr() for p in params])
        handle = C.c_void_p()
        check(_lib.lib().pimb200_lstm_create(arr, len(params), num_layers, 1 if bidirectional else 0, input_size,
                                             hidden_size, 1 if has_biases else 0, C.byref(handle)), "lstm_create")
        self._h = handle

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().pimb200_lstm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_variant(self, variant: int) -> None:
        check(_lib.lib().pimb200_lstm_set_variant(self._h, variant), "lstm_set_variant")

    def last_status(self) -> int:
        return _lib.lib().pimb200_lstm_last_status(self._h)

    def set_wavefront(self, on: bool) -> None:
        check(_lib.lib().pimb200_lstm_set_wavefront(self._h, 1 if on else 0), "lstm_set_wavefront")

    def set_packed_lockstep(self, on: bool) -> None:
        check(_lib.lib().pimb200_lstm_set_packed_lockstep(self._h, 1 if on else 0), "lstm_set_packed_lockstep")

    def forward(self, x: torch.Tensor, h0: Optional[torch.Tensor] = None, c0: Optional[torch.Tensor] = None,
                batch_first: bool = False, out=None):
        _req_half_cuda(x, h0, c0)
        if batch_first:
            B, T, _ = x.shape
        else:
            T, B, _ = x.shape
        DH = self.D * self.H
        if out is None:
            y = torch.empty((B, T, DH) if batch_first else (T, B, DH), dtype=torch.float16, device=x.device)
            hn = torch.empty(self.L * self.D, B, self.H, dtype=torch.float16, device=x.device)
            cn = torch.empty_like(hn)
        else:
            y, hn, cn = out
        check(_lib.lib().pimb200_lstm_forward(self._h, _ptr(x), T, B, _ptr(h0), _ptr(c0), _ptr(y), _ptr(hn),
                                              _ptr(cn), 1 if batch_first else 0, _stream()), "lstm_forward")
        return y, hn, cn

    def forward_step(self, x: torch.Tensor, h0: Optional[torch.Tensor], c0: Optional[torch.Tensor], y: torch.Tensor,
                     hn: torch.Tensor, cn: torch.Tensor, residual: Optional[torch.Tensor] = None) -> bool:
        """Decode step for B >= 8 sequences with strided rows: x [B, >= I] and y [B, >= H] may be column slices of wider
        buffers, y = h (+ residual).  Returns False when the shape is not the decode form (use forward())."""
        _req_half_cuda(h0, c0, hn, cn)
        _req_half_cuda_rows(x, y, residual)
        B = x.shape[0]
        rc = _lib.lib().pimb200_lstm_forward_step(self._h, _ptr(x), x.stride(0), B, _ptr(h0), _ptr(c0), _ptr(y), y.stride(0),
                                                  _ptr(hn), _ptr(cn), _ptr(residual),
                                                  residual.stride(0) if residual is not None else 0, _stream())
        if rc == _lib.ERR_UNSUPPORTED:
            return False
        check(rc, "lstm_forward_step")
        return True

    def forward_packed(self, data: torch.Tensor, batch_sizes: torch.Tensor, h0: Optional[torch.Tensor] = None,
                       c0: Optional[torch.Tensor] = None):
        _req_half_cuda(data, h0, c0)
        bs = [int(v) for v in batch_sizes.tolist()]
        T = len(bs)
        B = bs[0]
        arr = (C.c_int64 * T)(*bs)
        y = torch.empty(data.shape[0], self.D * self.H, dtype=torch.float16, device=data.device)
        hn = torch.empty(self.L * self.D, B, self.H, dtype=torch.float16, device=data.device)
        cn = torch.empty_like(hn)
        check(_lib.lib().pimb200_lstm_forward_packed(self._h, _ptr(data), arr, T, _ptr(h0), _ptr(c0), _ptr(y),
                                                     _ptr(hn), _ptr(cn), _stream()), "lstm_forward_packed")
        return y, hn, cn
