"""numpy-facing wrapper of oracle/liboracle.so (the C restatement in oracle/oracle.c).

Test infrastructure only: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU
baseline leg.  All arrays are float32 numpy arrays; fp16 inputs are widened by the caller.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None
_fp = C.POINTER(C.c_float)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build.build())
    return _lib


def _f(a):
    return None if a is None else a.ctypes.data_as(_fp)


def _c(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def linear(W, X, b=None, relu=False):
    W, X, b = _c(W), _c(X), _c(b)
    X2 = X.reshape(-1, W.shape[1])
    Y = np.empty((X2.shape[0], W.shape[0]), np.float32)
    lib().oracle_linear(_f(W), _f(X2), _f(b), _f(Y), W.shape[0], W.shape[1], X2.shape[0], int(relu))
    return Y.reshape(*X.shape[:-1], W.shape[0])


def vm(x, A, b=None, relu=False):
    x, A, b = _c(x), _c(A), _c(b)
    y = np.empty(A.shape[1], np.float32)
    lib().oracle_vm(_f(x), _f(A), _f(b), _f(y), A.shape[0], A.shape[1], int(relu))
    return y


def add(A, B):
    A, B = _c(A), _c(B)
    n = A.shape[-1]
    m = A.size // n
    out = np.empty_like(A)
    lib().oracle_add(_f(A), _f(B), _f(out), m, n, 0 if B.size == A.size else 1)
    return out


def softmax(x, log=False):
    x = _c(x)
    cols = x.shape[-1]
    y = np.empty_like(x)
    lib().oracle_softmax(_f(x), _f(y), C.c_long(x.size // cols), C.c_long(cols), int(log))
    return y


def argmax(x):
    x = _c(x)
    cols = x.shape[-1]
    idx = np.empty(x.shape[:-1], np.int64)
    lib().oracle_argmax(_f(x), idx.ctypes.data_as(C.POINTER(C.c_longlong)), C.c_long(x.size // cols), C.c_long(cols))
    return idx


def topk(x, k, largest=True):
    x = _c(x)
    cols = x.shape[-1]
    vals = np.empty(x.shape[:-1] + (k,), np.float32)
    idx = np.empty(x.shape[:-1] + (k,), np.int64)
    lib().oracle_topk(_f(x), _f(vals), idx.ctypes.data_as(C.POINTER(C.c_longlong)), C.c_long(x.size // cols), C.c_long(cols),
                      int(k), int(largest))
    return vals, idx


def layer_norm(x, gamma=None, beta=None, eps=1e-5):
    x, gamma, beta = _c(x), _c(gamma), _c(beta)
    cols = x.shape[-1]
    y = np.empty_like(x)
    lib().oracle_layer_norm(_f(x), _f(gamma), _f(beta), _f(y), C.c_long(x.size // cols), C.c_long(cols), C.c_float(eps))
    return y


def tanh(x):
    x = _c(x)
    y = np.empty_like(x)
    lib().oracle_tanh(_f(x), _f(y), C.c_size_t(x.size))
    return y


def masked_fill(x, mask, value):
    x = _c(x)
    mask = np.ascontiguousarray(mask, dtype=np.uint8)
    y = np.empty_like(x)
    lib().oracle_masked_fill(_f(x), mask.ctypes.data_as(C.POINTER(C.c_ubyte)), C.c_float(value), _f(y),
                             C.c_size_t(x.size), C.c_size_t(mask.size))
    return y


def attention_row(q, K, V, heads, length=None, scale=None):
    q, K, V = _c(q), _c(K), _c(V)
    d = q.size
    hd = d // heads
    L = K.shape[0] if length is None else int(length)
    out = np.empty(d, np.float32)
    lib().oracle_attention_row(_f(q), _f(K), _f(V), C.c_long(L), _f(out), heads, hd, C.c_long(K.shape[1]),
                               C.c_float(hd ** -0.5 if scale is None else scale))
    return out


def cat(arrays, dim):
    arrays = [np.ascontiguousarray(a) for a in arrays if a.size > 0]
    ref = arrays[0]
    dim = dim % ref.ndim
    shape = list(ref.shape)
    shape[dim] = sum(a.shape[dim] for a in arrays)
    out = np.empty(shape, ref.dtype)
    outer = int(np.prod(shape[:dim], dtype=np.int64)) if dim > 0 else 1
    n = len(arrays)
    srcs = (C.c_void_p * n)(*[a.ctypes.data for a in arrays])
    inner = (C.c_size_t * n)(*[a.nbytes // max(outer, 1) for a in arrays])
    lib().oracle_cat(C.c_void_p(out.ctypes.data), srcs, inner, n, C.c_size_t(outer))
    return out


def _params(params):
    ps = [_c(p) for p in params]
    arr = (_fp * len(ps))(*[_f(p) for p in ps])
    return ps, arr


def lstm(x, params, num_layers, bidirectional, has_biases=True, h0=None, c0=None, batch_first=False,
         emulate_fp16=False):
    """at::lstm(input, hx, params, has_biases, num_layers, 0, False, bidirectional, batch_first)."""
    x = _c(x)
    if batch_first:
        x = np.ascontiguousarray(x.transpose(1, 0, 2))
    T, B, I = x.shape
    H = params[1].shape[1]
    D = 2 if bidirectional else 1
    ps, arr = _params(params)
    h0, c0 = _c(h0), _c(c0)
    y = np.empty((T, B, D * H), np.float32)
    hn = np.empty((num_layers * D, B, H), np.float32)
    cn = np.empty_like(hn)
    lib().oracle_lstm(_f(x), T, B, I, H, num_layers, int(bidirectional), int(has_biases), arr, _f(h0), _f(c0),
                      _f(y), _f(hn), _f(cn), int(emulate_fp16))
    if batch_first:
        y = np.ascontiguousarray(y.transpose(1, 0, 2))
    return y, hn, cn


def lstm_packed(data, batch_sizes, params, num_layers, bidirectional, has_biases=True, h0=None, c0=None,
                emulate_fp16=False):
    """at::lstm(data, batch_sizes, hx, params, has_biases, num_layers, 0, False, bidirectional)."""
    data = _c(data)
    bs = np.ascontiguousarray(batch_sizes, dtype=np.int64)
    T, B = len(bs), int(bs[0])
    I = data.shape[1]
    H = params[1].shape[1]
    D = 2 if bidirectional else 1
    ps, arr = _params(params)
    h0, c0 = _c(h0), _c(c0)
    y = np.empty((data.shape[0], D * H), np.float32)
    hn = np.empty((num_layers * D, B, H), np.float32)
    cn = np.empty_like(hn)
    lib().oracle_lstm_packed(_f(data), bs.ctypes.data_as(C.POINTER(C.c_int64)), T, I, H, num_layers,
                             int(bidirectional), int(has_biases), arr, _f(h0), _f(c0), _f(y), _f(hn), _f(cn),
                             int(emulate_fp16))
    return y, hn, cn


def rnnt_greedy(w, feats, cfg, forced=None):
    """oracle_rnnt_greedy: returns (tokens, logits [Tp,V], choice [Tp]).  `w` holds numpy/torch fp32 arrays
    with the fields of oracle.torch_oracle.RnntWeights."""
    def arr(t):
        return _c(t.numpy() if hasattr(t, "numpy") else t)
    feats = arr(feats)
    T = feats.shape[0]
    Tp = T // cfg.stack_factor
    pre, pre_arr = _params([arr(p) for p in w.pre])
    post, post_arr = _params([arr(p) for p in w.post])
    pred, pred_arr = _params([arr(p) for p in w.pred])
    emb, w1, b1, w2, b2 = (arr(t) for t in (w.embedding, w.w1, w.b1, w.w2, w.b2))
    tokens = np.zeros(max(Tp, 1), np.int32)
    logits = np.zeros((Tp, cfg.vocab), np.float32)
    choice = np.zeros(max(Tp, 1), np.int32)
    ip = C.POINTER(C.c_int)
    forced_arr = None if forced is None else np.ascontiguousarray(forced, dtype=np.int32)
    fn = lib().oracle_rnnt_greedy
    fn.restype = C.c_int
    n = fn(_f(feats), T, cfg.feat_dim, cfg.enc_hidden, cfg.pre_layers, cfg.post_layers, cfg.stack_factor,
           cfg.pred_hidden, cfg.joint_hidden, cfg.vocab, cfg.blank, pre_arr, post_arr, _f(emb), pred_arr,
           _f(w1), _f(b1), _f(w2), _f(b2), None if forced_arr is None else forced_arr.ctypes.data_as(ip),
           tokens.ctypes.data_as(ip), _f(logits), choice.ctypes.data_as(ip))
    return tokens[:n].tolist(), logits, choice[:Tp].tolist()
