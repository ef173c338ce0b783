"""libtorch CPU fp32 backend for the decode models of pimaicompiler_b200.decode_models: the calls the reference's default
executors make (at::linear, at::lstm, at::cat, at::softmax, ...).  Test infrastructure: the oracle side of the C4 / C5
parity tests; the package never imports it."""
from __future__ import annotations

import math

import torch


class CpuBackend:
    """libtorch CPU fp32: the calls the reference's default executors make."""
    dev, dtype = "cpu", torch.float32

    def put(self, t):
        return t.clone()

    def linear(self, x, W, b=None, relu=False):
        y = torch.nn.functional.linear(x, W, b)
        return torch.relu(y) if relu else y

    def lstm_cell_stack(self, key, x, h, c, params, layers):
        y, hn, cn = torch.lstm(x.view(1, 1, -1), [h, c], params, True, layers, 0.0, False, False, False)
        return y.view(-1), hn, cn

    def add(self, a, b):
        return a + b

    def bmm_row(self, x, A):
        return x @ A

    def cat(self, ts, dim):
        return torch.cat(ts, dim)

    def kv_new(self, steps, d):
        return torch.zeros(0, d)

    def kv_append(self, cache, t, row):
        # the reference's form: the cache grows by an at::cat per step
        return torch.cat([cache, row.view(1, -1)], 0) if cache.shape[0] else row.view(1, -1).clone()

    def attend(self, q, K, Vv, heads):
        # per-head scaled dot-product attention of one query over K / V [t, d]: matmul -> softmax -> matmul
        d = q.numel()
        hd = d // heads
        qh = q.view(heads, 1, hd)
        Kh = K.view(-1, heads, hd).transpose(0, 1)
        Vh = Vv.view(-1, heads, hd).transpose(0, 1)
        return (torch.softmax(qh @ Kh.transpose(1, 2) / math.sqrt(hd), -1) @ Vh).reshape(d)

    def tanh(self, x):
        return torch.tanh(x)

    def softmax(self, x):
        return torch.softmax(x, -1)

    def layer_norm(self, x):
        return torch.nn.functional.layer_norm(x, (x.shape[-1],))

    def argmax(self, x):
        return int(torch.argmax(x))
