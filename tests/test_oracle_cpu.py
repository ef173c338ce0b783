"""CPU: the C oracle (oracle/oracle.c) against the libtorch-generated golden fixtures and against
libtorch CPU live, and the shapes of the reference's own GEMV unit tests."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as co
from tests.util import h16

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, name))


def _params(z):
    ps, i = [], 0
    while f"p{i}" in z:
        ps.append(z[f"p{i}"].astype(np.float32))
        i += 1
    return ps


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "lstm_*.npz"))))
def test_oracle_lstm_matches_libtorch_golden(path):
    z = np.load(path)
    T, B, I, H, L, bi, hb, bf = [int(v) for v in z["cfg"]]
    ps = _params(z)
    if "batch_sizes" in z:
        y, hn, cn = co.lstm_packed(z["data"].astype(np.float32), z["batch_sizes"], ps, L, bool(bi), bool(hb),
                                   z["h0"].astype(np.float32), z["c0"].astype(np.float32))
    else:
        y, hn, cn = co.lstm(z["x"].astype(np.float32), ps, L, bool(bi), bool(hb), z["h0"].astype(np.float32),
                            z["c0"].astype(np.float32), bool(bf))
    # fp32 vs fp32: only summation order differs
    np.testing.assert_allclose(y, z["y"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(hn, z["hn"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(cn, z["cn"], atol=4e-6, rtol=1e-5)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "linear_*.npz"))))
def test_oracle_linear_matches_libtorch_golden(path):
    z = np.load(path)
    W, b, X = (z[k].astype(np.float32) for k in ("W", "b", "X"))
    relu = bool(z["relu"])
    np.testing.assert_allclose(co.linear(W, X, b, relu), z["Y"], atol=1e-5, rtol=1e-5)
    A = np.ascontiguousarray(W.T)
    np.testing.assert_allclose(co.vm(X[0], A, b, relu), z["Yvm"][0], atol=1e-5, rtol=1e-5)


def test_oracle_glue_matches_golden():
    z = _load("glue.npz")
    A, B, Br = (z[k].astype(np.float32) for k in ("A", "B", "Br"))
    # fp16 add rounds once: fp32 sum rounded to fp16 must equal the fp16 result bit for bit
    assert np.array_equal(co.add(A, B).astype(np.float16), z["add_sym"])
    assert np.array_equal(co.add(A, Br).astype(np.float16), z["add_bcast"])
    assert np.array_equal(co.cat([z["cat0"], z["cat1"], z["cat2"]], 1), z["cat_out"])


def test_oracle_cat_split_roundtrip():
    # the reference's atenCatOpTest: split a tensor, cat it back, expect equality (aten_ops_ut.cpp:30-41)
    t = torch.rand(2, 6, 5).to(torch.float16)
    parts = [p.contiguous().numpy() for p in torch.split(t, 2, dim=1)]
    assert np.array_equal(co.cat(parts, 1), t.numpy())
    parts0 = [p.contiguous().numpy() for p in torch.split(t, 1, dim=0)]
    assert np.array_equal(co.cat(parts0, 0), t.numpy())


@pytest.mark.parametrize("K,N", [(1024, 4096), (320, 1280)])
def test_oracle_reference_gemv_shapes(K, N):
    # customGemvTest / pimCustomGemvTest shapes and input distribution (U[0,1) fp16), both operand
    # orders, vs at::matmul (custom_op_ut.cpp:20-148)
    g = torch.Generator().manual_seed(7)
    x = h16(torch.rand(K, generator=g))
    A = h16(torch.rand(K, N, generator=g))
    ref = torch.matmul(x.view(1, 1, 1, K), A).view(-1).numpy()
    np.testing.assert_allclose(co.vm(x.numpy(), A.numpy()), ref, rtol=1e-5, atol=1e-3)
    W = A.t().contiguous()
    ref2 = torch.matmul(W, x.view(1, 1, K, 1)).view(-1).numpy()
    np.testing.assert_allclose(co.linear(W.numpy(), x.numpy()[None, :]).reshape(-1), ref2, rtol=1e-5, atol=1e-3)


def test_oracle_fp16_emulation_rounds_hidden_state():
    g = torch.Generator().manual_seed(3)
    from tests.util import lstm_params
    ps = [p.numpy() for p in lstm_params(1, 1, 8, 8, g)]
    x = h16(torch.randn(6, 1, 8, generator=g)).numpy()
    y, hn, cn = co.lstm(x, ps, 1, False, emulate_fp16=True)
    assert np.array_equal(y, y.astype(np.float16).astype(np.float32))
    y32, _, _ = co.lstm(x, ps, 1, False)
    assert np.abs(y - y32).max() < 2e-3


def test_oracle_rowops_match_libtorch_golden():
    # softmax / log_softmax / argmax / tanh / layer_norm / masked_fill over the last dimension against libtorch CPU
    z = _load("rowops.npz")
    for name in ("logits", "scores", "model", "vocab"):
        x = z[f"{name}_x"].astype(np.float32)
        np.testing.assert_allclose(co.softmax(x), z[f"{name}_softmax"], atol=1e-6, rtol=1e-5)
        np.testing.assert_allclose(co.softmax(x, log=True), z[f"{name}_log_softmax"], atol=2e-6, rtol=1e-5)
        assert np.array_equal(co.argmax(x), z[f"{name}_argmax"])
        np.testing.assert_allclose(co.tanh(x), z[f"{name}_tanh"], atol=1e-6, rtol=1e-6)
    x, gamma, beta = (z[k].astype(np.float32) for k in ("ln_x", "ln_gamma", "ln_beta"))
    np.testing.assert_allclose(co.layer_norm(x, gamma, beta, 1e-5), z["ln_y"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(co.layer_norm(x, None, None, 1e-6), z["ln_y_plain"], atol=2e-6, rtol=1e-5)
    mx = z["mf_x"].astype(np.float32)
    assert np.array_equal(co.masked_fill(mx, z["mf_mask"], -65504.0), z["mf_y"])
    assert np.array_equal(co.masked_fill(mx, z["mf_row_mask"], 0.25), z["mf_y_row"])


@pytest.mark.parametrize("heads,hd,S,L", [(8, 64, 40, 40), (4, 16, 9, 5), (1, 32, 3, 1)])
def test_oracle_attention_row_matches_libtorch(heads, hd, S, L):
    g = torch.Generator().manual_seed(heads * 100 + S)
    d = heads * hd
    q, K, V = (torch.randn(*s, generator=g) for s in ((d,), (S, d), (S, d)))
    qh = q.view(heads, 1, hd)
    Kh = K[:L].view(L, heads, hd).transpose(0, 1)
    Vh = V[:L].view(L, heads, hd).transpose(0, 1)
    ref = (torch.softmax(qh @ Kh.transpose(1, 2) / hd ** 0.5, -1) @ Vh).reshape(d)
    np.testing.assert_allclose(co.attention_row(q.numpy(), K.numpy(), V.numpy(), heads, L), ref.numpy(), atol=2e-6, rtol=1e-5)
