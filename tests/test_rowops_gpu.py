"""GPU parity of the row-wise glue ops of the decode path (softmax, log_softmax, argmax, layer_norm, tanh,
masked_fill) through the C ABI: against the libtorch fixtures and against the C oracle on seeded inputs.

Tolerances: outputs are fp16, computed in fp32 from fp16 inputs.  A correctly rounded fp16 result differs from the
fp32 oracle by at most half an fp16 ulp (relative 2^-11 = 4.9e-4); softmax / tanh / layer_norm allow that plus 1e-3
absolute for values near zero.  argmax and masked_fill are exact.
"""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as co

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
RTOL, ATOL = 1e-3, 1e-3


def _ops():
    from pimaicompiler_b200 import ops
    return ops


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_rowops_golden():
    ops = _ops()
    z = np.load(os.path.join(GOLD, "rowops.npz"))
    for name in ("logits", "scores", "model", "vocab"):
        x = _dev(z[f"{name}_x"])
        np.testing.assert_allclose(ops.softmax(x).float().cpu().numpy(), z[f"{name}_softmax"], rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(ops.softmax(x, log=True).float().cpu().numpy(), z[f"{name}_log_softmax"],
                                   rtol=RTOL, atol=4e-3)   # values up to ~10: half an fp16 ulp is 4e-3 there
        assert np.array_equal(ops.argmax(x).cpu().numpy(), z[f"{name}_argmax"])
        np.testing.assert_allclose(ops.tanh(x).float().cpu().numpy(), z[f"{name}_tanh"], rtol=RTOL, atol=ATOL)
    x, gamma, beta = (_dev(z[k]) for k in ("ln_x", "ln_gamma", "ln_beta"))
    np.testing.assert_allclose(ops.layer_norm(x, gamma, beta, 1e-5).float().cpu().numpy(), z["ln_y"], rtol=RTOL,
                               atol=2e-3)
    np.testing.assert_allclose(ops.layer_norm(x, None, None, 1e-6).float().cpu().numpy(), z["ln_y_plain"], rtol=RTOL,
                               atol=2e-3)
    mx = _dev(z["mf_x"])
    assert np.array_equal(ops.masked_fill(mx, _dev(z["mf_mask"]), -65504.0).float().cpu().numpy(), z["mf_y"])
    assert np.array_equal(ops.masked_fill(mx, _dev(z["mf_row_mask"]), 0.25).float().cpu().numpy(), z["mf_y_row"])


@pytest.mark.parametrize("rows,cols", [(1, 29), (1, 32320), (7, 13), (3, 1), (64, 512), (2, 4097), (257, 8), (1, 5000)])
def test_softmax_argmax_match_oracle(rows, cols):
    # logit rows of the RNN-T / GNMT vocabularies, attention-score rows, odd and unaligned lengths
    ops = _ops()
    g = torch.Generator().manual_seed(rows * 131 + cols)
    x = (torch.randn(rows, cols, generator=g) * 4.0).to(torch.float16)
    xf = x.float().numpy()
    y = ops.softmax(x.cuda()).float().cpu().numpy()
    np.testing.assert_allclose(y, co.softmax(xf), rtol=RTOL, atol=1e-4)
    np.testing.assert_allclose(y.sum(-1), 1.0, atol=2e-3)   # rows sum to one up to the fp16 rounding of each entry
    yl = ops.softmax(x.cuda(), log=True).float().cpu().numpy()
    np.testing.assert_allclose(yl, co.softmax(xf, log=True), rtol=RTOL, atol=8e-3)
    assert np.array_equal(ops.argmax(x.cuda()).cpu().numpy(), co.argmax(xf))


def test_argmax_ties_take_the_lowest_index():
    ops = _ops()
    x = torch.zeros(4, 1000, dtype=torch.float16)
    x[0, [17, 400, 999]] = 3.0
    x[1, [999]] = 1.0
    x[2, :] = -2.0            # all equal: index 0
    x[3, [5, 6]] = 65504.0    # largest finite fp16
    assert ops.argmax(x.cuda()).cpu().tolist() == [17, 999, 0, 5]


@pytest.mark.parametrize("rows,cols", [(1, 512), (11, 512), (3, 1024), (5, 37), (2, 2048)])
def test_layer_norm_matches_oracle(rows, cols):
    ops = _ops()
    g = torch.Generator().manual_seed(rows * 17 + cols)
    x = (torch.randn(rows, cols, generator=g) * 1.5 + 0.3).to(torch.float16)
    gamma = (torch.rand(cols, generator=g) + 0.5).to(torch.float16)
    beta = (torch.randn(cols, generator=g) * 0.2).to(torch.float16)
    ref = co.layer_norm(x.float().numpy(), gamma.float().numpy(), beta.float().numpy(), 1e-5)
    got = ops.layer_norm(x.cuda(), gamma.cuda(), beta.cuda(), 1e-5).float().cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=RTOL, atol=3e-3)
    # normalised rows have zero mean and unit variance before the affine step
    plain = ops.layer_norm(x.cuda(), None, None, 1e-5).float().cpu().numpy()
    np.testing.assert_allclose(plain.mean(-1), 0.0, atol=2e-3)
    if cols >= 512:
        np.testing.assert_allclose(plain.var(-1), 1.0, atol=5e-3)


@pytest.mark.parametrize("shape", [(1, 1024), (8, 1, 13), (3, 5, 7), (100003,)])
def test_tanh_and_masked_fill_match_oracle(shape):
    ops = _ops()
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * 2.0).to(torch.float16)
    np.testing.assert_allclose(ops.tanh(x.cuda()).float().cpu().numpy(), co.tanh(x.float().numpy()), rtol=RTOL,
                               atol=ATOL)
    mask = torch.rand(*shape, generator=g) < 0.4
    ref = co.masked_fill(x.float().numpy(), mask.numpy(), -1e4)
    assert np.array_equal(ops.masked_fill(x.cuda(), mask.cuda(), -1e4).float().cpu().numpy(),
                          ref.astype(np.float16).astype(np.float32))
    if len(shape) > 1:
        row = torch.rand(shape[-1], generator=g) < 0.5
        ref = co.masked_fill(x.float().numpy(), row.numpy(), 0.5)
        assert np.array_equal(ops.masked_fill(x.cuda(), row.cuda(), 0.5).float().cpu().numpy(), ref)


def test_rowops_empty_and_bad_arguments():
    ops = _ops()
    from pimaicompiler_b200 import _lib
    e = torch.empty(0, 16, dtype=torch.float16, device="cuda")
    assert ops.softmax(e).shape == (0, 16)
    assert ops.argmax(e).shape == (0,)
    assert ops.tanh(e).numel() == 0
    lib = _lib.lib()
    x = torch.zeros(4, 8, dtype=torch.float16, device="cuda")
    assert lib.pimb200_softmax_rows(None, x.data_ptr(), 4, 8, 0, None) == _lib.ERR_BAD_ARG
    assert lib.pimb200_argmax_rows(x.data_ptr(), None, 4, 8, None) == _lib.ERR_BAD_ARG
    m = torch.zeros(5, dtype=torch.bool, device="cuda")
    assert lib.pimb200_masked_fill_f16(x.data_ptr(), m.data_ptr(), 0.0, x.data_ptr(), 32, 5, None) == _lib.ERR_BAD_ARG


@pytest.mark.parametrize("heads,hd,S,L", [(8, 64, 64, 64), (8, 64, 64, 1), (4, 16, 9, 5), (2, 40, 300, 257), (1, 8, 3, 0)])
def test_attention_row_matches_oracle(heads, hd, S, L):
    # decode-step attention over a key / value cache, host-side and device-side length
    ops = _ops()
    g = torch.Generator().manual_seed(heads * 1000 + S + L)
    d = heads * hd
    q = torch.randn(d, generator=g).to(torch.float16)
    K = torch.randn(S, d, generator=g).to(torch.float16)
    V = torch.randn(S, d, generator=g).to(torch.float16)
    ref = co.attention_row(q.float().numpy(), K.float().numpy(), V.float().numpy(), heads, L)
    got = ops.attention_row(q.cuda(), K.cuda(), V.cuda(), heads, length=L).float().cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=RTOL, atol=2e-3)
    pos = torch.tensor([L - 1], dtype=torch.int64, device="cuda")     # entries 0..pos are valid
    got_dev = ops.attention_row(q.cuda(), K.cuda(), V.cuda(), heads, length_dev=pos, length_add=1).float().cpu().numpy()
    assert np.array_equal(got_dev, got)
