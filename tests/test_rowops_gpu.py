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


@pytest.mark.parametrize("n,heads,hd,S", [(5, 8, 64, 64), (3, 4, 16, 9), (33, 2, 40, 70), (6, 4, 128, 100), (4, 8, 64, 128),
                                         (130, 8, 64, 37)])
def test_attention_rows_batched_matches_oracle(n, heads, hd, S):
    # lock-step decode of n sequences: one cache and one length per sequence (cross-attention over ragged sources), and a
    # shared device-side position (self-attention at step t)
    ops = _ops()
    g = torch.Generator().manual_seed(n * 100 + S)
    d = heads * hd
    q = torch.randn(n, d, generator=g).to(torch.float16)
    K = torch.randn(n, S, d, generator=g).to(torch.float16)
    V = torch.randn(n, S, d, generator=g).to(torch.float16)
    lens = torch.randint(0, S + 1, (n,), generator=g)
    lens[0] = S
    got = ops.attention_rows(q.cuda(), K.cuda(), V.cuda(), heads, len_dev=lens.cuda(), len_inc=1).float().cpu().numpy()
    for j in range(n):
        ref = co.attention_row(q[j].float().numpy(), K[j].float().numpy(), V[j].float().numpy(), heads, int(lens[j]))
        np.testing.assert_allclose(got[j], ref, rtol=RTOL, atol=2e-3)
    pos = torch.tensor([S // 2], dtype=torch.int64, device="cuda")
    got2 = ops.attention_rows(q.cuda(), K.cuda(), V.cuda(), heads, len_dev=pos, len_inc=0, len_add=1).float().cpu().numpy()
    for j in range(n):
        ref = co.attention_row(q[j].float().numpy(), K[j].float().numpy(), V[j].float().numpy(), heads, S // 2 + 1)
        np.testing.assert_allclose(got2[j], ref, rtol=RTOL, atol=2e-3)


@pytest.mark.parametrize("n,S,H", [(7, 50, 1024), (3, 9, 64), (4, 11, 70), (130, 5, 16)])
def test_additive_attention_matches_libtorch(n, S, H):
    # normalised Bahdanau attention for n sentences of ragged length over a time-major [S, n, H] encoder output, the
    # context written into the second half of a [n, 2H] buffer
    ops = _ops()
    g = torch.Generator().manual_seed(n + S + H)
    q = torch.randn(n, H, generator=g).half()
    kp = torch.randn(S, n, H, generator=g).half()
    vals = torch.tanh(torch.randn(S, n, H, generator=g)).half()
    v = (torch.randn(H, generator=g) / H ** 0.5).half()
    b = (torch.randn(H, generator=g) * 0.1).half()
    lens = torch.randint(1, S + 1, (n,), generator=g)
    lens[0] = S
    buf = torch.zeros(n, 2 * H, dtype=torch.float16, device="cuda")
    ops.additive_attention(q.cuda(), kp.cuda(), vals.cuda(), lens.cuda(), v.cuda(), b.cuda(), out=buf[:, H:])
    got = buf[:, H:].float().cpu()
    assert float(buf[:, :H].abs().max()) == 0.0
    for j in range(n):
        L = int(lens[j])
        e = torch.tanh(kp[:L, j].float() + q[j].float() + b.float()) @ v.float()
        ref = torch.softmax(e, 0) @ vals[:L, j].float()
        np.testing.assert_allclose(got[j].numpy(), ref.numpy(), rtol=2e-3, atol=2e-3)
    # no bias, full lengths
    out = ops.additive_attention(q.cuda(), kp.cuda(), vals.cuda(), None, v.cuda(), None).float().cpu()
    e = torch.einsum("snh,h->sn", torch.tanh(kp.float() + q.float().unsqueeze(0)), v.float())
    ref = torch.einsum("sn,snh->nh", torch.softmax(e, 0), vals.float())
    np.testing.assert_allclose(out.numpy(), ref.numpy(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("rows,cols,k", [(1, 32320, 4), (3, 29, 5), (5, 512, 1), (2, 4100, 8), (4, 37, 37)])
def test_topk_rows_match_oracle(rows, cols, k):
    # values bit-exact; indices equal to the oracle's (equal values: lower index first), largest and smallest
    ops = _ops()
    g = torch.Generator().manual_seed(rows * 1000 + cols + k)
    x = (torch.randn(rows, cols, generator=g) * 3).to(torch.float16)
    x[0, cols // 2] = x[0, 0]                       # a tie
    for largest in (True, False):
        rv, ri = co.topk(x.float().numpy(), k, largest)
        v, i = ops.topk(x.cuda(), k, largest)
        assert np.array_equal(v.float().cpu().numpy(), rv)
        assert np.array_equal(i.cpu().numpy(), ri)
        tv, _ = torch.topk(x.float(), k, largest=largest)
        assert np.array_equal(rv, tv.numpy())       # the oracle itself against libtorch
