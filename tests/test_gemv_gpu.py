"""GPU parity of the GEMV family through the C ABI, against the C oracle, the libtorch golden
fixtures, and the shapes/tolerance of the reference's own GEMV unit tests."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as co
from tests.util import assert_close, h16, to_dev

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")

# fp16 output of an fp32-accumulated sum: one rounding (rel 2^-11) plus summation-order noise
GEMV_RTOL = 1e-3
GEMV_ATOL = 2e-3

C2_SHAPES = [(4096, 1024), (4096, 2048), (1024, 1024), (32320, 1024), (29, 512)]


def _ops():
    from pimaicompiler_b200 import ops
    ops.init()
    return ops


def _c2_inputs(N, K, B=1, seed=1):
    g = torch.Generator().manual_seed(seed)
    k = 1.0 / K ** 0.5
    W = h16((torch.rand(N, K, generator=g) * 2 - 1) * k)
    b = h16((torch.rand(N, generator=g) * 2 - 1) * k)
    x = h16(torch.randn(B, K, generator=g))
    return W, b, x


@pytest.mark.parametrize("N,K", C2_SHAPES)
@pytest.mark.parametrize("relu", [False, True])
def test_gemv_mv_baseline_sweep(N, K, relu):
    ops = _ops()
    W, b, x = _c2_inputs(N, K)
    ref = co.linear(W.numpy(), x.numpy(), b.numpy(), relu)[0]
    y = ops.gemv_mv(to_dev(W), to_dev(x[0]), to_dev(b), ops.ACT_RELU if relu else ops.ACT_NONE)
    assert_close(y, ref, GEMV_ATOL, GEMV_RTOL, f"mv {N}x{K}")
    # libtorch CPU live, the library the reference calls
    ref_t = torch.nn.functional.linear(x, W, b)[0]
    if relu:
        ref_t = torch.relu(ref_t)
    assert_close(y, ref_t, GEMV_ATOL, GEMV_RTOL, f"mv {N}x{K} vs libtorch")


@pytest.mark.parametrize("N,K", [(4096, 1024), (1024, 1024), (29, 512), (1280, 320), (32320, 1024)])
def test_gemv_vm_matches_oracle(N, K):
    ops = _ops()
    W, b, x = _c2_inputs(N, K, seed=2)
    A = W.t().contiguous()
    ref = co.vm(x[0].numpy(), A.numpy(), b.numpy(), True)
    y = ops.gemv_vm(to_dev(x[0]), to_dev(A), to_dev(b), ops.ACT_RELU)
    assert_close(y, ref, GEMV_ATOL, GEMV_RTOL, f"vm {K}x{N}")
    # twice in a row: the split-K ticket counters must be left clean
    y2 = ops.gemv_vm(to_dev(x[0]), to_dev(A), None, ops.ACT_NONE)
    assert_close(y2, co.vm(x[0].numpy(), A.numpy()), GEMV_ATOL, GEMV_RTOL, f"vm {K}x{N} second call")


@pytest.mark.parametrize("K,N", [(1024, 4096), (320, 1280)])
def test_reference_unit_test_shapes_and_tolerance(K, N):
    # customGemvTest / pimCustomGemvTest (runtime/unit-tests/custom_op_ut.cpp:20-148): x~U[0,1) fp16,
    # x[1,K]·A[K,N] and A^T[N,K]·x[K,1] vs at::matmul with allclose(rtol=1e-3, atol=1e-5)
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    x = h16(torch.rand(K, generator=g))
    A = h16(torch.rand(K, N, generator=g))
    ref = torch.matmul(x.view(1, K), A).view(-1).to(torch.float16).float()
    y_vm = ops.gemv_vm(to_dev(x), to_dev(A))
    assert_close(y_vm, ref, 1e-5, 1e-3, "xAy")
    y_mv = ops.gemv_mv(to_dev(A.t().contiguous()), to_dev(x))
    assert_close(y_mv, ref, 1e-5, 1e-3, "Axy")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "linear_*.npz"))))
def test_linear_golden(path):
    ops = _ops()
    z = np.load(path)
    W, b, X = (torch.from_numpy(z[k]).cuda() for k in ("W", "b", "X"))
    act = ops.ACT_RELU if int(z["relu"]) else ops.ACT_NONE
    Y = ops.gemm_wx(W, X, b, act)
    assert_close(Y, z["Y"], GEMV_ATOL, GEMV_RTOL, "gemm_wx golden")
    y = ops.gemv_mv(W, X[0].contiguous(), b, act)
    assert_close(y, z["Y"][0], GEMV_ATOL, GEMV_RTOL, "mv golden")
    yv = ops.gemv_vm(X[0].contiguous(), W.t().contiguous(), b, act)
    assert_close(yv, z["Yvm"][0], GEMV_ATOL, GEMV_RTOL, "vm golden")


@pytest.mark.parametrize("N,K", [(1, 1), (1, 7), (29, 7), (5, 240), (3, 1344), (17, 8), (9, 4100)])
def test_gemv_edge_shapes_with_canaries(N, K):
    ops = _ops()
    W, b, x = _c2_inputs(N, K, seed=5)
    ref = co.linear(W.numpy(), x.numpy(), b.numpy())[0]
    buf = torch.full((N + 16,), 77.0, dtype=torch.float16, device="cuda")
    out = buf[8:8 + N]
    ops.gemv_mv(to_dev(W), to_dev(x[0]), to_dev(b), out=out)
    assert_close(out, ref, GEMV_ATOL, GEMV_RTOL, f"mv edge {N}x{K}")
    assert (buf[:8] == 77).all() and (buf[8 + N:] == 77).all(), "mv wrote outside its output"
    buf.fill_(77.0)
    A = W.t().contiguous()
    ops.gemv_vm(to_dev(x[0]), to_dev(A), to_dev(b), out=out)
    assert_close(out, co.vm(x[0].numpy(), A.numpy(), b.numpy()), GEMV_ATOL, GEMV_RTOL, f"vm edge {K}x{N}")
    assert (buf[:8] == 77).all() and (buf[8 + N:] == 77).all(), "vm wrote outside its output"


def test_gemv_unaligned_operands():
    ops = _ops()
    N, K = 33, 96
    W, b, x = _c2_inputs(N, K, seed=6)
    Wd = torch.empty(N * K + 1, dtype=torch.float16, device="cuda")
    Wd[1:] = to_dev(W).view(-1)
    xd = torch.empty(K + 3, dtype=torch.float16, device="cuda")
    xd[3:] = to_dev(x[0])
    y = torch.empty(N, dtype=torch.float16, device="cuda")
    from pimaicompiler_b200 import _lib
    _lib.check(_lib.lib().pimb200_gemv_mv(Wd.data_ptr() + 2, xd.data_ptr() + 6, None, y.data_ptr(), N, K, 0,
                                          torch.cuda.current_stream().cuda_stream), "mv")
    assert_close(y, co.linear(W.numpy(), x.numpy())[0], GEMV_ATOL, GEMV_RTOL, "mv unaligned")


def test_dot_vv_and_bmm_row():
    ops = _ops()
    g = torch.Generator().manual_seed(8)
    a = h16(torch.randn(1024, generator=g))
    b = h16(torch.randn(1024, generator=g))
    y = ops.dot_vv(to_dev(a), to_dev(b))
    assert_close(y, np.array([float((a.double() * b.double()).sum())]), 2e-2, 2e-3, "vv")
    for k in (1, 20, 37, 50):
        x = h16(torch.softmax(torch.randn(k, generator=g), 0))
        A = h16(torch.randn(k, 1024, generator=g))
        yb = ops.bmm_row(to_dev(x), to_dev(A))
        assert_close(yb, co.vm(x.numpy(), A.numpy()), GEMV_ATOL, GEMV_RTOL, f"bmm k={k}")


@pytest.mark.parametrize("B", [8, 32, 128])
@pytest.mark.parametrize("N,K", [(4096, 1024), (4096, 2048), (1024, 1024), (32320, 1024), (29, 512)])
def test_batched_stream_gemm(N, K, B):
    ops = _ops()
    W, b, X = _c2_inputs(N, K, B)
    ref = co.linear(W.numpy(), X.numpy(), b.numpy(), True)
    Y = ops.gemm_wx(to_dev(W), to_dev(X), to_dev(b), ops.ACT_RELU)
    assert_close(Y, ref, GEMV_ATOL, GEMV_RTOL, f"gemm {N}x{K} B={B}")
    Yf = ops.gemm_wx(to_dev(W), to_dev(X), None, ops.ACT_NONE, out_f32=True)
    assert_close(Yf, co.linear(W.numpy(), X.numpy()), 1e-3, 1e-4, f"gemm f32 {N}x{K} B={B}")
    from pimaicompiler_b200 import _lib
    assert _lib.lib().pimb200_gemm_last_status() == 0


@pytest.mark.parametrize("N,K,J", [(16400, 192, 19), (20001, 64, 9), (32320, 1024, 24), (16390, 2048, 17), (4100, 40, 5),
                                   (37, 72, 31), (2049, 264, 12), (16384, 96, 32)])
def test_few_row_gemm_ragged_shapes(N, K, J):
    # the streaming kernels for 1..32 activation rows: ragged row tiles, K tails, row counts between the 8-row tiles,
    # both the K-split form and the warp-per-tile form of the large vocabulary projections
    ops = _ops()
    W, b, X = _c2_inputs(N, K, J, seed=33)
    ref = co.linear(W.numpy(), X.numpy(), b.numpy())
    Yf = ops.gemm_wx(to_dev(W), to_dev(X), to_dev(b), ops.ACT_NONE, out_f32=True)
    assert_close(Yf, ref, 1e-3, 1e-4, f"few-row gemm f32 {N}x{K}x{J}")
    Yh = ops.gemm_wx(to_dev(W), to_dev(X), to_dev(b), ops.ACT_RELU)
    assert_close(Yh, np.maximum(ref, 0), GEMV_ATOL, GEMV_RTOL, f"few-row gemm f16 {N}x{K}x{J}")
    from pimaicompiler_b200 import _lib
    assert _lib.lib().pimb200_gemm_last_status() == 0


@pytest.mark.parametrize("N,K,J", [(4096, 240, 200), (512, 1024, 500), (4096, 2048, 130), (130, 72, 17), (128, 64, 16),
                                   (256, 8, 3), (1280, 320, 29)])
def test_dense_gemm_tensor_core_and_simt_agree_with_oracle(N, K, J):
    # the LSTM input-projection / joint shapes, ragged tiles in every dimension, both kernels
    ops = _ops()
    from pimaicompiler_b200 import _lib
    W, b, X = _c2_inputs(N, K, J, seed=21)
    ref = co.linear(W.numpy(), X.numpy(), b.numpy())
    for simt in (0, 1):
        _lib.lib().pimb200_gemm_force_simt(simt)
        try:
            Yf = ops.gemm_wx(to_dev(W), to_dev(X), to_dev(b), ops.ACT_NONE, out_f32=True)
            assert_close(Yf, ref, 1e-3, 1e-4, f"gemm f32 {N}x{K}x{J} simt={simt}")
            Yh = ops.gemm_wx(to_dev(W), to_dev(X), to_dev(b), ops.ACT_RELU)
            assert_close(Yh, np.maximum(ref, 0), GEMV_ATOL, GEMV_RTOL, f"gemm f16 {N}x{K}x{J} simt={simt}")
        finally:
            _lib.lib().pimb200_gemm_force_simt(0)
    assert _lib.lib().pimb200_gemm_last_status() == 0


def test_gemv_linearity_at_full_size():
    # size-independent property at the largest sweep shape: W(x1 + x2) = Wx1 + Wx2 up to fp16 rounding
    ops = _ops()
    W, b, x = _c2_inputs(32320, 1024, 2, seed=9)
    Wd = to_dev(W)
    y1 = ops.gemv_mv(Wd, to_dev(x[0])).float()
    y2 = ops.gemv_mv(Wd, to_dev(x[1])).float()
    xs = h16(x[0] + x[1])
    # x1+x2 rounded to fp16 differs from the exact sum: feed the rounded sum's exact decomposition
    y12 = ops.gemv_mv(Wd, to_dev(xs)).float()
    resid = h16(xs - x[0])  # exactly representable second operand
    y2b = ops.gemv_mv(Wd, to_dev(resid)).float()
    assert_close(y12, (y1 + y2b).cpu(), 4e-3, 2e-3, "linearity")
    assert y2.shape == y1.shape


def test_grouped_gemm_one_launch_for_independent_products():
    # the branches of a MULTISTREAM node: four expert projections of 26 token rows (one launch), a mix with ragged sizes
    # and a batch-1 product, and a group with a shape outside the few-row kernels (issued one by one by the same call)
    ops = _ops()
    cases = [[(1024, 512, 26)] * 4, [(37, 72, 5), (4096, 1024, 1), (300, 264, 31), (2048, 512, 130), (16, 8, 2)],
             [(512, 256, 8), (4096, 2048, 400), (64, 64, 64)], [(256, 128, 3)] * 11]
    for ci, shapes in enumerate(cases):
        probs, refs = [], []
        for k, (N, K, J) in enumerate(shapes):
            W, b, X = _c2_inputs(N, K, J, seed=100 * ci + k)
            probs.append((to_dev(W), to_dev(X), to_dev(b) if k % 2 == 0 else None))
            refs.append(co.linear(W.numpy(), X.numpy(), b.numpy() if k % 2 == 0 else None, True))
        outs = ops.gemm_wx_grouped(probs, ops.ACT_RELU)
        for k, (Y, ref) in enumerate(zip(outs, refs)):
            assert_close(Y, ref, GEMV_ATOL, GEMV_RTOL, f"grouped case {ci} problem {k} {shapes[k]}")
    from pimaicompiler_b200 import _lib
    assert _lib.lib().pimb200_gemm_last_status() == 0
