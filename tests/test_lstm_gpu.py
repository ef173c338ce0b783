"""GPU parity of the fused LSTM through the C ABI: both recurrence variants against the C oracle,
the libtorch golden fixtures, and libtorch CPU at the baseline's C1 shape."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as co
from tests.util import CONTRACT_ATOL, CONTRACT_RTOL, assert_close, h16, lstm_params, to_dev

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")

# vs the fp32 oracle: h is rounded to fp16 every step (rel 2^-11 of values in (-1,1)) and the
# rounding feeds back through the recurrence; the contract bound is 2e-2 / 1e-2
LSTM_ATOL = 4e-3
LSTM_RTOL = 4e-3


def _ops():
    from pimaicompiler_b200 import ops
    return ops


def _run(ops, ps, x, h0, c0, L, bi, hb, bf, variant, bulk_wide=None):
    T = x.shape[1] if bf else x.shape[0]
    I, H = x.shape[2], ps[1].shape[1]
    m = ops.Lstm([to_dev(p) for p in ps], L, bi, I, H, hb)
    m.set_variant(variant)
    if bulk_wide is not None:   # None = the library's default choice of persistent kernel by batch size
        from pimaicompiler_b200 import _lib
        assert _lib.lib().pimb200_lstm_set_bulk_wide(m._h, bulk_wide) == 0
    y, hn, cn = m.forward(to_dev(x), None if h0 is None else to_dev(h0), None if c0 is None else to_dev(c0), bf)
    torch.cuda.synchronize()
    assert m.last_status() == 0
    return y, hn, cn


@pytest.mark.parametrize("path", sorted(p for p in glob.glob(os.path.join(GOLD, "lstm_*.npz")) if "packed" not in p))
def test_lstm_golden_streamed(path):
    ops = _ops()
    z = np.load(path)
    T, B, I, H, L, bi, hb, bf = [int(v) for v in z["cfg"]]
    ps, i = [], 0
    while f"p{i}" in z:
        ps.append(torch.from_numpy(z[f"p{i}"]).float())
        i += 1
    y, hn, cn = _run(ops, ps, torch.from_numpy(z["x"]).float(), torch.from_numpy(z["h0"]).float(),
                     torch.from_numpy(z["c0"]).float(), L, bool(bi), bool(hb), bool(bf), ops.LSTM_STREAMED)
    assert_close(y, z["y"], LSTM_ATOL, LSTM_RTOL, "y")
    assert_close(hn, z["hn"], LSTM_ATOL, LSTM_RTOL, "hn")
    assert_close(cn, z["cn"], LSTM_ATOL, LSTM_RTOL, "cn")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "lstm_packed_*.npz"))))
def test_lstm_golden_packed(path):
    ops = _ops()
    z = np.load(path)
    T, B, I, H, L, bi, hb, bf = [int(v) for v in z["cfg"]]
    ps, i = [], 0
    while f"p{i}" in z:
        ps.append(torch.from_numpy(z[f"p{i}"]).cuda())
        i += 1
    m = ops.Lstm(ps, L, bool(bi), I, H, True)
    y, hn, cn = m.forward_packed(torch.from_numpy(z["data"]).cuda(), torch.from_numpy(z["batch_sizes"]),
                                 torch.from_numpy(z["h0"]).cuda(), torch.from_numpy(z["c0"]).cuda())
    assert_close(y, z["y"], LSTM_ATOL, LSTM_RTOL, "packed y")
    assert_close(hn, z["hn"], LSTM_ATOL, LSTM_RTOL, "packed hn")
    assert_close(cn, z["cn"], LSTM_ATOL, LSTM_RTOL, "packed cn")


# (T, B, I, H, L, bidirectional, has_biases, batch_first, nonzero state)
CASES = [
    (1, 1, 8, 16, 1, False, True, False, True),
    (2, 1, 16, 48, 2, False, True, False, False),
    (3, 1, 8, 24, 1, False, True, False, True),
    (20, 1, 240, 128, 2, False, True, False, True),
    (16, 1, 64, 320, 2, False, True, False, True),      # prediction-net width
    (12, 1, 40, 1024, 1, False, True, False, True),
    (9, 1, 32, 64, 3, True, True, False, True),
    (10, 1, 32, 64, 2, False, False, True, False),
    (7, 5, 24, 48, 2, True, True, True, True),           # B > 1, bidirectional, batch_first
    (11, 8, 40, 128, 2, False, True, False, True),       # a full tile of sequences
    (6, 8, 240, 1024, 1, False, True, True, False),      # eight utterances at the encoder width
    (5, 11, 16, 32, 1, False, True, False, True),        # two tiles of sequences, the second ragged
    (9, 32, 64, 256, 2, False, True, True, True),        # four full tiles, batch_first
    (4, 19, 24, 1024, 1, True, True, False, True),       # ragged third tile, bidirectional, encoder width
    (3, 40, 16, 32, 1, False, True, False, True),        # eight tiles, the last ones ragged
    (5, 64, 240, 1024, 1, False, True, True, False),     # 64 utterances at the encoder width, batch_first
    (4, 57, 32, 128, 2, True, True, False, True),        # ragged eighth tile, bidirectional, two layers
    (2, 70, 16, 32, 1, False, True, False, True),        # 65..128 sequences: two batch halves, the second ragged
    (4, 128, 32, 1024, 1, False, True, True, False),     # the largest lock-step batch at the encoder width, batch_first
    (3, 97, 24, 256, 2, True, True, False, True),        # ragged second half, bidirectional, two layers
    (5, 33, 16, 1024, 1, False, True, False, True),      # smallest batch the pipelined kernel takes by default
    (3, 2, 7, 5, 2, False, True, False, True),           # odd sizes: scalar path
    (1, 8, 16, 32, 1, False, True, False, True),         # decode form, 8+ sequences: products as GEMMs + gate kernel
    (1, 33, 64, 128, 2, False, True, False, True),       # ... two layers, ragged row tiles
    (1, 128, 2048, 1024, 1, False, True, True, True),    # ... a GNMT decoder layer for 128 sentences
    (1, 20, 24, 48, 2, True, False, False, False),       # ... bidirectional, no biases, zero state
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("variant", ["streamed", "persistent", "pipe", "wide", "ksplit", "tagged"])
def test_lstm_matches_oracle(case, variant):
    ops = _ops()
    T, B, I, H, L, bi, hb, bf, nz = case
    if variant in ("persistent", "pipe") and (B > 128 or H % 16):
        pytest.skip("the persistent kernels take up to 128 sequences and H % 16 == 0")
    if variant == "wide" and (B > 64 or H % 16):
        pytest.skip("the exchange-on-compute-warps kernel takes up to 64 sequences and H % 16 == 0")
    if variant == "ksplit" and (B < 2 or B > 32 or H % 16):
        pytest.skip("the K-split batched kernel takes 2..32 sequences and H % 16 == 0")
    if variant == "tagged" and (B > 8 or H % 16):
        pytest.skip("tagged-word exchange takes up to 8 sequences and H % 16 == 0")
    D = 2 if bi else 1
    g = torch.Generator().manual_seed(T * 131 + H)
    ps = lstm_params(L, D, I, H, g, has_biases=hb)
    x = h16(torch.randn((B, T, I) if bf else (T, B, I), generator=g))
    h0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5) if nz else None
    c0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5) if nz else None
    ref = co.lstm(x.numpy(), [p.numpy() for p in ps], L, bi, hb, None if h0 is None else h0.numpy(),
                  None if c0 is None else c0.numpy(), bf)
    vid = {"streamed": ops.LSTM_STREAMED, "persistent": ops.LSTM_PERSISTENT, "pipe": ops.LSTM_PERSISTENT,
           "wide": ops.LSTM_PERSISTENT, "ksplit": ops.LSTM_PERSISTENT, "tagged": ops.LSTM_PERSISTENT_TAGGED}[variant]
    got = _run(ops, ps, x, h0, c0, L, bi, hb, bf, vid, bulk_wide={"ksplit": 0, "wide": 1, "pipe": 3}.get(variant))
    for name, a, b in zip(("y", "hn", "cn"), got, ref):
        assert_close(a, b, LSTM_ATOL, LSTM_RTOL, f"{variant} {name} {case}")


@pytest.mark.parametrize("variant", ["streamed", "persistent"])
def test_lstm_baseline_c1_vs_libtorch(variant):
    # C1: 2 layers, input 240, hidden 1024, T=200, B=1; x~N(0,1); params~U(-1/32,1/32); h0=c0=0; seed 0
    ops = _ops()
    torch.manual_seed(0)
    T, I, H, L = 200, 240, 1024, 2
    x = h16(torch.randn(T, 1, I))
    ps = []
    for l in range(L):
        Il = I if l == 0 else H
        ps += [h16((torch.rand(4 * H, Il) * 2 - 1) / 32), h16((torch.rand(4 * H, H) * 2 - 1) / 32),
               h16((torch.rand(4 * H) * 2 - 1) / 32), h16((torch.rand(4 * H) * 2 - 1) / 32)]
    z = torch.zeros(L, 1, H)
    y_ref, hn_ref, cn_ref = torch.lstm(x, [z, z], ps, True, L, 0.0, False, False, False)
    y, hn, cn = _run(ops, ps, x, None, None, L, False, True, False,
                     ops.LSTM_STREAMED if variant == "streamed" else ops.LSTM_PERSISTENT)
    assert_close(y, y_ref, CONTRACT_ATOL, CONTRACT_RTOL, "C1 y (contract)")
    e = assert_close(y, y_ref, LSTM_ATOL, LSTM_RTOL, "C1 y")
    assert_close(hn, hn_ref, LSTM_ATOL, LSTM_RTOL, "C1 hn")
    assert_close(cn, cn_ref, 2 * LSTM_ATOL, LSTM_RTOL, "C1 cn")
    print(f"C1 {variant}: max abs err {e:.2e}")


def test_lstm_variants_agree_and_repeat():
    # same handle, three calls in a row: step tags of the persistent exchange must not collide
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    T, I, H, L = 33, 64, 256, 2
    ps = lstm_params(L, 1, I, H, g)
    x = h16(torch.randn(T, 1, I, generator=g))
    m = ops.Lstm([to_dev(p) for p in ps], L, False, I, H, True)
    m.set_variant(ops.LSTM_STREAMED)
    ys, hs, cs = m.forward(to_dev(x))
    m.set_variant(ops.LSTM_PERSISTENT)
    for _ in range(3):
        yp, hp, cp = m.forward(to_dev(x))
        torch.cuda.synchronize()
        assert m.last_status() == 0
        assert_close(yp, ys, 1e-3, 1e-3, "persistent vs streamed")
        assert_close(cp, cs, 2e-3, 1e-3, "persistent vs streamed cn")


def test_lstm_outputs_alias_slices_of_caller_buffers():
    # GNMT-style in-place "custom cat": y goes into the first half of a {1,1,2048} buffer, (h,c) into
    # slots of an {8,1,1024} state buffer (miopen_ops_executor.cpp:193-228)
    ops = _ops()
    g = torch.Generator().manual_seed(6)
    I = H = 1024
    ps = lstm_params(1, 1, I, H, g)
    x = h16(torch.randn(1, 1, I, generator=g))
    h0 = h16(torch.randn(1, 1, H, generator=g) * 0.5)
    c0 = h16(torch.randn(1, 1, H, generator=g) * 0.5)
    ref = co.lstm(x.numpy(), [p.numpy() for p in ps], 1, False, True, h0.numpy(), c0.numpy())
    cat_buf = torch.full((1, 1, 2048), 5.0, dtype=torch.float16, device="cuda")
    state_buf = torch.full((8, 1, 1024), 5.0, dtype=torch.float16, device="cuda")
    m = ops.Lstm([to_dev(p) for p in ps], 1, False, I, H, True)
    m.forward(to_dev(x), to_dev(h0), to_dev(c0), out=(cat_buf[..., :1024], state_buf[2:3], state_buf[3:4]))
    torch.cuda.synchronize()
    assert_close(cat_buf[..., :1024], ref[0], LSTM_ATOL, LSTM_RTOL, "aliased y")
    assert_close(state_buf[2:3], ref[1], LSTM_ATOL, LSTM_RTOL, "aliased hn")
    assert_close(state_buf[3:4], ref[2], LSTM_ATOL, LSTM_RTOL, "aliased cn")
    assert (cat_buf[..., 1024:] == 5).all() and (state_buf[:2] == 5).all() and (state_buf[4:] == 5).all()


@pytest.mark.parametrize("B,L", [(1, 1), (4, 1), (40, 1), (2, 2)])
def test_persistent_bounded_wait_reports_timeout_and_context_survives(B, L):
    # Fault handling without faulting anything: shrink the bounded wait to a single poll, so the hidden-state exchange
    # cannot complete in time; the kernel must give up, record ERR_TIMEOUT and return, and the next call (normal
    # limit) must still be correct.  L = 2 with two sequences is the layer-wavefront kernel.
    ops = _ops()
    from pimaicompiler_b200 import _lib
    g = torch.Generator().manual_seed(17)
    T, I, H = 64, 32, 256
    ps = lstm_params(L, 1, I, H, g)
    x = h16(torch.randn(T, B, I, generator=g))
    m = ops.Lstm([to_dev(p) for p in ps], L, False, I, H, True)
    m.set_variant(ops.LSTM_PERSISTENT)
    lib = _lib.lib()
    assert lib.pimb200_lstm_set_poll_limit(m._h, 1) == 0
    m.forward(to_dev(x))
    torch.cuda.synchronize()                      # returns: nothing hangs
    assert m.last_status() == _lib.ERR_TIMEOUT
    assert m.last_status() == 0                   # reading clears it
    assert lib.pimb200_lstm_set_poll_limit(m._h, 1 << 21) == 0
    y, hn, cn = m.forward(to_dev(x))
    torch.cuda.synchronize()
    assert m.last_status() == 0
    ref = co.lstm(x.numpy(), [p.numpy() for p in ps], L, False)
    assert_close(y, ref[0], LSTM_ATOL, LSTM_RTOL, "after a timed-out launch")
    # a timed-out launch must not poison the launches behind it: nobody reads (and thereby clears) the status between
    # the two calls here, the second call must be correct all the same, and the time-out is still reported afterwards
    assert lib.pimb200_lstm_set_poll_limit(m._h, 1) == 0
    m.forward(to_dev(x))
    assert lib.pimb200_lstm_set_poll_limit(m._h, 1 << 21) == 0
    y2, _, _ = m.forward(to_dev(x))
    torch.cuda.synchronize()
    assert_close(y2, ref[0], LSTM_ATOL, LSTM_RTOL, "directly behind a timed-out launch, status unread")
    assert m.last_status() == _lib.ERR_TIMEOUT


@pytest.mark.parametrize("T,B,I,H", [(6, 64, 64, 1024), (9, 23, 32, 256), (5, 40, 16, 128)])
def test_tcgen05_recurrence_variant_matches_oracle(T, B, I, H):
    # the opt-in tensor-memory variant of the batched recurrence must give the same results as the default kernels
    ops = _ops()
    from pimaicompiler_b200 import _lib
    g = torch.Generator().manual_seed(B * 7 + H)
    ps = lstm_params(1, 1, I, H, g)
    x = h16(torch.randn(T, B, I, generator=g))
    h0 = h16(torch.randn(1, B, H, generator=g) * 0.5)
    c0 = h16(torch.randn(1, B, H, generator=g) * 0.5)
    ref = co.lstm(x.numpy(), [p.numpy() for p in ps], 1, False, True, h0.numpy(), c0.numpy())
    m = ops.Lstm([to_dev(p) for p in ps], 1, False, I, H, True)
    m.set_variant(ops.LSTM_PERSISTENT)
    assert _lib.lib().pimb200_lstm_set_use_tc(m._h, 1) == 0
    got = m.forward(to_dev(x), to_dev(h0), to_dev(c0))
    torch.cuda.synchronize()
    assert m.last_status() == 0
    for name, a, b in zip(("y", "hn", "cn"), got, ref):
        assert_close(a, b, LSTM_ATOL, LSTM_RTOL, f"tcgen05 recurrence {name}")


def test_lstm_benchmark_shape_batched_properties():
    # the benchmark's pre-net shape at full size: 64 sequences x 1000 steps, batch-first (the projection is then written
    # time-major through the 3-D tensor map).  Size-independent properties instead of an oracle run:
    #   * the persistent kernel agrees with the streamed one (different kernels, different summation order);
    #   * a repeat is bit-identical;
    #   * every sequence is computed independently of its batch: a sub-batch reproduces its rows bit for bit
    ops = _ops()
    g = torch.Generator().manual_seed(64)
    T, B, I, H, L = 1000, 64, 240, 1024, 2
    ps = [to_dev(p) for p in lstm_params(L, 1, I, H, g, scale=1 / 32)]
    x = to_dev(h16(torch.randn(B, T, I, generator=g)))
    m = ops.Lstm(ps, L, False, I, H, True)
    m.set_variant(ops.LSTM_PERSISTENT)
    y, hn, cn = m.forward(x, batch_first=True)
    y2, hn2, cn2 = m.forward(x, batch_first=True)
    torch.cuda.synchronize()
    assert m.last_status() == 0
    assert torch.equal(y, y2) and torch.equal(hn, hn2) and torch.equal(cn, cn2)
    assert torch.isfinite(y.float()).all()
    m.set_variant(ops.LSTM_STREAMED)
    ys, hns, cns = m.forward(x, batch_first=True)
    assert_close(y, ys, LSTM_ATOL, LSTM_RTOL, "persistent vs streamed y at T=1000, B=64")
    assert_close(cn, cns, LSTM_ATOL, LSTM_RTOL, "persistent vs streamed c_n")
    m.set_variant(ops.LSTM_PERSISTENT)
    # a smaller lock-step batch of the same kernel family (33..128 sequences) reproduces its rows bit for bit
    yb, hnb, cnb = m.forward(x[20:60].contiguous(), batch_first=True)
    assert torch.equal(yb, y[20:60]) and torch.equal(hnb, hn[:, 20:60]) and torch.equal(cnb, cn[:, 20:60])
    # 32 sequences or fewer run on the kernel without batch groups (another summation order): within the tolerance
    yw, hnw, cnw = m.forward(x[20:44].contiguous(), batch_first=True)
    assert_close(yw, y[20:44], LSTM_ATOL, LSTM_RTOL, "24 sequences alone vs in the batch of 64")
    # a single sequence runs on the low-latency kernel (another summation order): equal within the LSTM tolerance
    for n in (0, 37, 63):
        y1, hn1, cn1 = m.forward(x[n:n + 1].contiguous(), batch_first=True)
        assert_close(y1[0], y[n], LSTM_ATOL, LSTM_RTOL, f"sequence {n} alone vs in the batch")
        assert_close(cn1[:, 0], cn[:, n], LSTM_ATOL, LSTM_RTOL, f"c_n of sequence {n} alone vs in the batch")


def test_lstm_benchmark_shape_batched_vs_libtorch():
    # the benchmark's pre-net recurrence at full size (2 layers, 240 -> 1024, 1000 steps, 64 sequences in lock step,
    # batch-first) against live libtorch CPU fp32 for three of the 64 sequences: the whole output sequence, h_n and c_n.
    # fp16 hidden states feed back through 1000 steps here; the error at the last step is printed.
    ops = _ops()
    g = torch.Generator().manual_seed(65)
    T, B, I, H, L = 1000, 64, 240, 1024, 2
    ps = lstm_params(L, 1, I, H, g, scale=1 / 32)
    x = h16(torch.randn(B, T, I, generator=g))
    m = ops.Lstm([to_dev(p) for p in ps], L, False, I, H, True)
    y, hn, cn = m.forward(to_dev(x), batch_first=True)
    torch.cuda.synchronize()
    assert m.last_status() == 0
    z = torch.zeros(L, 1, H)
    for n in (0, 21, 63):
        with torch.no_grad():
            yr, hr, cr = torch.lstm(x[n:n + 1], [z, z], ps, True, L, 0.0, False, False, True)
        e = assert_close(y[n], yr[0], CONTRACT_ATOL, CONTRACT_RTOL, f"y of sequence {n} at T=1000, B=64")
        e_last = float((y[n, -1].float().cpu() - yr[0, -1]).abs().max())
        assert_close(hn[:, n], hr[:, 0], CONTRACT_ATOL, CONTRACT_RTOL, f"h_n of sequence {n}")
        assert_close(cn[:, n], cr[:, 0], CONTRACT_ATOL, CONTRACT_RTOL, f"c_n of sequence {n}")
        print(f"sequence {n}: max err over 1000 steps {e:.2e}, at the last step {e_last:.2e}")


@pytest.mark.parametrize("B,I,H,L,bi,lo,hi", [(7, 24, 64, 2, True, 1, 9), (40, 1024, 1024, 1, True, 20, 50), (128, 48, 128, 2, False, 3, 30),
                                             (33, 40, 256, 3, True, 2, 12), (5, 16, 48, 1, False, 4, 4)])
def test_lstm_packed_sequences_on_the_lockstep_kernels_vs_libtorch(B, I, H, L, bi, lo, hi):
    # packed input (sequences of ragged length, sorted) runs as a padded lock-step batch on the persistent recurrences:
    # outputs, h_n and c_n against libtorch's packed overload, and against the timestep-by-timestep streamed path
    ops = _ops()
    g = torch.Generator().manual_seed(B * 7 + H)
    D = 2 if bi else 1
    lens = sorted((int(v) for v in torch.randint(lo, hi + 1, (B,), generator=g)), reverse=True)
    T = lens[0]
    ps = lstm_params(L, D, I, H, g)
    x = h16(torch.randn(T, B, I, generator=g))
    h0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5)
    c0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5)
    packed = torch.nn.utils.rnn.pack_padded_sequence(x, torch.tensor(lens), enforce_sorted=True)
    with torch.backends.mkldnn.flags(enabled=False):
        ry, rhn, rcn = torch.lstm(packed.data, packed.batch_sizes, [h0, c0], ps, True, L, 0.0, False, bi)
    m = ops.Lstm([to_dev(p) for p in ps], L, bi, I, H, True)
    y, hn, cn = m.forward_packed(to_dev(packed.data), packed.batch_sizes, to_dev(h0), to_dev(c0))
    assert m.last_status() == 0
    assert_close(y, ry, LSTM_ATOL, LSTM_RTOL, "packed y on the lock-step kernels")
    assert_close(hn, rhn, LSTM_ATOL, LSTM_RTOL, "packed h_n")
    assert_close(cn, rcn, LSTM_ATOL, LSTM_RTOL, "packed c_n")
    m.set_packed_lockstep(False)
    ys, hns, cns = m.forward_packed(to_dev(packed.data), packed.batch_sizes, to_dev(h0), to_dev(c0))
    assert_close(ys, ry, LSTM_ATOL, LSTM_RTOL, "packed y, streamed")
    assert_close(y, ys, LSTM_ATOL, LSTM_RTOL, "lock-step vs streamed")
    assert_close(cn, cns, LSTM_ATOL, LSTM_RTOL, "lock-step vs streamed c_n")


@pytest.mark.parametrize("B,I,H", [(8, 64, 32), (33, 256, 128), (128, 2048, 1024)])
def test_lstm_decode_step_with_strided_rows_and_residual(B, I, H):
    # the decode step that writes into one half of the next cell's concatenated input: equal to forward() with T = 1 bit
    # for bit, and to the fp16 add of a residual row
    ops = _ops()
    g = torch.Generator().manual_seed(B + I + H)
    ps = [to_dev(p) for p in lstm_params(1, 1, I, H, g)]
    m = ops.Lstm(ps, 1, False, I, H, True)
    xbuf = to_dev(h16(torch.randn(B, I + 24, generator=g)))          # the input is the first I columns of wider rows
    h0 = to_dev(h16(torch.randn(1, B, H, generator=g) * 0.5))
    c0 = to_dev(h16(torch.randn(1, B, H, generator=g) * 0.5))
    res = to_dev(h16(torch.randn(B, 2 * H, generator=g)))
    y_ref, hn_ref, cn_ref = m.forward(xbuf[:, :I].contiguous().view(1, B, I), h0, c0)
    out = torch.zeros(B, 2 * H, dtype=torch.float16, device="cuda")
    hn, cn = torch.empty(B, H, dtype=torch.float16, device="cuda"), torch.empty(B, H, dtype=torch.float16, device="cuda")
    assert m.forward_step(xbuf[:, :I], h0[0], c0[0], out[:, H:], hn, cn)
    assert torch.equal(out[:, H:], y_ref[0]) and torch.equal(hn, hn_ref[0]) and torch.equal(cn, cn_ref[0])
    assert float(out[:, :H].abs().max()) == 0.0
    assert m.forward_step(xbuf[:, :I], h0[0], c0[0], out[:, :H], hn, cn, residual=res[:, H:])
    assert torch.equal(out[:, :H], ops.add_f16(y_ref[0].contiguous(), res[:, H:].contiguous()))
    assert torch.equal(hn, hn_ref[0])
    small = ops.Lstm(ps, 1, False, I, H, True)
    assert not small.forward_step(xbuf[:4, :I], h0[0, :4].contiguous(), c0[0, :4].contiguous(), out[:4, :H], hn[:4], cn[:4])


@pytest.mark.parametrize("T,B,I,H,L,bf", [(20, 1, 240, 128, 2, False), (9, 3, 24, 64, 3, True), (12, 8, 40, 256, 4, False),
                                          (1000, 1, 240, 1024, 2, False), (33, 2, 2048, 1024, 3, False)])
def test_lstm_layer_wavefront_matches_oracle_and_sequential_layers(T, B, I, H, L, bf):
    # stacked layers of up to 8 sequences run in pairs, one step apart, in one launch (the batch-1 latency path): against
    # the C oracle, and against the same handle with the layers run one after the other
    ops = _ops()
    g = torch.Generator().manual_seed(T * 7 + H + L)
    ps = lstm_params(L, 1, I, H, g, scale=1 / 32 if H >= 1024 else None)
    x = h16(torch.randn((B, T, I) if bf else (T, B, I), generator=g))
    h0 = h16(torch.randn(L, B, H, generator=g) * 0.5)
    c0 = h16(torch.randn(L, B, H, generator=g) * 0.5)
    m = ops.Lstm([to_dev(p) for p in ps], L, False, I, H, True)
    y, hn, cn = m.forward(to_dev(x), to_dev(h0), to_dev(c0), batch_first=bf)
    y_again, _, _ = m.forward(to_dev(x), to_dev(h0), to_dev(c0), batch_first=bf)
    assert m.last_status() == 0 and torch.equal(y, y_again)
    m.set_wavefront(False)
    ys, hns, cns = m.forward(to_dev(x), to_dev(h0), to_dev(c0), batch_first=bf)
    assert_close(y, ys, LSTM_ATOL, LSTM_RTOL, "wavefront vs layer after layer: y")
    assert_close(hn, hns, LSTM_ATOL, LSTM_RTOL, "wavefront vs layer after layer: h_n")
    assert_close(cn, cns, LSTM_ATOL, LSTM_RTOL, "wavefront vs layer after layer: c_n")
    if T <= 40:
        ref = co.lstm(x.numpy(), [p.numpy() for p in ps], L, False, True, h0.numpy(), c0.numpy(), bf)
        for name, a, b in zip(("y", "hn", "cn"), (y, hn, cn), ref):
            assert_close(a, b, LSTM_ATOL, LSTM_RTOL, f"wavefront {name}")
