"""GPU parity of the fp16 add and the cat / copy glue ops (bit-exact)."""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as co

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _ops():
    from pimaicompiler_b200 import ops
    return ops


def test_add_golden_bit_exact():
    ops = _ops()
    z = np.load(os.path.join(GOLD, "glue.npz"))
    A, B, Br = (torch.from_numpy(z[k]).cuda() for k in ("A", "B", "Br"))
    assert np.array_equal(ops.add_f16(A, B).cpu().numpy(), z["add_sym"])
    assert np.array_equal(ops.add_f16(A, Br).cpu().numpy(), z["add_bcast"])


@pytest.mark.parametrize("m,n", [(1, 1024), (4, 1024), (3, 513), (1, 3), (7, 8), (64, 512), (1000, 1030)])
def test_add_matches_oracle_any_tail(m, n):
    ops = _ops()
    g = torch.Generator().manual_seed(m * 10007 + n)
    A = torch.randn(m, n, generator=g).to(torch.float16)
    B = torch.randn(m, n, generator=g).to(torch.float16)
    Br = torch.randn(n, generator=g).to(torch.float16)
    ref = co.add(A.float().numpy(), B.float().numpy()).astype(np.float16)
    assert np.array_equal(ops.add_f16(A.cuda(), B.cuda()).cpu().numpy(), ref)
    refb = co.add(A.float().numpy(), Br.float().numpy()).astype(np.float16)
    assert np.array_equal(ops.add_f16(A.cuda(), Br.cuda()).cpu().numpy(), refb)
    # in place into A, as the reference's executor does (aten_ops_executor.cpp:123-125)
    Ad = A.cuda()
    ops.add_f16(Ad, B.cuda(), out=Ad)
    assert np.array_equal(Ad.cpu().numpy(), ref)


def test_cat_golden_and_roundtrip():
    ops = _ops()
    z = np.load(os.path.join(GOLD, "glue.npz"))
    parts = [torch.from_numpy(z[k]).cuda() for k in ("cat0", "cat1", "cat2")]
    assert np.array_equal(ops.cat(parts, 1).cpu().numpy(), z["cat_out"])
    # atenCatOpTest (aten_ops_ut.cpp:30-41): split then cat gives the tensor back
    t = torch.rand(4, 6, 10).to(torch.float16).cuda()
    for dim, size in ((0, 1), (1, 2), (2, 5), (2, 3), (-1, 1)):
        pieces = [p.contiguous() for p in torch.split(t, size, dim=dim)]
        assert torch.equal(ops.cat(pieces, dim), t)
    # other element sizes, empty operand
    ti = torch.arange(24, dtype=torch.int64).view(2, 12).cuda()
    assert torch.equal(ops.cat([ti[:, :5].contiguous(), ti[:, 5:5].contiguous(), ti[:, 5:].contiguous()], 1), ti)
    tb = torch.arange(21, dtype=torch.uint8).view(3, 7).cuda()
    assert torch.equal(ops.cat([tb[:, :3].contiguous(), tb[:, 3:].contiguous()], 1), tb)


def test_kv_append_style_cat():
    # Transformer decode appends one [1,h,1,64] slice to a [1,h,t,64] cache every step
    ops = _ops()
    cache = torch.randn(1, 8, 5, 64).to(torch.float16).cuda()
    new = torch.randn(1, 8, 1, 64).to(torch.float16).cuda()
    assert torch.equal(ops.cat([cache, new], 2), torch.cat([cache, new], 2))


def test_copy_into_slice_of_a_larger_buffer():
    # the "custom cat" aliasing: write a [1,1,1024] result into the second half of a {1,1,2048} buffer
    ops = _ops()
    buf = torch.zeros(1, 1, 2048, dtype=torch.float16, device="cuda")
    src = torch.randn(1, 1, 1024).to(torch.float16).cuda()
    ops.copy_2d(buf, 1024 * 2, 2048 * 2, src, 0, 1024 * 2, 1024 * 2, 1)
    assert torch.equal(buf[..., 1024:], src) and (buf[..., :1024] == 0).all()
    # atenCopyOpTest size (aten_ops_ut.cpp:43-63), odd byte offsets
    s = torch.rand(100).cuda()
    d = torch.zeros(100, device="cuda")
    ops.copy_2d(d, 0, 400, s, 0, 400, 400, 1)
    assert torch.equal(d, s)
    sb = torch.arange(64, dtype=torch.uint8).cuda()
    db = torch.zeros(64, dtype=torch.uint8).cuda()
    ops.copy_2d(db, 1, 9, sb, 3, 11, 5, 4)
    exp = torch.zeros(64, dtype=torch.uint8)
    for r in range(4):
        exp[1 + r * 9:1 + r * 9 + 5] = torch.arange(64, dtype=torch.uint8)[3 + r * 11:3 + r * 11 + 5]
    assert torch.equal(db.cpu(), exp)
