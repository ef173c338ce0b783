"""GPU parity of the remaining benchmark configurations as test cases: a GNMT-style and a Transformer-style greedy
decode whose hot ops run through the C ABI, against the same model on libtorch CPU fp32.  The oracle replays the
device's token choices, so the logits of every step are comparable; token ids must equal the oracle's argmax wherever
its top-2 margin exceeds 1e-2."""
import numpy as np
import pytest
import torch

from pimaicompiler_b200 import decode_models as dm
from tests.cpu_backend import CpuBackend
from tests.util import CONTRACT_ATOL, CONTRACT_RTOL, assert_close

pytestmark = pytest.mark.gpu
MARGIN = 1e-2


def _check(gpu_toks, gpu_logits, ref_logits):
    assert_close(gpu_logits, ref_logits, CONTRACT_ATOL, CONTRACT_RTOL, "decode logits")
    srt = np.sort(ref_logits.numpy(), axis=1)
    decided = (srt[:, -1] - srt[:, -2]) > MARGIN
    ref_choice = ref_logits.argmax(1).numpy()
    assert (ref_choice[decided] == np.asarray(gpu_toks)[decided]).all()
    return int(decided.sum())


@pytest.mark.parametrize("H,V,S,steps,gain", [(128, 500, 13, 12, 3.0), (1024, 32320, 37, 6, 2.0)])
def test_gnmt_style_greedy_decode(H, V, S, steps, gain):
    gen = torch.Generator().manual_seed(H + S)
    w = dm.make_gnmt(H, V, S, gen, gain)
    toks, logits = dm.gnmt_greedy(dm.PimBackend(), w, H, steps)
    _, ref_logits = dm.gnmt_greedy(CpuBackend(), w, H, steps, forced=toks)
    n = _check(toks, logits, ref_logits)
    print(f"GNMT H={H} V={V}: {n}/{steps} decided steps")


@pytest.mark.parametrize("d,heads,ffn,V,layers,S,steps,gain", [(64, 4, 128, 300, 2, 9, 10, 3.0),
                                                               (512, 8, 2048, 32000, 6, 40, 5, 2.0)])
def test_transformer_style_greedy_decode(d, heads, ffn, V, layers, S, steps, gain):
    gen = torch.Generator().manual_seed(d + S)
    w = dm.make_transformer(d, heads, ffn, V, layers, S, gen, gain)
    toks, logits = dm.transformer_greedy(dm.PimBackend(), w, d, heads, steps)
    _, ref_logits = dm.transformer_greedy(CpuBackend(), w, d, heads, steps, forced=toks)
    n = _check(toks, logits, ref_logits)
    print(f"Transformer d={d} V={V}: {n}/{steps} decided steps")


@pytest.mark.parametrize("H,V,S,steps", [(128, 500, 13, 12), (1024, 32320, 37, 8)])
def test_gnmt_device_resident_step_matches_eager(H, V, S, steps):
    # the decode step captured in a CUDA graph with the token fed back on the device (arg max -> int64 index ->
    # embedding gather) must reproduce the op-by-op decode bit for bit: same kernels, same order, same inputs
    gen = torch.Generator().manual_seed(H + S)
    w = dm.make_gnmt(H, V, S, gen, 2.0)
    toks, logits = dm.gnmt_greedy(dm.PimBackend(), w, H, steps)
    gtoks, glogits, us = dm.gnmt_greedy_graph(w, H, steps)
    assert gtoks == toks
    assert torch.equal(glogits, logits)
    print(f"GNMT H={H} V={V}: {us / steps:.1f} us per token with the step resident on the device")


def test_gather_rows_by_device_index():
    from pimaicompiler_b200 import ops
    g = torch.Generator().manual_seed(3)
    table = torch.randn(29, 320, generator=g).half().cuda()
    idx = torch.tensor([28, 0, 5, 5, 17], dtype=torch.int64, device="cuda")
    assert torch.equal(ops.gather_rows(table, idx), table[idx])
    odd = torch.randn(7, 3, generator=g).half().cuda()           # 6-byte rows: the byte path
    assert torch.equal(ops.gather_rows(odd, idx[:3] % 7), odd[idx[:3] % 7])
    bad = torch.tensor([29, -1], dtype=torch.int64, device="cuda")
    assert float(ops.gather_rows(table, bad).abs().max()) == 0.0   # outside the table: a zero row, no fault


@pytest.mark.parametrize("d,heads,ffn,V,layers,S,steps", [(64, 4, 128, 300, 2, 9, 10), (512, 8, 2048, 32000, 6, 40, 8)])
def test_transformer_device_resident_step_matches_eager(d, heads, ffn, V, layers, S, steps):
    # the step as one replayed CUDA graph: token and position stay on the device, keys / values are appended in place
    # by a device-side index, self-attention takes its length from the device-side position.  Same kernels, same
    # inputs as the op-by-op decode
    gen = torch.Generator().manual_seed(d + S)
    w = dm.make_transformer(d, heads, ffn, V, layers, S, gen, 2.0)
    toks, logits = dm.transformer_greedy(dm.PimBackend(), w, d, heads, steps)
    gtoks, glogits, us = dm.transformer_greedy_graph(w, d, heads, steps)
    assert_close(glogits, logits, 1e-2, 1e-2, "graph vs eager logits")
    srt = np.sort(logits.numpy(), axis=1)
    decided = (srt[:, -1] - srt[:, -2]) > MARGIN
    assert (np.asarray(gtoks)[decided] == np.asarray(toks)[decided]).all()
    print(f"Transformer d={d} V={V}: {us / steps:.1f} us per token with the step resident on the device")


def test_scatter_rows_by_device_index():
    from pimaicompiler_b200 import ops
    g = torch.Generator().manual_seed(8)
    cache = torch.zeros(16, 512, dtype=torch.float16, device="cuda")
    rows = torch.randn(3, 512, generator=g).half().cuda()
    idx = torch.tensor([5, 0, 15], dtype=torch.int64, device="cuda")
    ops.scatter_rows(cache, idx, rows)
    ref = torch.zeros_like(cache)
    ref[idx] = rows
    assert torch.equal(cache, ref)
    ops.scatter_rows(cache, torch.tensor([16, -1], dtype=torch.int64, device="cuda"), rows[:2])   # outside: skipped
    assert torch.equal(cache, ref)
