"""Shared helpers of the parity tests."""
import numpy as np
import torch

# contract of the hot path: fp16 storage / fp32 accumulate vs the fp32 CPU oracle
CONTRACT_ATOL = 2e-2
CONTRACT_RTOL = 1e-2


def h16(t: torch.Tensor) -> torch.Tensor:
    """Round an fp32 CPU tensor to fp16 values (kept in fp32) — what both sides of a parity test consume."""
    return t.to(torch.float16).to(torch.float32)


def to_dev(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16).cuda().contiguous()


def assert_close(got, ref, atol, rtol, what=""):
    got = np.asarray(got.detach().float().cpu().numpy() if isinstance(got, torch.Tensor) else got, dtype=np.float64)
    ref = np.asarray(ref.detach().float().cpu().numpy() if isinstance(ref, torch.Tensor) else ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    err = np.abs(got - ref)
    bound = atol + rtol * np.abs(ref)
    bad = err > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} outside atol={atol} rtol={rtol}; "
                           f"max abs err {err.max():.3e} at ref {ref.flat[err.argmax()]:.3e}")
    return float(err.max())


def lstm_params(L, D, I, H, gen, scale=None, has_biases=True):
    """Flat at::lstm parameter list (fp32 CPU tensors holding fp16-representable values)."""
    ps = []
    k = scale if scale is not None else 1.0 / (H ** 0.5)
    for l in range(L):
        Il = I if l == 0 else D * H
        for _ in range(D):
            ps.append(h16((torch.rand(4 * H, Il, generator=gen) * 2 - 1) * k))
            ps.append(h16((torch.rand(4 * H, H, generator=gen) * 2 - 1) * k))
            if has_biases:
                ps.append(h16((torch.rand(4 * H, generator=gen) * 2 - 1) * k))
                ps.append(h16((torch.rand(4 * H, generator=gen) * 2 - 1) * k))
    return ps
