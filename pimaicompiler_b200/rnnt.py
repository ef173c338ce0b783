"""Host-side handle of the device-resident RNN-T greedy decoder (``include/pimb200_rnnt.h``)."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import check


def _arr(ts: Sequence[torch.Tensor]):
    return (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


class RnntDecoder:
    """Packs the model once; ``decode`` runs encoder + greedy loop on the device, no host round trips.

    ``cfg`` needs the attributes of ``struct pimb200_rnnt_config``; the weight tensors are CUDA fp16,
    laid out as the TorchScript constants are (at::lstm flat lists, Linear weight/bias, Embedding weight).
    """

    def __init__(self, cfg, pre: Sequence[torch.Tensor], post: Sequence[torch.Tensor], embedding: torch.Tensor,
                 pred: Sequence[torch.Tensor], w1: torch.Tensor, b1: torch.Tensor, w2: torch.Tensor,
                 b2: torch.Tensor):
        for t in [*pre, *post, embedding, *pred, w1, b1, w2, b2]:
            if not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous():
                raise TypeError("RNN-T weights must be contiguous CUDA fp16 tensors")
        self.cfg = cfg
        self.device = w1.device
        c = _lib.RnntConfigC(*[int(getattr(cfg, n)) for n, _ in _lib.RnntConfigC._fields_])
        keep = (_arr(pre), _arr(post), _arr(pred))
        w = _lib.RnntWeightsC(keep[0], len(pre), keep[1], len(post), embedding.data_ptr(), keep[2], len(pred),
                              w1.data_ptr(), b1.data_ptr(), w2.data_ptr(), b2.data_ptr())
        h = C.c_void_p()
        check(_lib.lib().pimb200_rnnt_create(C.byref(c), C.byref(w), C.byref(h)), "rnnt_create")
        self._h = h

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().pimb200_rnnt_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def info(self) -> dict:
        cs, mask, sm = C.c_int(), C.c_int(), C.c_size_t()
        check(_lib.lib().pimb200_rnnt_info(self._h, C.byref(cs), C.byref(mask), C.byref(sm)), "rnnt_info")
        return {"cluster_size": cs.value, "smem_mask": mask.value, "smem_bytes": sm.value}

    def set_encoder_batch(self, n: int) -> None:
        """Utterances the encoder advances in lock step (1..64)."""
        check(_lib.lib().pimb200_rnnt_set_encoder_batch(self._h, int(n)), "rnnt_set_encoder_batch")

    def set_greedy_multi(self, mode: int) -> None:
        """Greedy kernel for crowded calls: 1 = best available, 2 = FMA lock-step, 0 = one utterance per cluster."""
        check(_lib.lib().pimb200_rnnt_set_greedy_multi(self._h, int(mode)), "rnnt_set_greedy_multi")

    def profile(self, enable: bool) -> None:
        check(_lib.lib().pimb200_rnnt_profile_enable(self._h, 1 if enable else 0), "rnnt_profile_enable")

    def profile_read(self) -> dict:
        ms, n, by = C.c_double(), C.c_long(), C.c_double()
        check(_lib.lib().pimb200_rnnt_profile_read(self._h, C.byref(ms), C.byref(n), C.byref(by)),
              "rnnt_profile_read")
        return {"ms": ms.value, "recurrences": n.value, "bytes": by.value}

    def last_status(self) -> int:
        """Device-side status of the decodes since the last call (0, or ERR_TIMEOUT when a bounded wait gave up);
        synchronises the device and clears the status."""
        return int(_lib.lib().pimb200_rnnt_last_status(self._h))

    def check_status(self, where: str = "rnnt") -> None:
        """Raises when a kernel of an earlier decode gave up; call after synchronising ``decode_into``'s stream."""
        check(self.last_status(), where)

    def set_wavefront(self, on: bool) -> None:
        """Encoder layers in pairs, one step apart, for calls of up to 8 utterances (default on)."""
        check(_lib.lib().pimb200_rnnt_set_wavefront(self._h, 1 if on else 0), "rnnt_set_wavefront")

    def set_poll_limit(self, limit: int) -> None:
        """Test hook: iteration limit of the bounded waits (encoder recurrences, greedy kernel's exchanges)."""
        check(_lib.lib().pimb200_rnnt_set_poll_limit(self._h, int(limit)), "rnnt_set_poll_limit")

    def set_trace(self, buffer: Optional[torch.Tensor]) -> None:
        """Diagnostics: int64 CUDA tensor of (T / stack_factor) * 8 elements that the greedy kernel fills with eight
        clocks per frame of utterance 0 (``None`` switches it off).  The caller keeps the tensor alive."""
        check(_lib.lib().pimb200_rnnt_set_trace(self._h, None if buffer is None else buffer.data_ptr()),
              "rnnt_set_trace")

    def decode_into(self, feats: torch.Tensor, tokens: torch.Tensor, n_tokens: torch.Tensor,
                    logits: Optional[torch.Tensor] = None) -> None:
        """Asynchronous decode of feats [n_utts, T, feat_dim] into preallocated device outputs."""
        n_utts, T, _ = feats.shape
        check(_lib.lib().pimb200_rnnt_decode(self._h, feats.data_ptr(), T, n_utts, tokens.data_ptr(),
                                             n_tokens.data_ptr(), None if logits is None else logits.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream), "rnnt_decode")

    def decode(self, feats: torch.Tensor, want_logits: bool = False):
        """feats [n_utts, T, feat_dim] (or [T, feat_dim]) CUDA fp16 -> list of token lists (+ logits)."""
        if feats.dim() == 2:
            feats = feats.unsqueeze(0)
        feats = feats.contiguous()
        n_utts, T, _ = feats.shape
        Tp = T // self.cfg.stack_factor
        tokens = torch.zeros(n_utts, Tp, dtype=torch.int32, device=feats.device)
        n_tokens = torch.zeros(n_utts, dtype=torch.int32, device=feats.device)
        logits = torch.empty(n_utts, Tp, self.cfg.vocab, dtype=torch.float32, device=feats.device) if want_logits \
            else None
        self.decode_into(feats, tokens, n_tokens, logits)
        n = n_tokens.cpu().tolist()   # synchronises the stream
        self.check_status("rnnt_decode")
        tk = tokens.cpu()
        out = [tk[u, : n[u]].tolist() for u in range(n_utts)]
        return (out, logits) if want_logits else out


GREEDY_TRACE_PHASES_SINGLE = ("z + logits", "arg max", "layer 0: reduce", "layer 0: gates + exchange",
                              "layer 1: product + gates + exchange", "joint half: product",
                              "joint half: exchange + next state products")
GREEDY_TRACE_PHASES_GROUP = ("z", "logits product", "arg max", "layer 0: decisions + partial sums",
                             "layer 0: gates + exchange", "layer 1: product + gates + exchange",
                             "joint half: product + exchange")


def greedy_frame_trace(n_utts: int, frames: int, seed: int = 0) -> dict:
    """Mean SM cycles per phase of one greedy frame, from the kernel's own clocks (utterance 0, cluster 0, CTA 0).

    Builds the benchmark model with synthetic weights (every frame emits a label: the worst case for the prediction
    network), decodes ``n_utts`` utterances of ``frames`` feature frames once to warm up and once with the trace on.
    One utterance runs the one-utterance kernel; more utterances than clusters run the 8-per-cluster kernel.
    """
    from . import synthetic as syn
    cfg = syn.RnntConfig()
    w = syn.make_rnnt_weights(cfg, seed=seed)
    dev = lambda t: t.to(torch.float16).cuda().contiguous()
    dec = RnntDecoder(cfg, [dev(p) for p in w.pre], [dev(p) for p in w.post], dev(w.embedding),
                      [dev(p) for p in w.pred], dev(w.w1), dev(w.b1), dev(w.w2), dev(w.b2))
    feats = torch.stack([dev(syn.make_features(frames, cfg, i)) for i in range(n_utts)])
    dec.decode(feats)
    Tp = frames // cfg.stack_factor
    trace = torch.zeros(Tp * 8, dtype=torch.int64, device="cuda")
    dec.set_trace(trace)
    tokens = dec.decode(feats)
    dec.set_trace(None)
    t = trace.cpu().numpy().reshape(Tp, 8)[5:Tp - 5]
    names = GREEDY_TRACE_PHASES_SINGLE if n_utts == 1 else GREEDY_TRACE_PHASES_GROUP
    out = {name: float((t[:, i + 1] - t[:, i]).mean()) for i, name in enumerate(names)}
    out["frame"] = float((t[1:, 0] - t[:-1, 0]).mean())
    out["tokens of utterance 0"] = len(tokens[0])
    dec.close()
    return out
