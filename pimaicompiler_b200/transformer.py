"""Transformer-base greedy translation (configuration C5) for many sequences per GPU, every op through libpimb200.so.

The reference runs its Transformer graph for one sequence (input [1, 11] token ids,
examples/runtime/source/pipeline_manager.cpp:216-217): per generated token the interpreter dispatches each linear as a
batch-1 addmm, each attention as matmul -> softmax -> matmul with per-head reshapes, and grows the key / value cache with
an at::cat (runtime/source/executor/op_executor/aten_ops_executor.cpp:181-216, 2488-2505, 3402-3436, 772-819).  Sequences
are independent, so a GPU runs `group` of them in lock step:

  * encoder: the group's sequences, sorted by length and padded, form one [group, S, d] batch; each layer is one fused
    q/k/v projection GEMM, one attention launch (a CTA per head and sequence, own length), the output projection, the
    feed-forward pair (ReLU fused into the first GEMM) and two fused residual-add + layer-norm launches;
  * the cross-attention keys and values of all decoder layers come from one GEMM over the encoder output;
  * decoder: all `steps` steps of the group are captured into ONE CUDA graph.  Step t's projection GEMM writes q, k, v
    straight into row t of a [steps, group, 3d] cache (no append, no device-side position), single-query attention reads
    rows 0..t of it, the vocabulary projection is a GEMM over the group's rows and the arg max writes row t of the token
    table, which the next step's embedding gather reads.

`TransformerTranslator.translate` is the user call; `bench.py --workload c5` times it.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import ops


class TransformerTranslator:
    def __init__(self, cfg, weights: dict, group: int = 128, device: Optional[torch.device] = None):
        ops.init()
        self.cfg = cfg
        self.G = int(group)
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        d, G, S, T = cfg.d_model, self.G, cfg.max_len, cfg.max_steps
        self.d = d

        def put(t):
            return t.to(torch.float16).to(self.dev).contiguous()

        w = weights
        self.emb_src, self.emb_tgt, self.pe, self.Wo = put(w["emb_src"]), put(w["emb_tgt"]), put(w["pe"]), put(w["Wo"])

        def fuse(L, names):
            return put(torch.cat([L[n] for n in names])), put(torch.cat([L[n + "_b"] for n in names]))

        self.enc = []
        for L in w["enc"]:
            qkv, qkv_b = fuse(L, ("sq", "sk", "sv"))
            self.enc.append({"qkv": qkv, "qkv_b": qkv_b, **{k: put(L[k]) for k in ("so", "so_b", "f1", "f1_b", "f2", "f2_b")}})
        self.dec = []
        for L in w["dec"]:
            qkv, qkv_b = fuse(L, ("sq", "sk", "sv"))
            self.dec.append({"qkv": qkv, "qkv_b": qkv_b,
                             **{k: put(L[k]) for k in ("so", "so_b", "cq", "cq_b", "co", "co_b", "f1", "f1_b", "f2", "f2_b")}})
        # cross-attention key / value projections of all decoder layers side by side: [layers * 2d, d]
        self.ckv = put(torch.cat([torch.cat([L["ck"], L["cv"]]) for L in w["dec"]]))
        self.ckv_b = put(torch.cat([torch.cat([L["ck_b"], L["cv_b"]]) for L in w["dec"]]))
        f16 = dict(dtype=torch.float16, device=self.dev)
        i64 = dict(dtype=torch.int64, device=self.dev)
        nl = cfg.layers
        self.lengths = torch.ones(G, **i64)
        self.cross = torch.zeros(G, S, nl * 2 * d, **f16)            # encoder side, at its maximum size
        self.cache = [torch.zeros(T, G, 3 * d, **f16) for _ in range(nl)]
        self.toks = torch.zeros(T + 1, G, **i64)                     # row 0: start tokens, row t+1: choice of step t
        self.forced = torch.zeros(T + 1, G, **i64)
        self.logits = torch.zeros(G, cfg.vocab, **f16)
        self.logits_all = None
        self._graphs = {}
        self.launches_per_step = 0

    # ------------------------------------------------------------------------------------------------ encoder
    def encode(self, group: dict) -> None:
        """One staged group (see stage(); tensors on the device): `ids` [G, S_g] int64 (padded with any valid id) and
        `lengths` [G] int64.  Fills the cross-attention keys / values of every decoder layer."""
        cfg, d, G = self.cfg, self.d, self.G
        ids = group["ids"]
        Sg = ids.shape[1]
        n = G * Sg
        self.lengths.copy_(group["lengths"])
        x = ops.gather_rows(self.emb_src, ids.reshape(-1))                       # [n, d]
        x = ops.add_f16(x.view(G, Sg * d), self.pe[:Sg].reshape(1, Sg * d)).view(n, d)   # positions: one row per sequence
        for L in self.enc:
            qkv = ops.gemm_wx(L["qkv"], x, L["qkv_b"]).view(G, Sg, 3 * d)
            a = ops.attention_block(qkv[:, :, :d], qkv[:, :, d:2 * d], qkv[:, :, 2 * d:], cfg.heads, self.lengths)
            x = ops.add_layer_norm(x, ops.gemm_wx(L["so"], a.view(n, d), L["so_b"]))
            f = ops.gemm_wx(L["f2"], ops.gemm_wx(L["f1"], x, L["f1_b"], ops.ACT_RELU), L["f2_b"])
            x = ops.add_layer_norm(x, f)
        kv = ops.gemm_wx(self.ckv, x, self.ckv_b).view(G, Sg, -1)
        self.cross[:, :Sg].copy_(kv)

    # ------------------------------------------------------------------------------------------------ decoder
    def _step(self, t: int, forced: bool, want_logits: bool) -> int:
        cfg, d, G = self.cfg, self.d, self.G
        n = 0
        tok = (self.forced if forced else self.toks)[t]
        x = ops.gather_rows(self.emb_tgt, tok); n += 1
        x = ops.add_f16(x, self.pe[t]); n += 1
        for i, L in enumerate(self.dec):
            row = self.cache[i][t]                                               # [G, 3d]: q, k, v of step t
            ops.gemm_wx(L["qkv"], x, L["qkv_b"], out=row); n += 1
            a = ops.attention_rows(row[:, :d], self.cache[i][:, :, d:2 * d], self.cache[i][:, :, 2 * d:], cfg.heads,
                                   len_add=t + 1, time_major=True); n += 1
            x = ops.add_layer_norm(x, ops.gemm_wx(L["so"], a, L["so_b"])); n += 2
            cq = ops.gemm_wx(L["cq"], x, L["cq_b"]); n += 1
            ck = self.cross[:, :, (2 * i) * d:(2 * i + 1) * d]
            cv = self.cross[:, :, (2 * i + 1) * d:(2 * i + 2) * d]
            ca = ops.attention_rows(cq, ck, cv, cfg.heads, len_dev=self.lengths, len_inc=1); n += 1
            x = ops.add_layer_norm(x, ops.gemm_wx(L["co"], ca, L["co_b"])); n += 2
            f = ops.gemm_wx(L["f2"], ops.gemm_wx(L["f1"], x, L["f1_b"], ops.ACT_RELU), L["f2_b"]); n += 2
            x = ops.add_layer_norm(x, f); n += 1
        lg = self.logits_all[t] if want_logits else self.logits
        ops.gemm_wx(self.Wo, x, out=lg); n += 1
        ops.argmax(lg, out=self.toks[t + 1]); n += 1
        return n

    def _graph(self, steps: int, forced: bool, want_logits: bool):
        key = (steps, forced, want_logits)
        if key in self._graphs:
            return self._graphs[key]
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):          # eager once: workspaces exist before the capture
            self._step(0, forced, want_logits)
        torch.cuda.current_stream(self.dev).wait_stream(side)
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for t in range(steps):
                self.launches_per_step = self._step(t, forced, want_logits)
        self._graphs[key] = g
        return g

    def decode(self, steps: int, forced: Optional[torch.Tensor] = None, want_logits: bool = False):
        """All `steps` greedy steps of the encoded group (one graph launch).  Returns the token table [steps, G] (device)
        and, when asked, the logits [steps, G, V]."""
        cfg, G = self.cfg, self.G
        if steps > cfg.max_steps:
            raise ValueError("more steps than the configuration's maximum")
        if want_logits and (self.logits_all is None or self.logits_all.shape[0] < steps):
            self.logits_all = torch.zeros(steps, G, cfg.vocab, dtype=torch.float16, device=self.dev)
            self._graphs = {k: v for k, v in self._graphs.items() if not k[2]}
        self.toks[0].fill_(cfg.bos)
        if forced is not None:
            self.forced[0].fill_(cfg.bos)
            self.forced[1:steps].copy_(forced[:steps - 1].to(self.dev))          # step t is fed the token forced at t - 1
        self._graph(steps, forced is not None, want_logits).replay()
        toks = self.toks[1:steps + 1]
        return (toks, self.logits_all[:steps]) if want_logits else (toks, None)

    # ------------------------------------------------------------------------------------------------ user call
    def stage(self, sequences: Sequence[torch.Tensor]):
        """Sorts by length and packs lock-step groups: dicts of `idx` (sequence indices), `ids` (padded [G, S_g]) and
        `lengths` [G], the tensors in pinned host memory."""
        G = self.G
        order = sorted(range(len(sequences)), key=lambda i: -int(sequences[i].shape[0]))
        groups = []
        for g0 in range(0, len(order), G):
            idx = order[g0:g0 + G]
            lens = [int(sequences[i].shape[0]) for i in idx]
            if max(lens) > self.cfg.max_len or min(lens) < 1:
                raise ValueError("sequence length outside 1..max_len")
            ids = torch.full((G, max(lens)), 4, dtype=torch.int64)
            for j, i in enumerate(idx):
                ids[j, :lens[j]] = sequences[i]
            lens_t = torch.ones(G, dtype=torch.int64)
            lens_t[:len(idx)] = torch.tensor(lens, dtype=torch.int64)
            groups.append({"idx": idx, "ids": ids.pin_memory(), "lengths": lens_t.pin_memory()})
        return groups

    def to_device(self, group: dict) -> dict:
        return {"idx": group["idx"], "ids": group["ids"].to(self.dev, non_blocking=True),
                "lengths": group["lengths"].to(self.dev, non_blocking=True)}

    def h2d_bytes(self, group: dict) -> int:
        return 8 * (group["ids"].numel() + group["lengths"].numel())

    def check_status(self) -> None:
        """Raises if a bounded wait of the tensor-core GEMM gave up since the last check."""
        from . import _lib
        rc = _lib.lib().pimb200_gemm_last_status()
        if rc != 0:
            raise RuntimeError(f"device-side wait timed out (gemm status {rc})")

    def translate(self, sequences: Sequence[torch.Tensor], steps: Optional[int] = None,
                  forced: Optional[Sequence[Sequence[int]]] = None, want_logits: bool = False):
        """sequences: 1-D int64 CPU tensors of source token ids.  Returns one token list per sequence (cut behind the first
        end-of-sequence token unless `steps` is given) and, when asked, each one's logits [steps, V]."""
        cfg, G = self.cfg, self.G
        n = len(sequences)
        run_steps = cfg.max_steps if steps is None else steps
        out_toks: List[Optional[List[int]]] = [None] * n
        out_logits: List[Optional[torch.Tensor]] = [None] * n
        pending = []
        for group in self.stage(sequences):
            idx = group["idx"]
            self.encode(self.to_device(group))
            f = None
            if forced is not None:
                f = torch.zeros(run_steps, G, dtype=torch.int64)
                for j, i in enumerate(idx):
                    f[:, j] = torch.tensor(list(forced[i])[:run_steps], dtype=torch.int64)
            toks, logits = self.decode(run_steps, f, want_logits)
            host = torch.empty(toks.shape, dtype=torch.int64).pin_memory()
            host.copy_(toks, non_blocking=True)
            pending.append((idx, host, logits.float().cpu() if want_logits else None))
            torch.cuda.current_stream(self.dev).synchronize()   # the next group reuses the token table
            self.check_status()
        for idx, host, logits in pending:
            for j, i in enumerate(idx):
                seq = host[:, j].tolist()
                if steps is None and cfg.eos in seq:
                    seq = seq[:seq.index(cfg.eos) + 1]
                out_toks[i] = seq
                if logits is not None:
                    out_logits[i] = logits[:, j]
        return (out_toks, out_logits) if want_logits else out_toks
