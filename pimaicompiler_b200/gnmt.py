"""GNMT greedy translation (configuration C4) for many sentences per GPU, every op through libpimb200.so.

The reference serves one sentence at a time: its interpreter walks the GNMT graph once per token, each decoder layer one
aten::lstm call with seq_len 1, the attention a chain of add / tanh / matmul / softmax / bmm nodes and the vocabulary
projection a batch-1 addmm (runtime/source/executor/op_executor/aten_ops_executor.cpp:2135-2307, 181-216, 110-166; GNMT
inputs examples/runtime/source/pipeline_manager.cpp:143-151).  Sentences are independent, so a GPU that has to serve
hundreds of them runs `group` sentences in lock step instead:

  * encoder: the group's sentences, sorted by length, go through each layer as packed batches of up to 128 sentences
    (aten::lstm's packed overload, which the library runs as a padded lock-step batch on the persistent weight-stationary
    recurrence, the backward direction of the first layer on the sentences reversed one by one);
  * decoder: one step for the whole group is 4 x (two GEMMs over the group's rows + the gate kernel, which writes the
    cell's output, for the last two cells with the residual added, straight into the next cell's concatenated input), one
    attention launch (a CTA per sentence, own source length), the vocabulary projection as a GEMM (the 66 MB matrix is
    read once per step for all sentences) and a row-wise arg max; two steps (state buffers alternate) are captured into
    one CUDA graph and replayed, the chosen tokens staying on the device until the group is done.

`GnmtTranslator.translate` is the user call; `bench.py --workload c4` times it.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import ops


def stage_groups(sentences: Sequence[torch.Tensor], G: int, enc_batch: int, max_len: int, pin: bool = False):
    """Host-side packing of sentences into lock-step groups of G.  A group is a dict: `idx` (sentence indices, longest
    first), `S` (longest sentence), `lengths` [G] int64, and `slices`: per `enc_batch` sentences the packed token ids
    [sum of lengths] (timestep-major, the order of torch's pack_padded_sequence), `batch_sizes` (CPU int64, one per
    timestep) and `dst`, the row t * G + j of the padded [S, G] buffer each packed row belongs to.  A ragged last group
    is filled with one-token dummies.  With `pin` the tensors that travel to the device are in pinned host memory."""
    keep = (lambda t: t.pin_memory()) if pin else (lambda t: t)
    order = sorted(range(len(sentences)), key=lambda i: -int(sentences[i].shape[0]))
    groups = []
    for g0 in range(0, len(order), G):
        idx = order[g0:g0 + G]
        lens = [int(sentences[i].shape[0]) for i in idx]
        if max(lens) > max_len or min(lens) < 1:
            raise ValueError("sentence length outside 1..max_len")
        lens_all = lens + [1] * (G - len(idx))
        toks = [sentences[i] for i in idx] + [torch.full((1,), 4, dtype=torch.int64)] * (G - len(idx))
        slices = []
        for j0 in range(0, G, enc_batch):
            j1 = min(j0 + enc_batch, G)
            sl_lens = lens_all[j0:j1]
            nb, Ss = j1 - j0, sl_lens[0]
            pad = torch.full((Ss, nb), 4, dtype=torch.int64)
            for b in range(nb):
                pad[:sl_lens[b], b] = toks[j0 + b]
            steps_col = torch.arange(Ss, dtype=torch.int64).view(Ss, 1)
            mask = steps_col < torch.tensor(sl_lens, dtype=torch.int64).view(1, nb)      # [t, b]: sentence b has a step t
            dst = (steps_col * G + j0 + torch.arange(nb, dtype=torch.int64).view(1, nb))[mask]
            slices.append({"ids": keep(pad[mask]), "dst": keep(dst), "batch_sizes": mask.sum(1)})
        groups.append({"idx": idx, "S": max(lens_all), "lengths": keep(torch.tensor(lens_all, dtype=torch.int64)),
                       "slices": slices})
    return groups


class GnmtTranslator:
    def __init__(self, cfg, weights: dict, group: int = 128, device: Optional[torch.device] = None):
        ops.init()
        self.cfg = cfg
        self.G = int(group)
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        H, V, G, S = cfg.hidden, cfg.vocab, self.G, cfg.max_len
        self.H, self.V, self.S = H, V, S

        def put(t):
            return t.to(torch.float16).to(self.dev).contiguous()

        self.w = {k: ([put(t) for t in v] if isinstance(v, list) else put(v)) for k, v in weights.items()}
        self.v_norm = put(weights["att_v"] / weights["att_v"].norm() * float(weights["att_g"]))
        self.lstm = {"enc0": ops.Lstm(self.w["enc0_f"] + self.w["enc0_r"], 1, True, H, H, True)}   # bidirectional first layer
        for name in ("enc1", "enc2", "enc3", "dec0", "dec1", "dec2", "dec3"):
            p = self.w[name]
            self.lstm[name] = ops.Lstm(p, 1, False, p[0].shape[1], H, True)
        f16 = dict(dtype=torch.float16, device=self.dev)
        i64 = dict(dtype=torch.int64, device=self.dev)
        # encoder outputs / attention keys of the current group, time-major, at their maximum size
        self.enc_out = torch.zeros(S, G, H, **f16)
        self.keys_proj = torch.zeros(S, G, H, **f16)
        self.lengths = torch.ones(G, **i64)
        # decoder step buffers (addresses fixed: the step is replayed from a CUDA graph)
        self.tok = torch.zeros(G, **i64)
        self.step_idx = torch.zeros(1, **i64)
        self.x = torch.zeros(G, H, **f16)
        self.q = torch.zeros(G, H, **f16)
        self.scores = torch.zeros(G, S, dtype=torch.float32, device=self.dev)
        self.y = [torch.zeros(1, G, H, **f16) for _ in range(4)]
        self.r2 = torch.zeros(G, H, **f16)
        self.r3 = torch.zeros(G, H, **f16)
        self.cat = [torch.zeros(G, 2 * H, **f16) for _ in range(3)]
        self.logits = torch.zeros(G, V, **f16)
        self.state = [[torch.zeros(1, G, H, **f16) for _ in range(8)] for _ in range(2)]   # h0..3, c0..3, two sets
        self.toks_out = torch.zeros(cfg.max_steps, G, **i64)
        self.forced = None
        self.logits_out = None
        self._graphs = {}
        self.launches_per_step = 0

    # ------------------------------------------------------------------------------------------------ encoder
    ENC_BATCH = 128          # sequences per packed aten::lstm call (the lock-step recurrences take up to 128)

    def encode(self, group: dict) -> int:
        """One staged group (see stage(); tensors on the device).  Every slice of up to 128 sentences goes through the
        encoder as a PACKED batch (the aten::lstm overload the reference's GNMT graph uses for its encoder): rows of
        padding never reach a GEMM or an add, and the library runs the packed batch on the lock-step recurrences.  The
        encoder states are scattered into the padded time-major buffer the attention kernel reads.  Returns S_g."""
        H, G = self.H, self.G
        Sg = group["S"]
        self.lengths.copy_(group["lengths"])
        flat = self.enc_out.view(-1, H)
        for sl in group["slices"]:
            x = ops.gather_rows(self.w["emb_src"], sl["ids"])                       # packed rows [sum of lengths, H]
            y0, _, _ = self.lstm["enc0"].forward_packed(x, sl["batch_sizes"])       # [rows, 2H]
            y1, _, _ = self.lstm["enc1"].forward_packed(y0, sl["batch_sizes"])
            y2, _, _ = self.lstm["enc2"].forward_packed(y1, sl["batch_sizes"])
            y2 = ops.add_f16(y2, y1)
            y3, _, _ = self.lstm["enc3"].forward_packed(y2, sl["batch_sizes"])
            ops.scatter_rows(flat, sl["dst"], ops.add_f16(y3, y2))                  # row (t, j) of the padded buffer
        n = Sg * G
        ops.gemm_wx(self.w["Wk"], self.enc_out[:Sg].view(n, H), out=self.keys_proj[:Sg].view(n, H))
        return Sg

    # ------------------------------------------------------------------------------------------------ decoder
    def _step(self, src: List[torch.Tensor], dst: List[torch.Tensor]) -> int:
        """One decode step of the whole group; state read from `src`, written to `dst`.  Returns its launch count."""
        H, G, w = self.H, self.G, self.w
        row = 2 * H * 2          # bytes per row of a concatenation buffer
        half = H * 2
        n = 0
        cat = self.cat
        ops.gather_rows(w["emb_tgt"], self.tok, out=self.x); n += 1
        # groups of 8 or more sentences: every cell writes its output (the last two with their residual added) straight
        # into the first half of the next cell's concatenated input, as the reference's labelled GNMT graph does
        fused = self.lstm["dec0"].forward_step(self.x, src[0][0], src[4][0], cat[0][:, :H], dst[0][0], dst[4][0])
        if fused:
            n += 3
            y0 = cat[0][:, :H]
        else:
            self.lstm["dec0"].forward(self.x.view(1, G, H), src[0], src[4], out=(self.y[0], dst[0], dst[4])); n += 1
            y0 = self.y[0].view(G, H)
            ops.copy_2d(cat[0], 0, row, y0, 0, half, half, G); n += 1
        ops.gemm_wx(w["Wq"], y0, out=self.q); n += 1
        ops.additive_attention(self.q, self.keys_proj, self.enc_out, self.lengths, self.v_norm, w["att_b"],
                               out=cat[0][:, H:], scores=self.scores); n += 2
        for i in (1, 2):          # the context is the second half of every layer's input
            ops.copy_2d(cat[i], half, row, cat[0], half, row, half, G); n += 1
        if fused:
            self.lstm["dec1"].forward_step(cat[0], src[1][0], src[5][0], cat[1][:, :H], dst[1][0], dst[5][0]); n += 3
            self.lstm["dec2"].forward_step(cat[1], src[2][0], src[6][0], cat[2][:, :H], dst[2][0], dst[6][0],
                                           residual=cat[1][:, :H]); n += 3
            self.lstm["dec3"].forward_step(cat[2], src[3][0], src[7][0], self.r3, dst[3][0], dst[7][0],
                                           residual=cat[2][:, :H]); n += 3
        else:
            self.lstm["dec1"].forward(cat[0].view(1, G, 2 * H), src[1], src[5], out=(self.y[1], dst[1], dst[5])); n += 1
            y1 = self.y[1].view(G, H)
            ops.copy_2d(cat[1], 0, row, y1, 0, half, half, G); n += 1
            self.lstm["dec2"].forward(cat[1].view(1, G, 2 * H), src[2], src[6], out=(self.y[2], dst[2], dst[6])); n += 1
            ops.add_f16(self.y[2].view(G, H), y1, out=self.r2); n += 1
            ops.copy_2d(cat[2], 0, row, self.r2, 0, half, half, G); n += 1
            self.lstm["dec3"].forward(cat[2].view(1, G, 2 * H), src[3], src[7], out=(self.y[3], dst[3], dst[7])); n += 1
            ops.add_f16(self.y[3].view(G, H), self.r2, out=self.r3); n += 1
        ops.gemm_wx(w["Wc"], self.r3, w["bc"], out=self.logits); n += 1
        ops.argmax(self.logits, out=self.tok); n += 1
        # record the chosen tokens (and, for the parity tests, the logits) in row step_idx of the output tables
        ops.scatter_rows(self.toks_out.view(self.cfg.max_steps, G), self.step_idx, self.tok.view(1, G)); n += 1
        if self.logits_out is not None:
            ops.scatter_rows(self.logits_out.view(self.logits_out.shape[0], -1), self.step_idx, self.logits.view(1, -1)); n += 1
        if self.forced is not None:   # teacher forcing: the fed-back token comes from a table instead of the arg max
            ops.gather_rows(self.forced, self.step_idx, out=self.tok.view(1, G)); n += 1
        self.step_idx.add_(1)
        return n

    def _graph(self, key):
        """Two steps (state set 0 -> 1 -> 0) captured once per (forced, logits) mode."""
        if key in self._graphs:
            return self._graphs[key]
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):          # warm-up outside capture: buffers of the LSTM handles grow here
            self._step(self.state[0], self.state[1])
            self._step(self.state[1], self.state[0])
        torch.cuda.current_stream(self.dev).wait_stream(side)
        torch.cuda.synchronize(self.dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            n = self._step(self.state[0], self.state[1])
            self._step(self.state[1], self.state[0])
        self.launches_per_step = n
        self._graphs[key] = g
        return g

    def decode(self, steps: int, forced: Optional[torch.Tensor] = None, want_logits: bool = False):
        """Greedy decode of the encoded group for `steps` steps (rounded up to an even count internally).  Returns the
        token table [steps, G] (device, int64) and, when asked, the logits [steps, G, V]."""
        cfg, G = self.cfg, self.G
        steps2 = steps + (steps & 1)
        if steps2 > cfg.max_steps + (cfg.max_steps & 1) or steps2 > self.toks_out.shape[0] + 1:
            raise ValueError("more steps than the configuration's maximum")
        if self.toks_out.shape[0] < steps2:
            self.toks_out = torch.zeros(steps2, G, dtype=torch.int64, device=self.dev)
            self._graphs.clear()
        if forced is not None:
            f = torch.zeros(steps2, G, dtype=torch.int64, device=self.dev)
            f[:steps] = forced.to(self.dev)
            if self.forced is None or self.forced.shape != f.shape:
                self.forced = f
                self._graphs.clear()
            else:
                self.forced.copy_(f)
        elif self.forced is not None:
            self.forced = None
            self._graphs.clear()
        if want_logits and (self.logits_out is None or self.logits_out.shape[0] < steps2):
            self.logits_out = torch.zeros(steps2, G, self.V, dtype=torch.float16, device=self.dev)
            self._graphs.clear()
        if not want_logits and self.logits_out is not None:
            self.logits_out = None
            self._graphs.clear()
        g = self._graph((forced is not None, want_logits))
        for s in self.state[0]:
            s.zero_()
        self.tok.fill_(cfg.bos)
        self.step_idx.zero_()
        for _ in range(steps2 // 2):
            g.replay()
        toks = self.toks_out[:steps]
        return (toks, self.logits_out[:steps]) if want_logits else (toks, None)

    # ------------------------------------------------------------------------------------------------ user call
    def stage(self, sentences: Sequence[torch.Tensor]):
        """Sorts the sentences by length and packs them into lock-step groups (see stage_groups)."""
        return stage_groups(sentences, self.G, self.ENC_BATCH, self.S, pin=True)

    def to_device(self, group: dict) -> dict:
        """The group's tensors copied to the device (batch_sizes stays on the host, as aten::lstm takes it)."""
        mv = lambda t: t.to(self.dev, non_blocking=True)
        return {"idx": group["idx"], "S": group["S"], "lengths": mv(group["lengths"]),
                "slices": [{"ids": mv(sl["ids"]), "dst": mv(sl["dst"]), "batch_sizes": sl["batch_sizes"]} for sl in group["slices"]]}

    def h2d_bytes(self, group: dict) -> int:
        return 8 * (group["lengths"].numel() + sum(sl["ids"].numel() + sl["dst"].numel() for sl in group["slices"]))

    def run_group(self, group_dev: dict, steps: int, forced: Optional[torch.Tensor] = None, want_logits: bool = False):
        """Encoder + greedy decode of one staged group whose tensors are already on the device."""
        self.encode(group_dev)
        return self.decode(steps, forced, want_logits)

    def check_status(self) -> None:
        """Raises if a bounded device-side wait of a recurrence or of the tensor-core GEMM gave up since the last check
        (the launches that followed have run, but the results of the one that gave up are not valid)."""
        from . import _lib
        bad = [name for name, h in self.lstm.items() if h.last_status() != 0]
        rc = _lib.lib().pimb200_gemm_last_status()
        if bad or rc != 0:
            raise RuntimeError(f"device-side wait timed out (recurrences: {bad}, gemm status {rc})")

    def translate(self, sentences: Sequence[torch.Tensor], steps: Optional[int] = None,
                  forced: Optional[Sequence[Sequence[int]]] = None, want_logits: bool = False):
        """sentences: 1-D int64 CPU tensors of source token ids.  Returns one token list per sentence (cut behind the
        first end-of-sentence token unless `steps` is given, which decodes exactly that many steps) and, when asked,
        the logits [steps, V] of each."""
        cfg, G = self.cfg, self.G
        n = len(sentences)
        run_steps = cfg.max_steps if steps is None else steps
        out_toks: List[Optional[List[int]]] = [None] * n
        out_logits: List[Optional[torch.Tensor]] = [None] * n
        pending = []
        for group in self.stage(sentences):
            idx = group["idx"]
            f = None
            if forced is not None:
                f = torch.zeros(run_steps, G, dtype=torch.int64)
                for j, i in enumerate(idx):
                    f[:, j] = torch.tensor(list(forced[i])[:run_steps], dtype=torch.int64)
            toks, logits = self.run_group(self.to_device(group), run_steps, f, want_logits)
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
