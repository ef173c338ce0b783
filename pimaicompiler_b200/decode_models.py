"""GNMT-style and Transformer-style greedy decode steps written once against a small backend interface: `PimBackend`
runs every op on the device through the C ABI (fp16); the parity tests run the same model code on a libtorch-CPU fp32
backend of their own (tests/cpu_backend.py).

Random-init weights of the benchmark's architectures (C4: 4-layer LSTM decoder with normalised Bahdanau attention and a
vocabulary projection; C5: Transformer decoder layers with a KV cache); the corpora and checkpoints are not available
offline.  The hot ops (lstm with seq_len 1, batch-1 linear with fused ReLU, fp16 add, single-row bmm, cat / KV append)
and the glue around them (tanh, softmax, layer norm, arg max, single-query multi-head attention) go through the
backend.
"""
from __future__ import annotations

import math

import torch


def u(shape, fan_in, gen, gain=1.0):
    k = gain / math.sqrt(fan_in)
    return ((torch.rand(*shape, generator=gen) * 2 - 1) * k).to(torch.float16).to(torch.float32)


class PimBackend:
    """fp16 device ops through libpimb200.so."""
    dev, dtype = "cuda", torch.float16

    def __init__(self):
        from pimaicompiler_b200 import ops
        self.ops = ops
        ops.init()
        self._lstm = {}

    def put(self, t):
        return t.to(torch.float16).cuda().contiguous()

    def linear(self, x, W, b=None, relu=False, out=None):
        o = self.ops
        if x.dim() == 1:
            return o.gemv_mv(W, x.contiguous(), b, o.ACT_RELU if relu else o.ACT_NONE, out=out)
        return o.gemm_wx(W, x.contiguous(), b, o.ACT_RELU if relu else o.ACT_NONE, out=out)

    def lstm_cell_stack(self, key, x, h, c, params, layers):
        if key not in self._lstm:
            self._lstm[key] = self.ops.Lstm(params, layers, False, params[0].shape[1], params[1].shape[1], True)
        y, hn, cn = self._lstm[key].forward(x.view(1, 1, -1).contiguous(), h.contiguous(), c.contiguous())
        return y.view(-1), hn, cn

    def add(self, a, b):
        return self.ops.add_f16(a.contiguous(), b.contiguous())

    def bmm_row(self, x, A):
        return self.ops.bmm_row(x.contiguous(), A.contiguous())

    def cat(self, ts, dim):
        return self.ops.cat([t.contiguous() for t in ts], dim)

    def kv_new(self, steps, d):
        # pre-allocated [S_max, d] buffer; entries are written in place, the live prefix is a view
        self._kv_full = getattr(self, "_kv_full", {})
        buf = torch.zeros(steps, d, dtype=torch.float16, device="cuda")
        view = buf[:0]
        self._kv_full[id(view)] = buf
        return view

    def kv_append(self, cache, t, row):
        buf = self._kv_full.pop(id(cache))
        d = buf.shape[1]
        self.ops.copy_2d(buf, t * d * 2, d * 2, row.contiguous(), 0, d * 2, d * 2, 1)   # one row at offset t
        view = buf[: t + 1]
        self._kv_full[id(view)] = buf
        return view

    def attend(self, q, K, Vv, heads):
        return self.ops.attention_row(q.contiguous(), K.contiguous(), Vv.contiguous(), heads)

    def tanh(self, x):
        return self.ops.tanh(x.contiguous())

    def softmax(self, x):
        return self.ops.softmax(x.contiguous())

    def layer_norm(self, x):
        return self.ops.layer_norm(x.contiguous().view(1, -1)).view(x.shape)

    def argmax(self, x):
        return int(self.ops.argmax(x.contiguous().view(1, -1)).item())


# ------------------------------------------------------------------------------------------------ GNMT-style decoder
def make_gnmt(H, V, src_len, gen, gain=1.0):
    w = {"emb": torch.randn(V, H, generator=gen).half().float() * 0.5,
         "keys": torch.tanh(torch.randn(src_len, H, generator=gen)).half().float(),   # encoder states
         "Wq": u((H, H), H, gen, gain), "Wk": u((H, H), H, gen, gain), "att_b": u((H,), H, gen, gain),
         "att_v": u((H,), H, gen, gain), "att_g": torch.tensor(1.0),
         "Wc": u((V, H), H, gen, gain), "bc": u((V,), H, gen, gain)}
    for l in range(4):
        I = H if l == 0 else 2 * H
        w[f"l{l}"] = [u((4 * H, I), H, gen, gain), u((4 * H, H), H, gen, gain), u((4 * H,), H, gen, gain),
                      u((4 * H,), H, gen, gain)]
    return w


def gnmt_greedy(be, w, H, steps, bos=2, forced=None):
    """Returns (token ids, logits [steps, V]).  One decoder step: LSTM1 -> attention context -> cat -> 3 LSTMs with
    residual adds -> vocabulary projection -> argmax; `forced[t]` overrides the fed-back token ("follow" mode)."""
    W = {k: ([be.put(t) for t in v] if isinstance(v, list) else be.put(v)) for k, v in w.items()}
    keys_proj = be.linear(W["keys"], W["Wk"])                               # [S, H], once per sentence
    v_norm = be.put(w["att_v"] / w["att_v"].norm() * float(w["att_g"]))       # normalised Bahdanau score vector
    hs = [torch.zeros(1, 1, H, dtype=be.dtype, device=be.dev) for _ in range(4)]
    cs = [torch.zeros(1, 1, H, dtype=be.dtype, device=be.dev) for _ in range(4)]
    tok, toks, logits = bos, [], []
    for t in range(steps):
        x = W["emb"][tok]
        y0, hs[0], cs[0] = be.lstm_cell_stack("l0", x, hs[0], cs[0], W["l0"], 1)
        q = be.linear(y0, W["Wq"])
        scores = be.tanh(be.add(keys_proj, be.add(q, W["att_b"])))          # [S, H]: row broadcast add, tanh
        e = be.linear(v_norm, scores)                                       # [S] = scores . v
        att = be.softmax(e)
        ctx = be.bmm_row(att, W["keys"])                                    # [H]
        x1 = be.cat([y0.view(1, H), ctx.view(1, H)], 1).view(-1)            # the {1,1,2048} buffer of the reference
        y1, hs[1], cs[1] = be.lstm_cell_stack("l1", x1, hs[1], cs[1], W["l1"], 1)
        x2 = be.cat([y1.view(1, H), ctx.view(1, H)], 1).view(-1)
        y2, hs[2], cs[2] = be.lstm_cell_stack("l2", x2, hs[2], cs[2], W["l2"], 1)
        r2 = be.add(y2, y1)                                                 # residual connections
        x3 = be.cat([r2.view(1, H), ctx.view(1, H)], 1).view(-1)
        y3, hs[3], cs[3] = be.lstm_cell_stack("l3", x3, hs[3], cs[3], W["l3"], 1)
        r3 = be.add(y3, r2)
        lgd = be.linear(r3, W["Wc"], W["bc"])
        logits.append(lgd.float().cpu())
        best = be.argmax(lgd)
        toks.append(best)
        tok = best if forced is None else int(forced[t])
    return toks, torch.stack(logits)


def gnmt_greedy_graph(w, H, steps, bos=2):
    """The same decode with the whole step resident on the device: arg max writes the chosen token's int64 index into
    device memory, the next step gathers its embedding row by that index, the recurrent states ping-pong between two
    sets of fixed buffers, and the step (about 25 launches) is captured in two CUDA graphs replayed alternately.  Nothing is read back until the
    sentence is done, where the reference's interpreter synchronises at least once per token
    (aten_ops_executor.cpp:1276-1287).  Returns (token ids, logits [steps, V], the graph replays' device time in us)."""
    be = PimBackend()
    ops = be.ops
    W = {k: ([be.put(t) for t in v] if isinstance(v, list) else be.put(v)) for k, v in w.items()}
    keys_proj = be.linear(W["keys"], W["Wk"])
    v_norm = be.put(w["att_v"] / w["att_v"].norm() * float(w["att_g"]))
    V = W["Wc"].shape[0]
    tok = torch.full((1,), bos, dtype=torch.int64, device="cuda")
    # recurrent states ping-pong between two sets of buffers (an LSTM call must not write the state it reads), so the
    # step exists as two graphs, one per direction
    hs = [[torch.zeros(1, 1, H, dtype=torch.float16, device="cuda") for _ in range(4)] for _ in range(2)]
    cs = [[torch.zeros(1, 1, H, dtype=torch.float16, device="cuda") for _ in range(4)] for _ in range(2)]
    ys = [torch.zeros(1, 1, H, dtype=torch.float16, device="cuda") for _ in range(4)]
    toks_dev = torch.zeros(steps, dtype=torch.int64, device="cuda")
    logits_dev = torch.zeros(steps, V, dtype=torch.float16, device="cuda")

    def cell(key, x, i, src, dst):
        if key not in be._lstm:
            p = W[key]
            be._lstm[key] = ops.Lstm(p, 1, False, p[0].shape[1], p[1].shape[1], True)
        be._lstm[key].forward(x.view(1, 1, -1), hs[src][i], cs[src][i], out=(ys[i], hs[dst][i], cs[dst][i]))
        return ys[i].view(-1)

    def step(src, dst, t_out):
        x = ops.gather_rows(W["emb"], tok).view(-1)                         # embedding lookup by a device-side index
        y0 = cell("l0", x, 0, src, dst)
        q = be.linear(y0, W["Wq"])
        scores = be.tanh(be.add(keys_proj, be.add(q, W["att_b"])))
        att = be.softmax(be.linear(v_norm, scores))
        ctx = be.bmm_row(att, W["keys"])
        y1 = cell("l1", be.cat([y0.view(1, H), ctx.view(1, H)], 1).view(-1), 1, src, dst)
        y2 = cell("l2", be.cat([y1.view(1, H), ctx.view(1, H)], 1).view(-1), 2, src, dst)
        r2 = be.add(y2, y1)
        y3 = cell("l3", be.cat([r2.view(1, H), ctx.view(1, H)], 1).view(-1), 3, src, dst)
        r3 = be.add(y3, r2)
        lgd = be.linear(r3, W["Wc"], W["bc"], out=t_out)
        ops.argmax(lgd.view(1, -1), out=tok)                                # the token stays on the device

    lg_buf = torch.zeros(V, dtype=torch.float16, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):          # one eager step: handle creation and workspace growth happen outside capture
        step(0, 1, lg_buf)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graphs = []
    for src in (0, 1):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step(src, 1 - src, lg_buf)
        graphs.append(g)
    tok.fill_(bos)
    for t in hs[0] + cs[0]:
        t.zero_()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for t in range(steps):
        graphs[t & 1].replay()
        toks_dev[t:t + 1].copy_(tok)       # device-to-device; no host synchronisation inside the loop
        logits_dev[t].copy_(lg_buf)
    e1.record()
    torch.cuda.synchronize()
    return toks_dev.cpu().tolist(), logits_dev.float().cpu(), e0.elapsed_time(e1) * 1e3


# ------------------------------------------------------------------------------------ Transformer-style decoder
def make_transformer(d, heads, ffn, V, layers, src_len, gen, gain=1.0):
    w = {"emb": torch.randn(V, d, generator=gen).half().float() * 0.3, "Wo": u((V, d), d, gen, gain),
         "mem": torch.randn(src_len, d, generator=gen).half().float() * 0.5, "layers": []}
    for _ in range(layers):
        L = {}
        for name in ("sq", "sk", "sv", "so", "cq", "ck", "cv", "co"):
            L[name] = u((d, d), d, gen, gain)
            L[name + "_b"] = u((d,), d, gen, gain)
        L["f1"], L["f1_b"] = u((ffn, d), d, gen, gain), u((ffn,), d, gen, gain)
        L["f2"], L["f2_b"] = u((d, ffn), ffn, gen, gain), u((d,), ffn, gen, gain)
        w["layers"].append(L)
    return w


def transformer_greedy(be, w, d, heads, steps, bos=1, forced=None):
    ln = be.layer_norm
    P = lambda t: be.put(t)
    emb, Wo, mem = P(w["emb"]), P(w["Wo"]), P(w["mem"])
    Ls = [{k: P(v) for k, v in L.items()} for L in w["layers"]]
    cross = [(be.linear(mem, L["ck"], L["ck_b"]), be.linear(mem, L["cv"], L["cv_b"])) for L in Ls]
    kcache = [be.kv_new(steps, d) for _ in Ls]
    vcache = [be.kv_new(steps, d) for _ in Ls]
    tok, toks, logits = bos, [], []
    for t in range(steps):
        x = emb[tok]
        for i, L in enumerate(Ls):
            q = be.linear(x, L["sq"], L["sq_b"])
            k = be.linear(x, L["sk"], L["sk_b"])
            v = be.linear(x, L["sv"], L["sv_b"])
            kcache[i] = be.kv_append(kcache[i], t, k)      # KV append
            vcache[i] = be.kv_append(vcache[i], t, v)
            a = be.attend(q, kcache[i], vcache[i], heads)
            x = ln(be.add(x, be.linear(a, L["so"], L["so_b"])))
            cq = be.linear(x, L["cq"], L["cq_b"])
            ca = be.attend(cq, cross[i][0], cross[i][1], heads)
            x = ln(be.add(x, be.linear(ca, L["co"], L["co_b"])))
            f = be.linear(be.linear(x, L["f1"], L["f1_b"], relu=True), L["f2"], L["f2_b"])
            x = ln(be.add(x, f))
        lgd = be.linear(x, Wo)
        logits.append(lgd.float().cpu())
        best = be.argmax(lgd)
        toks.append(best)
        tok = best if forced is None else int(forced[t])
    return toks, torch.stack(logits)


def transformer_greedy_graph(w, d, heads, steps, bos=1):
    """The Transformer decode step resident on the device: token and position live in device memory (arg max writes the
    token, the embedding is gathered by it, keys and values are appended in place at the device-side position into
    pre-allocated [S_max, d] caches), self-attention reads the attended length from the device-side position, and the
    step is one CUDA graph replayed `steps` times.  Returns (token ids, logits, device us)."""
    be = PimBackend()
    ops = be.ops
    P = be.put
    emb, Wo, mem = P(w["emb"]), P(w["Wo"]), P(w["mem"])
    Ls = [{k: P(v) for k, v in L.items()} for L in w["layers"]]
    cross = [(be.linear(mem, L["ck"], L["ck_b"]), be.linear(mem, L["cv"], L["cv_b"])) for L in Ls]
    S_max, V = steps, Wo.shape[0]
    kc = [torch.zeros(S_max, d, dtype=torch.float16, device="cuda") for _ in Ls]
    vc = [torch.zeros(S_max, d, dtype=torch.float16, device="cuda") for _ in Ls]
    tok = torch.full((1,), bos, dtype=torch.int64, device="cuda")
    pos = torch.zeros(1, dtype=torch.int64, device="cuda")
    lg_buf = torch.zeros(V, dtype=torch.float16, device="cuda")
    toks_dev = torch.zeros(steps, dtype=torch.int64, device="cuda")
    logits_dev = torch.zeros(steps, V, dtype=torch.float16, device="cuda")

    def step():
        x = ops.gather_rows(emb, tok).view(-1)
        for i, L in enumerate(Ls):
            q = be.linear(x, L["sq"], L["sq_b"])
            ops.scatter_rows(kc[i], pos, be.linear(x, L["sk"], L["sk_b"]).view(1, d))      # KV append in place
            ops.scatter_rows(vc[i], pos, be.linear(x, L["sv"], L["sv_b"]).view(1, d))
            a = ops.attention_row(q, kc[i], vc[i], heads, length_dev=pos, length_add=1)   # entries 0..pos
            x = be.layer_norm(be.add(x, be.linear(a, L["so"], L["so_b"])))
            cq = be.linear(x, L["cq"], L["cq_b"])
            ca = be.attend(cq, cross[i][0], cross[i][1], heads)
            x = be.layer_norm(be.add(x, be.linear(ca, L["co"], L["co_b"])))
            f = be.linear(be.linear(x, L["f1"], L["f1_b"], relu=True), L["f2"], L["f2_b"])
            x = be.layer_norm(be.add(x, f))
        lgd = be.linear(x, Wo, out=lg_buf)
        ops.argmax(lgd.view(1, -1), out=tok)
        pos.add_(1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                              # eager once: workspaces and the split-K scratch exist before capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    tok.fill_(bos)
    pos.zero_()
    for c in kc + vc:
        c.zero_()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for t in range(steps):
        g.replay()
        toks_dev[t:t + 1].copy_(tok)
        logits_dev[t].copy_(lg_buf)
    e1.record()
    torch.cuda.synchronize()
    return toks_dev.cpu().tolist(), logits_dev.float().cpu(), e0.elapsed_time(e1) * 1e3
