"""libtorch-CPU oracle: the very library calls the reference's default executors make for this path
(at::lstm, at::linear/addmm/matmul, at::cat; runtime/source/executor/op_executor/aten_ops.cpp:47-51,
97, 304-307, 328-344, 362), driven from Python, fp32, on the host cores.

Test infrastructure and the benchmark's CPU arm only; the product package never imports this.
The seeded synthetic RNN-T model it runs comes from pimaicompiler_b200.synthetic.
"""
from __future__ import annotations

from typing import List, Optional

import torch


from pimaicompiler_b200.synthetic import (GnmtConfig, RnntConfig, RnntWeights, TransformerConfig,  # noqa: F401,E402
                                          make_features, make_transformer_weights,
                                          make_gnmt_weights, make_rnnt_weights, make_sentences)


def rnnt_encoder(w: RnntWeights, feats: torch.Tensor, cfg: RnntConfig) -> torch.Tensor:
    T = feats.shape[0]
    z = torch.zeros(cfg.pre_layers, 1, cfg.enc_hidden)
    y1, _, _ = torch.lstm(feats.view(T, 1, -1), [z, z], w.pre, True, cfg.pre_layers, 0.0, False, False, False)
    Tp = T // cfg.stack_factor
    x2 = y1[: Tp * cfg.stack_factor].reshape(Tp, 1, cfg.stack_factor * cfg.enc_hidden)
    z2 = torch.zeros(cfg.post_layers, 1, cfg.enc_hidden)
    y2, _, _ = torch.lstm(x2, [z2, z2], w.post, True, cfg.post_layers, 0.0, False, False, False)
    return y2.view(Tp, cfg.enc_hidden)


def rnnt_greedy(w: RnntWeights, feats: torch.Tensor, cfg: RnntConfig, forced: Optional[List[int]] = None):
    """Greedy decode (<= 1 symbol per frame).  Returns (tokens, logits [Tp,V], choice [Tp]).
    `forced[t]` (a label or cfg.blank) overrides the decision of frame t ("follow" mode)."""
    with torch.no_grad():
        enc = rnnt_encoder(w, feats, cfg)
        Tp = enc.shape[0]
        h = torch.zeros(cfg.pred_layers, 1, cfg.pred_hidden)
        c = torch.zeros_like(h)
        label = cfg.blank

        def pred(label, h, c):
            x = w.embedding[label].view(1, 1, -1)
            g, hn, cn = torch.lstm(x, [h, c], w.pred, True, cfg.pred_layers, 0.0, False, False, False)
            return g.view(-1), hn, cn

        g, hp, cp = pred(label, h, c)
        tokens, logits, choice = [], torch.empty(Tp, cfg.vocab), []
        for t in range(Tp):
            z = torch.relu(torch.nn.functional.linear(torch.cat([enc[t], g]), w.w1, w.b1))
            lg = torch.nn.functional.linear(z, w.w2, w.b2)
            logits[t] = lg
            best = int(torch.argmax(lg))
            choice.append(best)
            k = best if forced is None else int(forced[t])
            if k != cfg.blank:
                tokens.append(k)
                label, h, c = k, hp, cp
                g, hp, cp = pred(label, h, c)
        return tokens, logits, choice


# ------------------------------------------------------------------------------------------------ GNMT (configuration C4)
def gnmt_encode(w: dict, src: torch.Tensor, cfg) -> torch.Tensor:
    """Encoder states [S, H] of one sentence: at::lstm per layer (aten_ops.cpp:328-344), bidirectional first layer,
    residual adds from the third layer."""
    H = cfg.hidden
    S = src.shape[0]
    x = w["emb_src"][src].view(S, 1, H)
    z2, z1 = torch.zeros(2, 1, H), torch.zeros(1, 1, H)
    y0, _, _ = torch.lstm(x, [z2, z2], w["enc0_f"] + w["enc0_r"], True, 1, 0.0, False, True, False)
    y1, _, _ = torch.lstm(y0, [z1, z1], w["enc1"], True, 1, 0.0, False, False, False)
    y2, _, _ = torch.lstm(y1, [z1, z1], w["enc2"], True, 1, 0.0, False, False, False)
    y2 = y2 + y1
    y3, _, _ = torch.lstm(y2, [z1, z1], w["enc3"], True, 1, 0.0, False, False, False)
    return (y3 + y2).view(S, H)


def gnmt_translate(w: dict, src: torch.Tensor, cfg, steps: Optional[int] = None, forced: Optional[List[int]] = None):
    """Greedy decode of one sentence for `steps` steps (no stop at the end-of-sentence token: the caller truncates).
    Returns (tokens, logits [steps, V]); `forced[t]` overrides the token fed back after step t."""
    H = cfg.hidden
    steps = cfg.max_steps if steps is None else steps
    keys = gnmt_encode(w, src, cfg)
    keys_proj = torch.nn.functional.linear(keys, w["Wk"])
    v_norm = w["att_v"] / w["att_v"].norm() * float(w["att_g"])
    hs = [torch.zeros(1, 1, H) for _ in range(4)]
    cs = [torch.zeros(1, 1, H) for _ in range(4)]

    def cell(name, x, i):
        y, hs[i], cs[i] = torch.lstm(x.view(1, 1, -1), [hs[i], cs[i]], w[name], True, 1, 0.0, False, False, False)
        return y.view(-1)

    tok, toks, logits = cfg.bos, [], []
    for t in range(steps):
        y0 = cell("dec0", w["emb_tgt"][tok], 0)
        q = torch.nn.functional.linear(y0, w["Wq"])
        e = torch.tanh(keys_proj + q + w["att_b"]) @ v_norm
        ctx = torch.softmax(e, 0) @ keys
        y1 = cell("dec1", torch.cat([y0, ctx]), 1)
        r2 = cell("dec2", torch.cat([y1, ctx]), 2) + y1
        r3 = cell("dec3", torch.cat([r2, ctx]), 3) + r2
        lg = torch.nn.functional.linear(r3, w["Wc"], w["bc"])
        logits.append(lg)
        best = int(torch.argmax(lg))
        toks.append(best)
        tok = best if forced is None else int(forced[t])
    return toks, torch.stack(logits)


# ------------------------------------------------------------------------------------------------ Transformer (configuration C5)
def _mha(q, k, v, heads):
    """q [Tq, d], k / v [Tk, d] -> [Tq, d]: at::matmul -> softmax -> matmul per head."""
    Tq, d = q.shape
    hd = d // heads
    qh = q.view(Tq, heads, hd).transpose(0, 1)
    kh = k.view(-1, heads, hd).transpose(0, 1)
    vh = v.view(-1, heads, hd).transpose(0, 1)
    p = torch.softmax(qh @ kh.transpose(1, 2) / hd ** 0.5, -1)
    return (p @ vh).transpose(0, 1).reshape(Tq, d)


def _ln(x):
    return torch.nn.functional.layer_norm(x, x.shape[-1:])


def transformer_encode(w: dict, src: torch.Tensor, cfg) -> torch.Tensor:
    lin = torch.nn.functional.linear
    S = src.shape[0]
    x = w["emb_src"][src] + w["pe"][:S]
    for L in w["enc"]:
        a = _mha(lin(x, L["sq"], L["sq_b"]), lin(x, L["sk"], L["sk_b"]), lin(x, L["sv"], L["sv_b"]), cfg.heads)
        x = _ln(x + lin(a, L["so"], L["so_b"]))
        x = _ln(x + lin(torch.relu(lin(x, L["f1"], L["f1_b"])), L["f2"], L["f2_b"]))
    return x


def transformer_translate(w: dict, src: torch.Tensor, cfg, steps: Optional[int] = None, forced: Optional[List[int]] = None):
    """Greedy decode of one sequence with a key / value cache; returns (tokens, logits [steps, V])."""
    lin = torch.nn.functional.linear
    steps = cfg.max_steps if steps is None else steps
    mem = transformer_encode(w, src, cfg)
    cross = [(lin(mem, L["ck"], L["ck_b"]), lin(mem, L["cv"], L["cv_b"])) for L in w["dec"]]
    kc = [[] for _ in w["dec"]]
    vc = [[] for _ in w["dec"]]
    tok, toks, logits = cfg.bos, [], []
    for t in range(steps):
        x = (w["emb_tgt"][tok] + w["pe"][t]).view(1, -1)
        for i, L in enumerate(w["dec"]):
            kc[i].append(lin(x, L["sk"], L["sk_b"]))
            vc[i].append(lin(x, L["sv"], L["sv_b"]))
            a = _mha(lin(x, L["sq"], L["sq_b"]), torch.cat(kc[i]), torch.cat(vc[i]), cfg.heads)
            x = _ln(x + lin(a, L["so"], L["so_b"]))
            ca = _mha(lin(x, L["cq"], L["cq_b"]), cross[i][0], cross[i][1], cfg.heads)
            x = _ln(x + lin(ca, L["co"], L["co_b"]))
            x = _ln(x + lin(torch.relu(lin(x, L["f1"], L["f1_b"])), L["f2"], L["f2_b"]))
        lg = lin(x, w["Wo"]).view(-1)
        logits.append(lg)
        best = int(torch.argmax(lg))
        toks.append(best)
        tok = best if forced is None else int(forced[t])
    return toks, torch.stack(logits)
