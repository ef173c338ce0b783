"""libtorch-CPU oracle: the very library calls the reference's default executors make for this path
(at::lstm, at::linear/addmm/matmul, at::cat; runtime/source/executor/op_executor/aten_ops.cpp:47-51,
97, 304-307, 328-344, 362), driven from Python, fp32, on the host cores.

Test infrastructure and the benchmark's CPU arm only; the product package never imports this.
The seeded synthetic RNN-T model it runs comes from pimaicompiler_b200.synthetic.
"""
from __future__ import annotations

from typing import List, Optional

import torch


from pimaicompiler_b200.synthetic import RnntConfig, RnntWeights, make_features, make_rnnt_weights  # noqa: F401,E402


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
