"""libtorch-CPU oracle: the very library calls the reference's default executors make for this path
(at::lstm, at::linear/addmm/matmul, at::cat; runtime/source/executor/op_executor/aten_ops.cpp:47-51,
97, 304-307, 328-344, 362), driven from Python, fp32, on the host cores.

Test infrastructure and the benchmark's CPU arm only; the product package never imports this.
Also holds the seeded synthetic RNN-T model (random-init weights of the benchmark's architecture;
the real checkpoints and speech corpora are not available offline).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class RnntConfig:
    feat_dim: int = 240
    enc_hidden: int = 1024
    pre_layers: int = 2
    post_layers: int = 3
    stack_factor: int = 2
    pred_hidden: int = 320
    pred_layers: int = 2
    joint_hidden: int = 512
    vocab: int = 29
    blank: int = 28
    max_symbols: int = 1


@dataclass
class RnntWeights:
    """fp32 CPU tensors whose values are fp16-representable (both sides of a parity test use them)."""
    pre: List[torch.Tensor] = field(default_factory=list)
    post: List[torch.Tensor] = field(default_factory=list)
    embedding: Optional[torch.Tensor] = None
    pred: List[torch.Tensor] = field(default_factory=list)
    w1: Optional[torch.Tensor] = None
    b1: Optional[torch.Tensor] = None
    w2: Optional[torch.Tensor] = None
    b2: Optional[torch.Tensor] = None


def _u(shape, fan_in, gen, gain=1.0):
    k = gain / fan_in ** 0.5
    return ((torch.rand(*shape, generator=gen) * 2 - 1) * k).to(torch.float16).to(torch.float32)


def _lstm_params(L, I, H, gen, gain=1.0):
    ps = []
    for l in range(L):
        Il = I if l == 0 else H
        ps += [_u((4 * H, Il), H, gen, gain), _u((4 * H, H), H, gen, gain), _u((4 * H,), H, gen, gain),
               _u((4 * H,), H, gen, gain)]
    return ps


def make_rnnt_weights(cfg: RnntConfig, seed: int = 0, gain: float = 1.0, logit_gain: float = 1.0) -> RnntWeights:
    """U(-1/sqrt(fan_in), 1/sqrt(fan_in)) init (PyTorch's default for LSTM/Linear), N(0,1) embedding.
    `gain`/`logit_gain` > 1 widen the distributions so tests can get a mix of blank and label decisions."""
    g = torch.Generator().manual_seed(seed)
    w = RnntWeights()
    w.pre = _lstm_params(cfg.pre_layers, cfg.feat_dim, cfg.enc_hidden, g, gain)
    w.post = _lstm_params(cfg.post_layers, cfg.stack_factor * cfg.enc_hidden, cfg.enc_hidden, g, gain)
    w.embedding = torch.randn(cfg.vocab, cfg.pred_hidden, generator=g).to(torch.float16).to(torch.float32)
    w.pred = _lstm_params(cfg.pred_layers, cfg.pred_hidden, cfg.pred_hidden, g, gain)
    fan1 = cfg.enc_hidden + cfg.pred_hidden
    w.w1 = _u((cfg.joint_hidden, fan1), fan1, g, gain)
    w.b1 = _u((cfg.joint_hidden,), fan1, g, gain)
    w.w2 = _u((cfg.vocab, cfg.joint_hidden), cfg.joint_hidden, g, gain * logit_gain)
    w.b2 = _u((cfg.vocab,), cfg.joint_hidden, g, gain * logit_gain)
    return w


def make_features(T: int, cfg: RnntConfig, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, cfg.feat_dim, generator=g).to(torch.float16).to(torch.float32)


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
