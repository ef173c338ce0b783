"""Seeded synthetic workloads of the benchmark configurations.

The models the reference is normally run on (RNN-T, GNMT, Transformer checkpoints) and their corpora are
not available offline, so the benchmark and the parity tests use random-init weights of the stated
architectures and N(0,1) features.  Everything is generated on the CPU as fp32 tensors holding
fp16-representable values, so the fp16 device path and the fp32 CPU oracle consume identical numbers.
"""
from __future__ import annotations

import math
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


class _RnntModule(torch.nn.Module):
    """Container with the parameter names PipelineManager('...', 'RNNT') looks for.  forward() is the encoder only
    (the greedy loop of the benchmark is data-dependent control flow; the reference interprets it op by op)."""

    def __init__(self, cfg: RnntConfig):
        super().__init__()
        self.pre_rnn = torch.nn.LSTM(cfg.feat_dim, cfg.enc_hidden, cfg.pre_layers)
        self.post_rnn = torch.nn.LSTM(cfg.stack_factor * cfg.enc_hidden, cfg.enc_hidden, cfg.post_layers)
        self.pred_embed = torch.nn.Embedding(cfg.vocab, cfg.pred_hidden)
        self.pred_rnn = torch.nn.LSTM(cfg.pred_hidden, cfg.pred_hidden, cfg.pred_layers)
        self.joint1 = torch.nn.Linear(cfg.enc_hidden + cfg.pred_hidden, cfg.joint_hidden)
        self.joint2 = torch.nn.Linear(cfg.joint_hidden, cfg.vocab)
        self.stack = cfg.stack_factor

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y, _ = self.pre_rnn(x)
        T, B, H = y.shape
        Tp = T // self.stack
        y = y[: Tp * self.stack].transpose(0, 1).reshape(B, Tp, self.stack * H).transpose(0, 1)
        y, _ = self.post_rnn(y.contiguous())
        return y


def save_rnnt_torchscript(path: str, cfg: RnntConfig, w: RnntWeights) -> None:
    """Writes a TorchScript file holding the synthetic RNN-T weights under the names PipelineManager reads."""
    m = _RnntModule(cfg)
    sd = {}
    for prefix, ps, layers in (("pre_rnn", w.pre, cfg.pre_layers), ("post_rnn", w.post, cfg.post_layers),
                               ("pred_rnn", w.pred, cfg.pred_layers)):
        for l in range(layers):
            for k, name in enumerate(("weight_ih", "weight_hh", "bias_ih", "bias_hh")):
                sd[f"{prefix}.{name}_l{l}"] = ps[4 * l + k]
    sd["pred_embed.weight"] = w.embedding
    sd["joint1.weight"], sd["joint1.bias"] = w.w1, w.b1
    sd["joint2.weight"], sd["joint2.bias"] = w.w2, w.b2
    m.load_state_dict(sd)
    torch.jit.script(m).save(path)


# ------------------------------------------------------------------------------------------------ GNMT (configuration C4)
@dataclass
class GnmtConfig:
    """4-layer LSTM encoder (first layer bidirectional, residual connections from the third layer), 4-layer LSTM
    decoder with normalised Bahdanau attention fed by the first decoder layer, vocabulary projection; greedy search."""
    vocab: int = 32320
    hidden: int = 1024
    max_steps: int = 80
    min_len: int = 20
    max_len: int = 50
    bos: int = 2
    eos: int = 3


def make_gnmt_weights(cfg: GnmtConfig, seed: int = 0, gain: float = 1.0, logit_gain: float = 1.0) -> dict:
    """fp32 CPU tensors with fp16-representable values: U(-1/sqrt(fan_in), 1/sqrt(fan_in)) matrices, N(0, 0.5) embeddings."""
    g = torch.Generator().manual_seed(seed)
    H, V = cfg.hidden, cfg.vocab

    def lstm(I):
        return [_u((4 * H, I), H, g, gain), _u((4 * H, H), H, g, gain), _u((4 * H,), H, g, gain), _u((4 * H,), H, g, gain)]

    w = {"emb_src": (torch.randn(V, H, generator=g) * 0.5).half().float(),
         "emb_tgt": (torch.randn(V, H, generator=g) * 0.5).half().float(),
         "enc0_f": lstm(H), "enc0_r": lstm(H), "enc1": lstm(2 * H), "enc2": lstm(H), "enc3": lstm(H),
         "dec0": lstm(H), "dec1": lstm(2 * H), "dec2": lstm(2 * H), "dec3": lstm(2 * H),
         "Wq": _u((H, H), H, g, gain), "Wk": _u((H, H), H, g, gain), "att_b": _u((H,), H, g, gain),
         "att_v": _u((H,), H, g, gain), "att_g": torch.tensor(1.0),
         "Wc": _u((V, H), H, g, logit_gain), "bc": _u((V,), H, g, logit_gain)}
    return w


def make_sentences(n: int, cfg: GnmtConfig, seed: int) -> List[torch.Tensor]:
    """n source sentences: lengths U[min_len, max_len], token ids U[4, vocab)."""
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(cfg.min_len, cfg.max_len + 1, (n,), generator=g)
    return [torch.randint(4, cfg.vocab, (int(L),), generator=g) for L in lens]


# ------------------------------------------------------------------------------------------------ Transformer (configuration C5)
@dataclass
class TransformerConfig:
    """Transformer-base: 6 encoder + 6 decoder layers (post-norm, no affine parameters in the layer norms), model width
    512, 8 heads, feed-forward width 2048, sinusoidal positions, greedy search with a key / value cache."""
    vocab: int = 32000
    d_model: int = 512
    heads: int = 8
    ffn: int = 2048
    layers: int = 6
    max_steps: int = 64
    min_len: int = 16
    max_len: int = 64
    bos: int = 1
    eos: int = 2


def positional_table(n: int, d: int) -> torch.Tensor:
    """Sinusoidal position encodings [n, d], fp16-representable."""
    pos = torch.arange(n, dtype=torch.float32).unsqueeze(1)
    inv = torch.exp(torch.arange(0, d, 2, dtype=torch.float32) * (-math.log(10000.0) / d))
    pe = torch.zeros(n, d)
    pe[:, 0::2] = torch.sin(pos * inv)
    pe[:, 1::2] = torch.cos(pos * inv)
    return pe.to(torch.float16).to(torch.float32)


def make_transformer_weights(cfg: TransformerConfig, seed: int = 0, gain: float = 1.0, logit_gain: float = 1.0) -> dict:
    g = torch.Generator().manual_seed(seed)
    d, f, V = cfg.d_model, cfg.ffn, cfg.vocab

    def lin(n_out, n_in, gn=gain):
        return _u((n_out, n_in), n_in, g, gn), _u((n_out,), n_in, g, gn)

    def layer(cross: bool):
        L = {}
        names = ("sq", "sk", "sv", "so") + (("cq", "ck", "cv", "co") if cross else ())
        for name in names:
            L[name], L[name + "_b"] = lin(d, d)
        L["f1"], L["f1_b"] = lin(f, d)
        L["f2"], L["f2_b"] = lin(d, f)
        return L

    return {"emb_src": (torch.randn(V, d, generator=g) * 0.3).half().float(),
            "emb_tgt": (torch.randn(V, d, generator=g) * 0.3).half().float(),
            "pe": positional_table(max(cfg.max_len, cfg.max_steps), d),
            "enc": [layer(False) for _ in range(cfg.layers)], "dec": [layer(True) for _ in range(cfg.layers)],
            "Wo": _u((V, d), d, g, logit_gain)}
