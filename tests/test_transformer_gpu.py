"""GPU: Transformer greedy translation (configuration C5) for groups of sequences in lock step against the libtorch-CPU
fp32 oracle run sequence by sequence (oracle/torch_oracle.py transformer_translate): padded encoder batches with ragged
lengths, the key / value cache written in place, single-query attention, vocabulary projection, over every step."""
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _translator(cfg, w, group):
    from pimaicompiler_b200.transformer import TransformerTranslator
    return TransformerTranslator(cfg, w, group=group)


def _follow(cfg, w, seqs, group, steps, atol, rtol, min_margin):
    ref = [to.transformer_translate(w, s, cfg, steps) for s in seqs]
    tr = _translator(cfg, w, group)
    toks, logits = tr.translate(seqs, steps=steps, forced=[r[0] for r in ref], want_logits=True)
    decided, worst = 0, 0.0
    for i, (rt, rl) in enumerate(ref):
        worst = max(worst, float((logits[i] - rl).abs().max()))
        assert_close(logits[i], rl, atol, rtol, f"logits of sequence {i} ({len(seqs[i])} tokens)")
        top2 = torch.topk(rl, 2, dim=1).values
        margin = (top2[:, 0] - top2[:, 1]).numpy()
        for t in range(steps):
            if margin[t] > min_margin:
                assert toks[i][t] == rt[t], f"sequence {i} step {t}: token {toks[i][t]} vs {rt[t]} at margin {margin[t]:.4f}"
                decided += 1
    print(f"largest logit error {worst:.4f}; tokens compared at a clear margin: {decided} of {len(ref) * steps}")
    return decided, len(ref) * steps


@pytest.mark.parametrize("group", [4, 8])
def test_transformer_small_model_ragged_groups(group):
    cfg = to.TransformerConfig(vocab=200, d_model=64, heads=4, ffn=128, layers=2, max_steps=10, min_len=3, max_len=9)
    w = to.make_transformer_weights(cfg, seed=3, gain=1.5, logit_gain=4.0)
    seqs = to.make_sentences(11, cfg, seed=5)
    decided, total = _follow(cfg, w, seqs, group, 10, 2e-2, 2e-2, 0.1)
    assert decided > total // 3


def test_transformer_free_running_and_repeatable():
    cfg = to.TransformerConfig(vocab=200, d_model=64, heads=4, ffn=128, layers=2, max_steps=12, min_len=3, max_len=9)
    w = to.make_transformer_weights(cfg, seed=4, gain=1.5, logit_gain=8.0)
    seqs = to.make_sentences(9, cfg, seed=6)
    tr = _translator(cfg, w, 8)
    toks = tr.translate(seqs, steps=12)
    assert tr.translate(seqs, steps=12) == toks
    compared = 0
    for i, s in enumerate(seqs):
        rt, rl = to.transformer_translate(w, s, cfg, 12)
        top2 = torch.topk(rl, 2, dim=1).values
        if float((top2[:, 0] - top2[:, 1]).min()) < 0.1:
            continue
        assert toks[i] == rt
        compared += 1
    assert compared >= 2
    cut = tr.translate(seqs)
    for full, c in zip(toks, cut):
        assert c == (full[:full.index(cfg.eos) + 1] if cfg.eos in full else full)


def test_transformer_benchmark_configuration_full_length():
    # the benchmark's sizes (6 + 6 layers, width 512, 8 heads, vocabulary 32000, sources of 16..64 tokens) over all 64
    # steps for five sequences decoded in one lock-step group of 32 (the rest of the group is padding)
    cfg = to.TransformerConfig()
    w = to.make_transformer_weights(cfg, seed=1, logit_gain=4.0)
    seqs = to.make_sentences(5, cfg, seed=2)
    decided, total = _follow(cfg, w, seqs, 32, cfg.max_steps, 3e-2, 2e-2, 0.1)
    assert decided > total // 5
