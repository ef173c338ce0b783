"""GPU: GNMT greedy translation (configuration C4) for groups of sentences in lock step against the libtorch-CPU fp32
oracle run sentence by sentence (oracle/torch_oracle.py gnmt_translate): the encoder over ragged sentence lengths, the
batched decoder step, the attention kernel and the vocabulary projection, over every decode step."""
import numpy as np
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _translator(cfg, w, group):
    from pimaicompiler_b200.gnmt import GnmtTranslator
    return GnmtTranslator(cfg, w, group=group)


def _follow(cfg, w, sentences, group, steps, atol, rtol, min_margin):
    """Teacher-forced comparison: the oracle decodes freely, the device is fed the oracle's tokens; logits of every step
    are compared, and the chosen token wherever the oracle's top-2 margin exceeds the tolerance."""
    ref = [to.gnmt_translate(w, s, cfg, steps) for s in sentences]
    tr = _translator(cfg, w, group)
    toks, logits = tr.translate(sentences, steps=steps, forced=[r[0] for r in ref], want_logits=True)
    decided = 0
    worst = 0.0
    for i, (rt, rl) in enumerate(ref):
        worst = max(worst, float((logits[i] - rl).abs().max()))
        assert_close(logits[i], rl, atol, rtol, f"logits of sentence {i} ({len(sentences[i])} tokens)")
        top2 = torch.topk(rl, 2, dim=1).values
        margin = (top2[:, 0] - top2[:, 1]).numpy()
        for t in range(steps):
            if margin[t] > min_margin:
                assert toks[i][t] == rt[t], f"sentence {i} step {t}: token {toks[i][t]} vs {rt[t]} at margin {margin[t]:.4f}"
                decided += 1
    print(f"largest logit error {worst:.4f}; tokens compared at a clear margin: {decided} of {len(ref) * steps}")
    return decided, len(ref) * steps


@pytest.mark.parametrize("group", [4, 8])
def test_gnmt_small_model_ragged_groups(group):
    # 11 sentences of 3..17 tokens in groups of 4 (decode form of the cell kernel) or 8 (GEMM form): ragged last group
    cfg = to.GnmtConfig(vocab=300, hidden=64, max_steps=12, min_len=3, max_len=17)
    w = to.make_gnmt_weights(cfg, seed=3, gain=2.0, logit_gain=4.0)
    sentences = to.make_sentences(11, cfg, seed=5)
    decided, total = _follow(cfg, w, sentences, group, 12, 1e-2, 1e-2, 0.05)
    assert decided > total // 2


def test_gnmt_small_model_free_running_matches_oracle():
    # sharper logits: the free-running transcripts themselves must agree while every step's margin is clear
    cfg = to.GnmtConfig(vocab=300, hidden=64, max_steps=16, min_len=3, max_len=17)
    w = to.make_gnmt_weights(cfg, seed=4, gain=2.0, logit_gain=8.0)
    sentences = to.make_sentences(9, cfg, seed=6)
    tr = _translator(cfg, w, 8)
    toks = tr.translate(sentences, steps=16)
    compared = 0
    for i, s in enumerate(sentences):
        rt, rl = to.gnmt_translate(w, s, cfg, 16)
        top2 = torch.topk(rl, 2, dim=1).values
        if float((top2[:, 0] - top2[:, 1]).min()) < 0.05:
            continue
        assert toks[i] == rt
        compared += 1
    assert compared >= 3


def test_gnmt_benchmark_configuration_full_length():
    # the benchmark's sizes (hidden 1024, vocabulary 32320, sentences of 20..50 tokens) over all 80 decode steps for six
    # sentences decoded in one lock-step group of 32 (the rest of the group is padding)
    cfg = to.GnmtConfig()
    w = to.make_gnmt_weights(cfg, seed=1, logit_gain=4.0)
    sentences = to.make_sentences(6, cfg, seed=2)
    decided, total = _follow(cfg, w, sentences, 32, cfg.max_steps, 5e-3, 5e-3, 0.03)
    assert decided > total // 5


def test_gnmt_results_independent_of_group_and_repeatable():
    cfg = to.GnmtConfig(vocab=300, hidden=64, max_steps=10, min_len=3, max_len=17)
    w = to.make_gnmt_weights(cfg, seed=7, gain=2.0, logit_gain=8.0)
    sentences = to.make_sentences(20, cfg, seed=8)
    tr = _translator(cfg, w, 16)
    a = tr.translate(sentences, steps=10)
    b = tr.translate(sentences, steps=10)
    assert a == b
    # the end-of-sentence cut of the user call
    cut = tr.translate(sentences)
    for full, c in zip(a, cut):
        assert c == (full[:full.index(cfg.eos) + 1] if cfg.eos in full else full)
