"""CPU: host-side logic of the translation workloads: packing of sentences into lock-step groups (against torch's own
pack_padded_sequence) and the round-robin sharding of the streams over ranks."""
import torch

from pimaicompiler_b200 import synthetic as syn
from pimaicompiler_b200.gnmt import stage_groups


def test_stage_groups_matches_pack_padded_sequence_and_covers_every_sentence():
    cfg = syn.GnmtConfig(vocab=300, hidden=64, max_steps=12, min_len=3, max_len=17)
    sents = syn.make_sentences(21, cfg, 5)
    G, EB = 8, 3
    groups = stage_groups(sents, G, EB, cfg.max_len)
    seen = []
    for g in groups:
        idx = g["idx"]
        seen += idx
        lens = [len(sents[i]) for i in idx] + [1] * (G - len(idx))
        assert g["lengths"].tolist() == lens and lens == sorted(lens, reverse=True) and g["S"] == lens[0]
        padded = torch.full((g["S"], G), -1, dtype=torch.int64)       # what the slices scatter into
        for k, sl in enumerate(g["slices"]):
            j0 = k * EB
            sl_idx = idx[j0:j0 + EB]
            if sl_idx:
                sl_lens = [len(sents[i]) for i in sl_idx]
                pad = torch.zeros(sl_lens[0], len(sl_idx), dtype=torch.int64)
                for b, i in enumerate(sl_idx):
                    pad[:sl_lens[b], b] = sents[i]
                if len(sl_idx) == min(EB, G - j0):                     # slice without dummies: torch's own packing
                    pk = torch.nn.utils.rnn.pack_padded_sequence(pad, torch.tensor(sl_lens))
                    assert torch.equal(pk.data, sl["ids"]) and torch.equal(pk.batch_sizes, sl["batch_sizes"])
            assert int(sl["batch_sizes"].sum()) == sl["ids"].numel() == sl["dst"].numel()
            padded.view(-1)[sl["dst"]] = sl["ids"]
        for j, i in enumerate(idx):                                    # every token lands at row t, column j
            assert torch.equal(padded[:len(sents[i]), j], sents[i])
            assert (padded[len(sents[i]):, j] == -1).all()
    assert sorted(seen) == list(range(len(sents)))


def test_round_robin_shards_partition_the_streams():
    cfg = syn.TransformerConfig()
    seqs = syn.make_sentences(50, cfg, 11)
    for world in (1, 2, 4, 8):
        shards = [seqs[r::world] for r in range(world)]
        assert sum(len(s) for s in shards) == len(seqs)
        assert max(len(s) for s in shards) - min(len(s) for s in shards) <= 1
        back = [None] * len(seqs)
        for r, sh in enumerate(shards):
            for k, s in enumerate(sh):
                back[r + k * world] = s
        assert all(torch.equal(a, b) for a, b in zip(back, seqs))
