"""GPU parity of the device-resident RNN-T greedy decode against the libtorch-CPU and C oracles."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as co
from oracle import torch_oracle as to
from tests.util import CONTRACT_ATOL, CONTRACT_RTOL, assert_close

pytestmark = pytest.mark.gpu
MARGIN = 1e-2  # token ids must match wherever the oracle's top-2 logit margin exceeds this


def _decoder(cfg, w):
    from pimaicompiler_b200.rnnt import RnntDecoder
    d = lambda t: t.to(torch.float16).cuda().contiguous()
    return RnntDecoder(cfg, [d(p) for p in w.pre], [d(p) for p in w.post], d(w.embedding), [d(p) for p in w.pred],
                       d(w.w1), d(w.b1), d(w.w2), d(w.b2))


def _check_utterance(cfg, w, feats, got_tokens, got_logits, oracle):
    """Follow-mode check: the oracle replays the GPU's decisions, so every frame is comparable; the GPU's
    decision must equal the oracle's argmax at every frame whose oracle margin exceeds MARGIN."""
    Tp = got_logits.shape[0]
    got_choice = got_logits.argmax(1)
    # the GPU's per-frame decisions, reconstructed from its logits (it emits iff argmax != blank)
    forced = got_choice.tolist()
    emitted = [k for k in forced if k != cfg.blank]
    assert emitted == got_tokens, "token list is not the sequence of non-blank argmaxes of the returned logits"
    _, ref_logits, ref_choice = oracle(w, feats, cfg, forced)
    ref_logits = np.asarray(ref_logits)
    assert_close(got_logits, ref_logits, CONTRACT_ATOL, CONTRACT_RTOL, "joint logits")
    srt = np.sort(ref_logits, axis=1)
    margin = srt[:, -1] - srt[:, -2]
    decided = margin > MARGIN
    assert (np.asarray(ref_choice)[decided] == np.asarray(forced)[decided]).all(), "token mismatch at a decided frame"
    err = float(np.abs(got_logits - ref_logits).max())
    return int(decided.sum()), Tp, err


@pytest.mark.parametrize("seed,gain,logit_gain", [(0, 1.0, 1.0), (1, 2.0, 6.0), (2, 3.0, 10.0)])
def test_rnnt_small_model_vs_c_oracle(seed, gain, logit_gain):
    cfg = to.RnntConfig(feat_dim=24, enc_hidden=64, pred_hidden=32, joint_hidden=48, vocab=11, blank=10)
    w = to.make_rnnt_weights(cfg, seed=seed, gain=gain, logit_gain=logit_gain)
    dec = _decoder(cfg, w)
    for T in (2, 9, 40, 61):
        feats = to.make_features(T, cfg, 100 + T)
        toks, logits = dec.decode(feats.to(torch.float16).cuda(), want_logits=True)
        _check_utterance(cfg, w, feats, toks[0], logits[0].cpu().numpy(), co.rnnt_greedy)


def test_rnnt_baseline_config_vs_libtorch():
    # the benchmark's architecture, a 2 s utterance (the oracle stays within seconds), mixed decisions
    cfg = to.RnntConfig()
    w = to.make_rnnt_weights(cfg, seed=0, gain=1.0, logit_gain=1.0)
    dec = _decoder(cfg, w)
    info = dec.info()
    print("greedy kernel:", info)
    feats = to.make_features(200, cfg, 7)
    toks, logits = dec.decode(feats.to(torch.float16).cuda(), want_logits=True)
    nd, Tp, err = _check_utterance(cfg, w, feats, toks[0], logits[0].cpu().numpy(), to.rnnt_greedy)
    print(f"decided frames {nd}/{Tp}, max logit err {err:.2e}")
    # free-running oracle: identical transcript when every frame is decided
    ref_tokens, ref_logits, _ = to.rnnt_greedy(w, feats, cfg)
    srt = np.sort(ref_logits.numpy(), axis=1)
    all_decided = bool(((srt[:, -1] - srt[:, -2]) > MARGIN).all())
    print(f"free-running transcript compared: {all_decided}")
    if all_decided:
        assert toks[0] == ref_tokens
    # the free-running comparison must not be vacuous: a model with sharper logits (every frame decided) is decoded
    # freely on both sides and the transcripts must be identical
    w2 = to.make_rnnt_weights(cfg, seed=3, gain=2.0, logit_gain=30.0)
    dec2 = _decoder(cfg, w2)
    compared = 0
    for s in range(6):
        f2 = to.make_features(120, cfg, 40 + s)
        ref_t, ref_l, _ = to.rnnt_greedy(w2, f2, cfg)
        srt2 = np.sort(ref_l.numpy(), axis=1)
        if not ((srt2[:, -1] - srt2[:, -2]) > MARGIN).all():
            continue
        t2, _ = dec2.decode(f2.to(torch.float16).cuda(), want_logits=True)
        assert t2[0] == ref_t, "free-running transcript differs although every frame is decided"
        compared += 1
    print(f"free-running transcripts compared on the sharper model: {compared} of 6")
    assert compared >= 2


def test_rnnt_baseline_config_blank_mix():
    cfg = to.RnntConfig()
    w = to.make_rnnt_weights(cfg, seed=5, gain=2.0, logit_gain=8.0)
    dec = _decoder(cfg, w)
    feats = to.make_features(120, cfg, 9)
    toks, logits = dec.decode(feats.to(torch.float16).cuda(), want_logits=True)
    _check_utterance(cfg, w, feats, toks[0], logits[0].cpu().numpy(), to.rnnt_greedy)


def test_rnnt_batch_of_utterances_matches_single():
    cfg = to.RnntConfig(feat_dim=24, enc_hidden=64, pred_hidden=32, joint_hidden=48, vocab=11, blank=10)
    w = to.make_rnnt_weights(cfg, seed=4, gain=2.0, logit_gain=6.0)
    dec = _decoder(cfg, w)
    # more utterances than clusters fit on the device; 600 frames (300 after the time reduction), so that every
    # projection has more than 256 rows at any batch and takes the same GEMM kernel (the streaming kernels for few rows
    # sum in another order)
    n, T = 13, 600
    feats = torch.stack([to.make_features(T, cfg, 200 + i) for i in range(n)]).to(torch.float16).cuda()
    dec.set_greedy_multi(2)   # FMA lock-step kernel: same summation order as the one-utterance kernel
    dec.set_wavefront(False)  # calls of up to 8 utterances would otherwise pair the encoder layers (another summation order)
    toks, logits = dec.decode(feats, want_logits=True)
    # lock-step encoding of several utterances must not change any utterance's result: the per-sequence
    # arithmetic (tensor-core tile column, fp32 accumulation order) is the same at every batch size
    dec.set_encoder_batch(1)
    for i in range(n):
        ti, li = dec.decode(feats[i], want_logits=True)
        assert ti[0] == toks[i]
        assert torch.equal(li[0], logits[i])
    dec.set_encoder_batch(3)
    toks3, logits3 = dec.decode(feats, want_logits=True)
    assert toks3 == toks and torch.equal(logits3, logits)


@pytest.mark.parametrize("n_utts", [12, 19])
def test_rnnt_tensor_core_greedy_small_model(n_utts):
    # a model whose shapes the tensor-core greedy kernel accepts (PH, JH multiples of 64, 16 CTAs per cluster); more
    # utterances than clusters, so 8 share a cluster in lock step; every utterance checked against the C oracle
    cfg = to.RnntConfig(feat_dim=24, enc_hidden=64, pred_hidden=64, joint_hidden=256, vocab=11, blank=10)
    w = to.make_rnnt_weights(cfg, seed=6, gain=2.0, logit_gain=6.0)
    w.b2[cfg.blank] += 2.3                     # lifts the blank logit into contention: blank and label frames mix
    w.b2 = w.b2.to(torch.float16).to(torch.float32)
    dec = _decoder(cfg, w)
    T = 36
    feats = [to.make_features(T, cfg, 300 + i) for i in range(n_utts)]
    dev = torch.stack(feats).to(torch.float16).cuda()
    dec.set_greedy_multi(1)
    toks, logits = dec.decode(dev, want_logits=True)
    blanks = 0
    for i in range(n_utts):
        lg = logits[i].cpu().numpy()
        _check_utterance(cfg, w, feats[i], toks[i], lg, co.rnnt_greedy)
        blanks += int((lg.argmax(1) == cfg.blank).sum())
    assert 0 < blanks < n_utts * (T // 2)      # the utterances really do emit in different frames
    # one utterance per cluster gives the same transcripts wherever the oracle is decided (checked above for both)
    dec.set_greedy_multi(0)
    toks0, logits0 = dec.decode(dev, want_logits=True)
    assert_close(logits0, logits.cpu().numpy(), CONTRACT_ATOL, CONTRACT_RTOL, "mma vs one-per-cluster logits")


def test_rnnt_tensor_core_greedy_baseline_config():
    cfg = to.RnntConfig()
    w = to.make_rnnt_weights(cfg, seed=5, gain=2.0, logit_gain=8.0)
    dec = _decoder(cfg, w)
    n, T = 12, 100
    feats = [to.make_features(T, cfg, 400 + i) for i in range(n)]
    toks, logits = dec.decode(torch.stack(feats).to(torch.float16).cuda(), want_logits=True)
    for i in (0, 5, 11):
        _check_utterance(cfg, w, feats[i], toks[i], logits[i].cpu().numpy(), to.rnnt_greedy)


def test_rnnt_ragged_group_sizes_and_odd_frame_count():
    # 70 utterances = one encoder group of 64 + one of 6, nine greedy groups of 8 (the last one ragged); and an odd
    # number of frames, where the time stacking drops the last frame and the encoder falls back to one utterance at a time
    cfg = to.RnntConfig(feat_dim=24, enc_hidden=64, pred_hidden=64, joint_hidden=256, vocab=11, blank=10)
    w = to.make_rnnt_weights(cfg, seed=8, gain=2.0, logit_gain=6.0)
    w.b2[cfg.blank] += 2.3
    w.b2 = w.b2.to(torch.float16).to(torch.float32)
    dec = _decoder(cfg, w)
    for n_utts, T in ((70, 20), (11, 21)):
        feats = [to.make_features(T, cfg, 500 + i) for i in range(n_utts)]
        toks, logits = dec.decode(torch.stack(feats).to(torch.float16).cuda(), want_logits=True)
        assert logits.shape == (n_utts, T // 2, cfg.vocab)
        for i in (0, 5, n_utts - 7, n_utts - 1):
            _check_utterance(cfg, w, feats[i], toks[i], logits[i].cpu().numpy(), co.rnnt_greedy)


def test_rnnt_benchmark_scale_is_independent_of_batching():
    # The benchmark's configuration at full length (1000 frames): 72 utterances in one call (one encoder group of two
    # batch halves, nine greedy groups over two rounds of clusters) against the first 40 of them in a call of their own
    # (one narrower encoder group of the same kernel family, five greedy groups).  Every utterance is a column of the same lock-step arithmetic whatever the
    # batch, so transcripts and logits must be bit-identical; a repeat of the large call as well.
    cfg = to.RnntConfig()
    w = to.make_rnnt_weights(cfg, seed=9, gain=2.0, logit_gain=8.0)
    w.b2[cfg.blank] += 2.0                     # ~5 % blank frames (libtorch CPU: 463..489 labels in 500 frames), so the
                                               # utterances emit in different frames; at 1.5 a blank is a once-per-run event
    w.b2 = w.b2.to(torch.float16).to(torch.float32)
    dec = _decoder(cfg, w)
    g = torch.Generator().manual_seed(72)
    feats = torch.randn(72, 1000, cfg.feat_dim, generator=g).to(torch.float16).cuda()
    toks, logits = dec.decode(feats, want_logits=True)
    toks_again, logits_again = dec.decode(feats, want_logits=True)
    assert toks_again == toks and torch.equal(logits_again, logits)
    toks40, logits40 = dec.decode(feats[:40].contiguous(), want_logits=True)
    assert toks40 == toks[:40]
    assert torch.equal(logits40, logits[:40])
    lens = [len(t) for t in toks]
    assert 0 < min(lens) and max(lens) <= 500 and len(set(lens)) > 1   # transcripts differ, none empty


def test_rnnt_benchmark_configuration_vs_libtorch_full_length():
    # The configuration the benchmark times: 1000 frames per utterance, 64 utterances advanced in lock step (the
    # 64-sequence recurrence kernel, the batched joint GEMM and the tensor-core greedy kernel).  Three utterances taken
    # out of that call, and the same three decoded alone (the one-sequence recurrence and the one-utterance greedy
    # kernel), are compared with libtorch CPU fp32 over all 500 joint frames: logits within the contract, token ids
    # equal to the oracle's arg max wherever its top-2 margin exceeds MARGIN.  fp16 hidden states feed back through
    # 1000 steps of five layers here, which shorter utterances do not exercise.
    cfg = to.RnntConfig()
    w = to.make_rnnt_weights(cfg, seed=9, gain=2.0, logit_gain=8.0)
    w.b2[cfg.blank] += 1.5
    w.b2 = w.b2.to(torch.float16).to(torch.float32)
    dec = _decoder(cfg, w)
    g = torch.Generator().manual_seed(64)
    feats = torch.randn(64, 1000, cfg.feat_dim, generator=g).to(torch.float16)
    toks, logits = dec.decode(feats.cuda(), want_logits=True)
    assert logits.shape == (64, 500, cfg.vocab)
    for i in (0, 37, 63):
        f32 = feats[i].float()
        nd, Tp, err = _check_utterance(cfg, w, f32, toks[i], logits[i].cpu().numpy(), to.rnnt_greedy)
        ref = np.asarray(to.rnnt_greedy(w, f32, cfg, logits[i].argmax(1).tolist())[1])
        err_last = float(np.abs(logits[i, Tp - 1].cpu().numpy() - ref[Tp - 1]).max())
        print(f"utterance {i} in a 64-utterance call: decided frames {nd}/{Tp}, max logit err {err:.2e}, "
              f"at frame {Tp - 1}: {err_last:.2e}, {len(toks[i])} tokens")
        assert nd > Tp // 2
        t1, l1 = dec.decode(feats[i].cuda(), want_logits=True)
        nd1, _, err1 = _check_utterance(cfg, w, f32, t1[0], l1[0].cpu().numpy(), to.rnnt_greedy)
        print(f"utterance {i} decoded alone: decided frames {nd1}/{Tp}, max logit err {err1:.2e}")


def test_rnnt_timeout_is_reported_and_does_not_poison_later_decodes():
    # Fault handling without faulting anything: the bounded waits of the encoder recurrences and of the greedy kernel's
    # exchange barriers are shrunk to one poll, so the first decode gives up (a CTA of the greedy kernel that gave up stops
    # sending and still joins the final cluster barrier); decode() must raise ERR_TIMEOUT.  A second timed-out decode is then issued through the
    # asynchronous entry point and nobody reads the status; the decode behind it (normal limit) must still be correct,
    # and the time-out must still be on record afterwards.
    from pimaicompiler_b200 import _lib
    cfg = to.RnntConfig(feat_dim=24, enc_hidden=256, pred_hidden=32, joint_hidden=48, vocab=11, blank=10)
    w = to.make_rnnt_weights(cfg, seed=11, gain=2.0, logit_gain=6.0)
    dec = _decoder(cfg, w)
    feats = to.make_features(64, cfg, 77)
    dev = feats.to(torch.float16).cuda().unsqueeze(0).contiguous()
    good_tokens, good_logits = dec.decode(dev, want_logits=True)
    _check_utterance(cfg, w, feats, good_tokens[0], good_logits[0].cpu().numpy(), co.rnnt_greedy)
    dec.set_poll_limit(1)
    with pytest.raises(_lib.Pimb200Error) as e:
        dec.decode(dev)
    assert e.value.status == _lib.ERR_TIMEOUT
    assert dec.last_status() == 0                      # reading cleared it
    Tp = 32
    tokens = torch.zeros(1, Tp, dtype=torch.int32, device="cuda")
    n_tokens = torch.zeros(1, dtype=torch.int32, device="cuda")
    dec.decode_into(dev, tokens, n_tokens)             # gives up again; status left unread
    dec.set_poll_limit(1 << 21)
    logits = torch.empty(1, Tp, cfg.vocab, dtype=torch.float32, device="cuda")
    dec.decode_into(dev, tokens, n_tokens, logits)
    torch.cuda.synchronize()
    assert torch.equal(logits, good_logits)
    assert tokens[0, : int(n_tokens[0])].tolist() == good_tokens[0]
    assert dec.last_status() == _lib.ERR_TIMEOUT       # the earlier time-out is still reported
    assert dec.last_status() == 0
