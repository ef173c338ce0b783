"""GPU: the C++ op executors (registered by ir::LayerType, driven through hand-built hot-path graphs) and the
PipelineManager class, against libtorch CPU on the same inputs."""
import os
import tempfile

import numpy as np
import pytest
import torch

from oracle import torch_oracle as to
from tests.util import assert_close, h16, lstm_params, to_dev

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-3


def _host():
    from pimaicompiler_b200.host import build
    build.build()
    from pimaicompiler_b200 import _pimb200_host
    return _pimb200_host


def test_addmm_mv_swapped_form_with_fused_relu():
    # the graph form after ConvertLinearToAddmm + SwapAddmmInputs + FuseActivation: addmm(b[N], W[N,K], x^T[1,1,K,1])
    h = _host()
    g = torch.Generator().manual_seed(0)
    N, K = 512, 1344
    W, b, x = h16(torch.randn(N, K, generator=g) * 0.03), h16(torch.randn(N, generator=g)), h16(torch.randn(K, generator=g))
    gr = h.Graph()
    i_b, i_W, i_x = gr.add_input(), gr.add_input(), gr.add_input()
    gr.mark_output(gr.add_addmm(i_b, i_W, i_x, act="aten::relu"))
    rt = h.NNRuntime(gr, "RNNT")
    (out,) = rt.inferenceModel([to_dev(b), to_dev(W), to_dev(x).view(1, 1, K, 1)])
    ref = torch.relu(torch.nn.functional.linear(x, W, b))
    assert out.shape == (1, 1, N, 1)
    assert_close(out.view(-1), ref, ATOL, RTOL, "addmm MV")


def test_addmm_vm_and_matmul_classes():
    h = _host()
    g = torch.Generator().manual_seed(1)
    K, N = 320, 1280
    x, A, b = h16(torch.rand(K, generator=g)), h16(torch.rand(K, N, generator=g)), h16(torch.rand(N, generator=g))
    gr = h.Graph()
    i_b, i_x, i_A, i_v = gr.add_input(), gr.add_input(), gr.add_input(), gr.add_input()
    gr.mark_output(gr.add_addmm(i_b, i_x, i_A))       # VM with bias
    gr.mark_output(gr.add_matmul(i_x, i_A))           # VM
    gr.mark_output(gr.add_matmul(i_x, i_v))           # VV
    rt = h.NNRuntime(gr)
    xd = to_dev(x).view(1, 1, 1, K)
    vm_b, vm, vv = rt.inferenceModel([to_dev(b), xd, to_dev(A), to_dev(x).view(K, 1)])
    assert vm.shape == (1, 1, 1, N) and vv.shape == (1, 1, 1, 1)
    assert_close(vm.view(-1), x @ A, 4e-2, RTOL, "matmul VM")
    assert_close(vm_b.view(-1), x @ A + b, 4e-2, RTOL, "addmm VM")
    assert_close(vv.view(-1), (x @ x).view(1), 4e-2, 2e-3, "matmul VV")


def test_addmm_mm_forms_and_linear():
    h = _host()
    g = torch.Generator().manual_seed(2)
    N, K, J = 256, 96, 8
    W, b, X = h16(torch.randn(N, K, generator=g) * 0.1), h16(torch.randn(N, generator=g)), h16(torch.randn(J, K, generator=g))
    gr = h.Graph()
    i_b, i_W, i_Xt, i_X = gr.add_input(), gr.add_input(), gr.add_input(), gr.add_input()
    gr.mark_output(gr.add_addmm(i_b, i_W, i_Xt))                       # swapped MM: W[N,K] @ X^T[K,J] + b per row
    gr.mark_output(gr.add_linear(i_X, to_dev(W), to_dev(b)))           # aten::linear, batched streams
    gr.mark_output(gr.add_matmul(i_X, i_Xt))                           # plain MM without bias
    rt = h.NNRuntime(gr)
    Xd = to_dev(X)
    mm, lin, xx = rt.inferenceModel([to_dev(b), to_dev(W), Xd.t(), Xd])
    ref = torch.nn.functional.linear(X, W, b)
    assert_close(mm, ref.t(), ATOL, RTOL, "addmm MM swapped")
    assert_close(lin, ref, ATOL, RTOL, "linear")
    assert_close(xx, X @ X.t(), 2e-2, 2e-3, "matmul MM")


def test_add_bmm_cat_copy_executors():
    h = _host()
    g = torch.Generator().manual_seed(3)
    a, b, row = (torch.randn(4, 1024, generator=g).half(), torch.randn(4, 1024, generator=g).half(),
                 torch.randn(1024, generator=g).half())
    k = 37
    x, A = torch.softmax(torch.randn(1, 1, k, generator=g), -1).half(), torch.randn(1, k, 1024, generator=g).half()
    gr = h.Graph()
    ia, ib, irow, ix, iA, idst = (gr.add_input() for _ in range(6))
    s1 = gr.add_add(ia, ib)
    s2 = gr.add_add(ia, irow)
    ctx = gr.add_bmm(ix, iA)
    cat = gr.add_cat(gr.add_list([s1, s2]), 1)
    cp = gr.add_copy(idst, s1)
    for o in (s1, s2, ctx, cat, cp):
        gr.mark_output(o)
    rt = h.NNRuntime(gr, "GNMT")
    dst = torch.zeros(4, 1024, dtype=torch.float16, device="cuda")
    o1, o2, octx, ocat, ocp = rt.inferenceModel([a.cuda(), b.cuda(), row.cuda(), x.cuda(), A.cuda(), dst])
    assert torch.equal(o1.cpu(), a + b) and torch.equal(o2.cpu(), a + row)
    assert_close(octx, torch.bmm(x.float(), A.float()), ATOL, RTOL, "bmm")
    assert torch.equal(ocat.cpu(), torch.cat([a + b, a + row], 1))
    assert torch.equal(ocp.cpu(), a + b) and ocp.data_ptr() == dst.data_ptr()


def test_decode_glue_executors_attention_and_classifier_tail():
    # The tail of a GNMT / Transformer decode step as one graph: attention scores -> tanh -> masked_fill ->
    # softmax; model vector -> layer_norm; logits -> log_softmax and argmax.  fp16 CUDA inputs take the device
    # kernels, the fp32 CPU run of the same graph takes the executors' libtorch branch (the reference's calls).
    h = _host()
    g = torch.Generator().manual_seed(5)
    scores = h16(torch.randn(8, 1, 13, generator=g) * 2.0)
    mask = torch.rand(13, generator=g) < 0.3
    vec = h16(torch.randn(1, 512, generator=g))
    gamma, beta = h16(torch.rand(512, generator=g) + 0.5), h16(torch.randn(512, generator=g) * 0.1)
    logits = h16(torch.randn(1, 32320, generator=g) * 3.0)
    table = h16(torch.randn(32320, 64, generator=g))

    def build(dev):
        gr = h.Graph()
        i_s, i_m, i_v, i_l, i_t = gr.add_input(), gr.add_input(), gr.add_input(), gr.add_input(), gr.add_input()
        t = gr.add_tanh(i_s)
        f = gr.add_masked_fill(t, i_m, -65504.0)
        gr.mark_output(gr.add_softmax(f, -1))
        gr.mark_output(gr.add_layer_norm(i_v, [512], dev(gamma), dev(beta), 1e-5))
        gr.mark_output(gr.add_softmax(i_l, -1, log=True))
        gr.mark_output(gr.add_argmax(i_l, -1, keepdim=True))
        am = gr.add_argmax(i_l, -1, keepdim=False)
        gr.mark_output(gr.add_embedding(i_t, am))          # the chosen token's embedding row; the index stays on the device
        return h.NNRuntime(gr)

    got = build(to_dev).inferenceModel([to_dev(scores), mask.cuda(), to_dev(vec), to_dev(logits), to_dev(table)])
    ref = build(lambda t: t).inferenceModel([scores, mask, vec, logits, table])
    assert got[0].dtype == torch.float16 and got[3].dtype == torch.int64 and got[3].shape == (1, 1)
    assert got[4].shape == (1, 64) and torch.equal(got[4].float().cpu(), ref[4])
    assert_close(got[0], ref[0], 1e-3, 1e-3, "tanh -> masked_fill -> softmax")
    assert_close(got[1], ref[1], 3e-3, 1e-3, "layer_norm")
    assert_close(got[2], ref[2], 8e-3, 1e-3, "log_softmax")
    assert torch.equal(got[3].cpu(), ref[3])
    # masked positions carry no attention weight
    assert float(got[0].float().cpu()[..., mask].abs().max()) == 0.0


def test_custom_cat_returns_prefilled_buffer_without_copy():
    h = _host()
    gr = h.Graph()
    buf = torch.arange(2048, dtype=torch.float16, device="cuda").view(1, 1, 2048)
    bid = gr.preset_blob(buf)
    ia, ib = gr.add_input(), gr.add_input()
    gr.mark_output(gr.add_cat(gr.add_list([ia, ib]), 2, mem_layer_id=bid))
    rt = h.NNRuntime(gr, "GNMT")
    z = torch.zeros(1, 1, 1024, dtype=torch.float16, device="cuda")
    (out,) = rt.inferenceModel([z, z])
    assert out.data_ptr() == buf.data_ptr() and torch.equal(out, buf)


@pytest.mark.parametrize("bidirectional,batch_first", [(False, False), (True, True)])
def test_lstm1_executor(bidirectional, batch_first):
    h = _host()
    g = torch.Generator().manual_seed(4)
    T, B, I, H, L = 9, 2, 32, 64, 2
    D = 2 if bidirectional else 1
    ps = lstm_params(L, D, I, H, g)
    x = h16(torch.randn((B, T, I) if batch_first else (T, B, I), generator=g))
    h0, c0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5), h16(torch.randn(L * D, B, H, generator=g) * 0.5)
    gr = h.Graph()
    ix, ih, ic = gr.add_input(), gr.add_input(), gr.add_input()
    y = gr.add_lstm([ix, gr.add_list([ih, ic])], [to_dev(p) for p in ps], True, L, bidirectional, batch_first)
    for o in (y, y + 1, y + 2):
        gr.mark_output(o)
    rt = h.NNRuntime(gr)
    out = rt.inferenceModel([to_dev(x), to_dev(h0), to_dev(c0)])
    ref = torch.lstm(x, [h0, c0], ps, True, L, 0.0, False, bidirectional, batch_first)
    for name, a, b in zip(("y", "hn", "cn"), out, ref):
        assert_close(a, b, 4e-3, 4e-3, name)


def test_lstm1_gnmt_style_output_aliasing():
    # decoder cell, seq_len 1: output goes to the first half of a {1,1,2048} cat buffer, (h,c) into slots of {8,1,1024}
    h = _host()
    g = torch.Generator().manual_seed(5)
    I = H = 1024
    ps = lstm_params(1, 1, I, H, g)
    x = h16(torch.randn(1, 1, I, generator=g))
    h0, c0 = h16(torch.randn(1, 1, H, generator=g) * 0.5), h16(torch.randn(1, 1, H, generator=g) * 0.5)
    gr = h.Graph()
    cat_buf = torch.full((1, 1, 2048), 3.0, dtype=torch.float16, device="cuda")
    st_buf = torch.full((8, 1, 1024), 3.0, dtype=torch.float16, device="cuda")
    b_cat, b_st = gr.preset_blob(cat_buf), gr.preset_blob(st_buf)
    ix, ih, ic = gr.add_input(), gr.add_input(), gr.add_input()
    y = gr.add_lstm([ix, gr.add_list([ih, ic])], [to_dev(p) for p in ps], True, 1, False, False,
                    aliases=[(b_cat, 0), (b_st, 2 * 1024), (b_st, 3 * 1024)])
    gr.mark_output(y)
    rt = h.NNRuntime(gr, "GNMT")
    (out,) = rt.inferenceModel([to_dev(x), to_dev(h0), to_dev(c0)])
    ref = torch.lstm(x, [h0, c0], ps, True, 1, 0.0, False, False, False)
    assert out.data_ptr() == cat_buf.data_ptr()
    assert_close(cat_buf[..., :1024], ref[0], 4e-3, 4e-3, "aliased y")
    assert_close(st_buf[2:3], ref[1], 4e-3, 4e-3, "aliased hn")
    assert_close(st_buf[3:4], ref[2], 4e-3, 4e-3, "aliased cn")
    assert (cat_buf[..., 1024:] == 3).all() and (st_buf[:2] == 3).all() and (st_buf[4:] == 3).all()


def test_lstm2_packed_executor():
    h = _host()
    g = torch.Generator().manual_seed(6)
    T, B, I, H, L = 7, 4, 16, 32, 2
    ps = lstm_params(L, 1, I, H, g)
    x = h16(torch.randn(T, B, I, generator=g))
    pk = torch.nn.utils.rnn.pack_padded_sequence(x, torch.tensor([7, 6, 3, 1]))
    h0, c0 = h16(torch.randn(L, B, H, generator=g) * 0.5), h16(torch.randn(L, B, H, generator=g) * 0.5)
    gr = h.Graph()
    idata, ibs, ih, ic = (gr.add_input() for _ in range(4))
    y = gr.add_lstm([idata, ibs, gr.add_list([ih, ic])], [to_dev(p) for p in ps], True, L, False, False, packed=True)
    for o in (y, y + 1, y + 2):
        gr.mark_output(o)
    rt = h.NNRuntime(gr, "GNMT")
    out = rt.inferenceModel([to_dev(pk.data), pk.batch_sizes, to_dev(h0), to_dev(c0)])
    ref = torch.lstm(pk.data, pk.batch_sizes, [h0, c0], ps, True, L, 0.0, False, False)
    for name, a, b in zip(("y", "hn", "cn"), out, ref):
        assert_close(a, b, 4e-3, 4e-3, "packed " + name)


def test_multistream_runs_independent_branches():
    # four expert-style matmul/addmm branches on side streams (SwitchTransformer pattern)
    h = _host()
    g = torch.Generator().manual_seed(7)
    K, N = 512, 2048
    x = h16(torch.randn(K, generator=g))
    Ws = [h16(torch.randn(N, K, generator=g) * 0.05) for _ in range(4)]
    b = h16(torch.randn(N, generator=g))
    gr = h.Graph()
    ix, ib = gr.add_input(), gr.add_input()
    iW = [gr.add_input() for _ in range(4)]
    outs = gr.add_multistream([("matmul", [iW[0], ix], ""), ("matmul", [iW[1], ix], ""),
                               ("addmm", [ib, iW[2], ix], "aten::relu"), ("addmm", [ib, iW[3], ix], "none")])
    for o in outs:
        gr.mark_output(o)
    rt = h.NNRuntime(gr, "SwitchTransformer")
    res = rt.inferenceModel([to_dev(x).view(K, 1), to_dev(b)] + [to_dev(W) for W in Ws])
    refs = [Ws[0] @ x, Ws[1] @ x, torch.relu(Ws[2] @ x + b), Ws[3] @ x + b]
    for r, ref in zip(res, refs):
        assert_close(r.view(-1), ref, ATOL, RTOL, "multistream branch")


def test_pipeline_manager_rnnt_from_torchscript():
    from pimaicompiler_b200 import synthetic as syn
    from pimaicompiler_b200.NNCompiler import PipelineManager
    cfg = syn.RnntConfig(feat_dim=24, enc_hidden=64, pred_hidden=32, joint_hidden=48, vocab=11, blank=10)
    w = syn.make_rnnt_weights(cfg, seed=2, gain=2.0, logit_gain=6.0)
    feats = syn.make_features(41, cfg, 11)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "rnnt.torchscript")
        syn.save_rnnt_torchscript(path, cfg, w)
        pm = PipelineManager(path, "RNNT")
    out = pm.inferenceModel([feats.view(41, 1, -1).half().cuda(), torch.tensor([41])])
    logits, n, transcript = out
    forced = logits.argmax(1).tolist()
    _, ref_logits, ref_choice = to.rnnt_greedy(w, feats, cfg, forced)
    assert_close(logits, ref_logits, 2e-2, 1e-2, "PipelineManager logits")
    assert transcript.tolist() == [k for k in forced if k != cfg.blank] and int(n) == len(transcript)


def test_multistream_with_matrix_branches_and_transposed_views():
    # MULTISTREAM branches whose operands need temporaries (an MM-class product, a transposed view of a row-major
    # weight, a non-contiguous activation): the copies must be made on the branch's own stream.  Repeated, so that a
    # race between the preparation and the kernel, or a recycled temporary, shows as a wrong result.
    h = _host()
    g = torch.Generator().manual_seed(17)
    K, N, J = 256, 384, 24
    X = h16(torch.randn(J, K, generator=g))
    Wt = h16(torch.randn(K, N, generator=g) * 0.05)          # used as Wt.t(): a transposed view, K-major rows
    W2 = h16(torch.randn(N, K, generator=g) * 0.05)
    xs = h16(torch.randn(K, 2, generator=g))                  # column 0 of a [K, 2] tensor: non-contiguous vector
    b = h16(torch.randn(N, generator=g))
    gr = h.Graph()
    iX, iWt, iW2, ixs, ib = (gr.add_input() for _ in range(5))
    outs = gr.add_multistream([("matmul", [iX, iWt], ""), ("matmul", [iW2, ixs], ""),
                               ("addmm", [ib, iW2, ixs], "aten::relu"), ("matmul", [iX, iWt], "")])
    for o in outs:
        gr.mark_output(o)
    rt = h.NNRuntime(gr, "SwitchTransformer")
    Xd, Wtd, W2d, bd = to_dev(X), to_dev(Wt), to_dev(W2), to_dev(b)
    xsd = xs.to(torch.float16).cuda()[:, :1]                  # [K, 1] view with stride 2
    refs = [X @ Wt, W2 @ xs[:, :1], torch.relu(W2 @ xs[:, :1] + b.view(-1, 1)), X @ Wt]
    for _ in range(20):
        res = rt.inferenceModel([Xd, Wtd, W2d, xsd, bd])
        for r, ref in zip(res, refs):
            assert_close(r.reshape(ref.shape), ref, 4e-3, 2e-3, "multistream branch with temporaries")


def test_multistream_of_matrix_branches_is_one_grouped_launch():
    # four expert projections of 26 token rows (the SwitchTransformer pattern the reference runs on four streams): every
    # branch is a matrix-class product, so the node is one grouped launch; a biased branch indexes its bias by the row of
    # mat1, as the reference's MM branch does
    h = _host()
    g = torch.Generator().manual_seed(23)
    J, K, N = 26, 512, 1024
    X = h16(torch.randn(J, K, generator=g))
    Wts = [h16(torch.randn(K, N, generator=g) * 0.05) for _ in range(3)]
    W4 = h16(torch.randn(N, K, generator=g) * 0.05)
    b = h16(torch.randn(J, generator=g))
    gr = h.Graph()
    iX, ib, iW4 = gr.add_input(), gr.add_input(), gr.add_input()
    iW = [gr.add_input() for _ in range(3)]
    outs = gr.add_multistream([("matmul", [iX, iW[0]], ""), ("matmul", [iX, iW[1]], ""), ("addmm", [ib, iX, iW[2]], "none"),
                               ("matmul", [iX, iW4], "")])
    for o in outs:
        gr.mark_output(o)
    rt = h.NNRuntime(gr, "SwitchTransformer")
    before = h.grouped_launch_count()
    res = rt.inferenceModel([to_dev(X), to_dev(b), to_dev(W4).t()] + [to_dev(W) for W in Wts])
    assert h.grouped_launch_count() == before + 1
    refs = [X @ Wts[0], X @ Wts[1], X @ Wts[2] + b.view(-1, 1), X @ W4.t()]
    for r, ref in zip(res, refs):
        assert r.shape == ref.shape
        assert_close(r, ref, 4e-3, 2e-3, "grouped multistream branch")


def test_profiling_writes_a_chrome_trace_with_one_span_per_op():
    import json
    h = _host()
    g = torch.Generator().manual_seed(3)
    N, K = 256, 512
    W, b, x = h16(torch.randn(N, K, generator=g) * 0.05), h16(torch.randn(N, generator=g)), h16(torch.randn(K, generator=g))
    gr = h.Graph()
    i_b, i_W, i_x = gr.add_input(), gr.add_input(), gr.add_input()
    y = gr.add_addmm(i_b, i_W, i_x, act="aten::relu")
    gr.mark_output(gr.add_tanh(y))
    rt = h.NNRuntime(gr)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "trace.json")
        (out,) = rt.inferenceModel([to_dev(b), to_dev(W), to_dev(x).view(K, 1)], profiling=True, profile_path=path)
        with open(path) as f:
            trace = json.load(f)
    ev = trace["traceEvents"]
    assert [e["name"] for e in ev] == ["aten::addmm", "aten::tanh"]
    assert all(e["ph"] == "X" and e["dur"] > 0 for e in ev) and ev[1]["ts"] >= ev[0]["ts"]
    assert_close(out.view(-1), torch.tanh(torch.relu(W @ x + b)), ATOL, RTOL, "profiled run result")


def test_hot_shapes_never_fall_back_to_the_library_call():
    # the shapes of the benchmark configurations (batch-1 linear layers in the swapped addmm form, the RNN-T joint pair,
    # decoder-style add / softmax / argmax / layer_norm / cat rows) must all run on this library's kernels
    h = _host()
    g = torch.Generator().manual_seed(5)
    h.reset_fallback_count()
    for (N, K) in ((4096, 1024), (1024, 1024), (29, 512), (512, 1024), (512, 320), (2048, 512), (512, 2048)):
        W, b, x = h16(torch.randn(N, K, generator=g) * 0.03), h16(torch.randn(N, generator=g)), h16(torch.randn(K, generator=g))
        gr = h.Graph()
        i_b, i_W, i_x = gr.add_input(), gr.add_input(), gr.add_input()
        y = gr.add_addmm(i_b, i_W, i_x, act="aten::relu")
        gr.mark_output(y)
        gr.mark_output(gr.add_matmul(i_W, i_x))
        rt = h.NNRuntime(gr)
        o1, o2 = rt.inferenceModel([to_dev(b), to_dev(W), to_dev(x).view(1, 1, K, 1)])
        assert_close(o1.view(-1), torch.relu(W @ x + b), 4e-3, 2e-3, f"addmm {N}x{K}")
    gr = h.Graph()
    ia, ib2 = gr.add_input(), gr.add_input()
    s = gr.add_add(ia, ib2)
    gr.mark_output(gr.add_softmax(s))
    gr.mark_output(gr.add_argmax(s))
    gr.mark_output(gr.add_layer_norm(s, [512]))
    gr.mark_output(gr.add_cat(gr.add_list([s, s]), 1))
    rt = h.NNRuntime(gr)
    a = to_dev(h16(torch.randn(1, 512, generator=g)))
    rt.inferenceModel([a, a])
    assert h.fallback_count() == 0
