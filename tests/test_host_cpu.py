"""CPU: host-side logic — the GEMM shape classifier (Python and C++), the executor registry module loads, the
synthetic TorchScript container round-trips."""
import os
import tempfile

import pytest
import torch

from pimaicompiler_b200 import executor as ex
from pimaicompiler_b200 import synthetic as syn

CASES = [
    # (left shape, right shape, class)   shapes as the graphs of the hot path produce them
    ([4096, 1024], [1, 1, 1024, 1], ex.MV),       # W·x^T after SwapAddmmInputs
    ([1, 1, 1, 1024], [1024, 4096], ex.VM),        # customGemvTest x·A
    ([4096, 1024], [1024], ex.MV),
    ([1024], [1024, 4096], ex.VM),
    ([1024], [1024], ex.VV),
    ([1, 1, 1, 8], [1, 1, 8, 1], ex.VV),
    ([8, 1024], [1024, 4096], ex.MM),
    ([2, 1, 1024], [1024, 16], ex.MM),             # a real batch dimension is never a vector class
    ([1, 1, 1], [1, 1], ex.MM),                    # degenerate 1x1: no extent differs from 1
]


@pytest.mark.parametrize("a,b,cls", CASES)
def test_gemm_classifier_python(a, b, cls):
    assert ex.classify(a, b) == cls


def _host():
    from pimaicompiler_b200.host import build
    build.build()
    from pimaicompiler_b200 import _pimb200_host
    return _pimb200_host


@pytest.mark.parametrize("a,b,cls", CASES)
def test_gemm_classifier_cpp_agrees(a, b, cls):
    h = _host()
    pa, pb = ex.gemm_broadcast(a, b)
    assert h.get_gemm_type(pa, pb) == ex.get_gemm_type(pa, pb) == cls


def test_graph_builder_assigns_ids_in_order():
    h = _host()
    g = h.Graph()
    a, b = g.add_input(), g.add_input()
    lst = g.add_list([a, b])
    c = g.add_cat(lst, 1)
    g.mark_output(c)
    assert (a, b, lst, c) == (0, 1, 2, 3)


def test_rnnt_torchscript_container_roundtrip():
    cfg = syn.RnntConfig(feat_dim=8, enc_hidden=16, pred_hidden=8, joint_hidden=8, vocab=5, blank=4)
    w = syn.make_rnnt_weights(cfg, seed=1)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "rnnt.torchscript")
        syn.save_rnnt_torchscript(path, cfg, w)
        sd = torch.jit.load(path).state_dict()
    assert torch.equal(sd["pre_rnn.weight_hh_l1"], w.pre[5])
    assert torch.equal(sd["joint1.weight"], w.w1)
    assert torch.equal(sd["pred_embed.weight"], w.embedding)


def test_pipeline_manager_rejects_what_it_cannot_run():
    from pimaicompiler_b200.NNCompiler import PipelineManager
    with pytest.raises(NotImplementedError):
        PipelineManager("model.torchscript", "GNMT")
