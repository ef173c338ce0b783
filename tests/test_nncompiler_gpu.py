"""GPU: TorchScript files compiled by the reference's own importer and graph passes (built where they lie by
pimaicompiler_b200/runtime/build.py) and executed by this library's runtime through the pybind module `NNCompiler`,
class `PipelineManager` — the harness of the reference's examples/runtime/python/simpleMain.py:28-81 (eager result
`equal` to the compiled one) on toy graphs written here, plus an LSTM / linear model on the hot path."""
import json
import os
import tempfile

import pytest
import torch

from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _module():
    from pimaicompiler_b200.runtime import build as rb
    if not rb.available():
        pytest.skip("the NNCompiler module is built from the reference tree, which is not present on this machine")
    return rb.load()


class AddNet(torch.nn.Module):
    def forward(self, x1, x2):
        y1 = torch.add(x1, 10)
        y2 = torch.add(x2, 5)
        y3 = torch.add(y1, y2)
        return torch.add(y3, 10)


class IfNet(torch.nn.Module):
    def forward(self, x1: torch.Tensor, x2: torch.Tensor, x3: torch.Tensor, x4: torch.Tensor):
        y = torch.add(x1, 20)
        y = torch.add(x2, y)
        z1 = x3.item()
        z2 = x4.item()
        if z1 > 10:
            y = torch.add(y, 15)
            if z2 > 5:
                y = torch.add(y, 25)
            else:
                y = torch.add(y, -25)
        else:
            y = torch.add(y, 100)
        y = torch.add(y, z1)
        return y


class LoopNet(torch.nn.Module):
    def forward(self, x1, x2, n):
        y = x1
        k = int(n.item())
        for i in range(k):
            y = torch.add(y, x2)
            y = torch.add(y, i)
        return torch.add(y, 25)


class NestedLoopNet(torch.nn.Module):
    def forward(self, x1, x2, n):
        y = x1
        z = x2
        k = int(n.item())
        for i in range(k):
            for j in range(2):
                y = torch.add(y, z)
                z = torch.add(z, j)
            if i > 1:
                y = torch.add(y, 100)
        return y, z


def _compile(nn_module, model_type=""):
    mod = _module()
    sm = torch.jit.freeze(torch.jit.script(nn_module.eval()))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "net.torchscript")
        sm.save(path)
        return mod.PipelineManager(path, model_type), sm


def _dev(ts):
    return [t.cuda() for t in ts]


def test_add_net_equal():
    pm, sm = _compile(AddNet())
    x1, x2 = torch.tensor([[1, 2, 3], [4, 5, 6]]), torch.tensor([[10, 20, 20], [40, 50, 60]])
    (out,) = pm.inferenceModel(_dev([x1, x2]))
    assert torch.equal(out.cpu(), sm(x1, x2))


@pytest.mark.parametrize("z1,z2", [(20, 9), (20, 1), (3, 9)])
def test_nested_if_net_equal(z1, z2):
    pm, sm = _compile(IfNet())
    x1, x2 = torch.tensor([[1, 2, 3], [4, 5, 6]]), torch.tensor([[10, 20, 20], [40, 50, 60]])
    ins = [x1, x2, torch.tensor(z1), torch.tensor(z2)]
    (out,) = pm.inferenceModel(_dev(ins))
    assert torch.equal(out.cpu(), sm(*ins))


@pytest.mark.parametrize("trips", [0, 1, 3, 5])
def test_loop_nets_equal(trips):
    x1, x2 = torch.tensor([[1, 2, 3], [4, 5, 6]]), torch.tensor([[20, 2, 30], [-4, 50, 70]])
    n = torch.tensor(trips)
    pm, sm = _compile(LoopNet())
    (out,) = pm.inferenceModel(_dev([x1, x2, n]))
    assert torch.equal(out.cpu(), sm(x1, x2, n))
    # the same compiled model again with another trip count: loop state must not leak between runs
    n2 = torch.tensor(trips + 2)
    (out2,) = pm.inferenceModel(_dev([x1, x2, n2]))
    assert torch.equal(out2.cpu(), sm(x1, x2, n2))
    pm2, sm2 = _compile(NestedLoopNet())
    y, z = pm2.inferenceModel(_dev([x1, x2, n]))
    ry, rz = sm2(x1, x2, n)
    assert torch.equal(y.cpu(), ry) and torch.equal(z.cpu(), rz)


class LstmFc(torch.nn.Module):
    """aten::lstm (padded overload, flat parameter list) followed by linear + relu + linear: the importer lifts the
    LSTM weights, ConvertLinearToAddmm / SwapAddmmInputs / FuseActivation turn the linears into addmm(b, W, x^T) with the
    activation folded in."""

    def __init__(self, I=240, H=256, L=2, N1=64, N2=29):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        k = 1.0 / H ** 0.5

        def u(*s):
            return ((torch.rand(*s, generator=g) * 2 - 1) * k).half()
        self.w_ih0, self.w_hh0, self.b_ih0, self.b_hh0 = u(4 * H, I), u(4 * H, H), u(4 * H), u(4 * H)
        self.w_ih1, self.w_hh1, self.b_ih1, self.b_hh1 = u(4 * H, H), u(4 * H, H), u(4 * H), u(4 * H)
        self.fc = torch.nn.Linear(H, N1)
        self.fc2 = torch.nn.Linear(N1, N2)

    def forward(self, x, h0, c0):
        y, hn, cn = torch.lstm(x, [h0, c0], [self.w_ih0, self.w_hh0, self.b_ih0, self.b_hh0, self.w_ih1, self.w_hh1,
                                             self.b_ih1, self.b_hh1], True, 2, 0.0, False, False, False)
        z = torch.relu(self.fc(y))
        return self.fc2(z), hn, cn


@pytest.mark.parametrize("T", [1, 40])
def test_lstm_and_linear_model_through_the_reference_compiler(T):
    mod = _module()
    m = LstmFc().half()
    pm, sm = _compile(m)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, 1, 240, generator=g).half()
    h0 = (torch.randn(2, 1, 256, generator=g) * 0.5).half()
    c0 = (torch.randn(2, 1, 256, generator=g) * 0.5).half()
    mod.reset_fallback_count()
    logits, hn, cn = pm.inferenceModel(_dev([x, h0, c0]))
    assert mod.fallback_count() == 0, "a hot-path op fell back to the library call"
    m = m.float()
    for name in ("w_ih0", "w_hh0", "b_ih0", "b_hh0", "w_ih1", "w_hh1", "b_ih1", "b_hh1"):   # plain attributes, not parameters
        setattr(m, name, getattr(m, name).float())
    with torch.backends.mkldnn.flags(enabled=False):   # oneDNN has no LSTM primitive for every shape on every host
        ref = m(x.float(), h0.float(), c0.float())
    assert logits.shape == ref[0].shape
    assert_close(logits, ref[0], 2e-2, 1e-2, "logits")
    assert_close(hn, ref[1], 4e-3, 4e-3, "h_n")
    assert_close(cn, ref[2], 4e-3, 4e-3, "c_n")
    # a second run reuses the preloaded constants and packed weights
    logits2, _, _ = pm.inferenceModel(_dev([x, h0, c0]))
    assert torch.equal(logits2, logits)


def test_profiling_flag_writes_a_chrome_trace():
    mod = _module()
    sm = torch.jit.freeze(torch.jit.script(LstmFc().half().eval()))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "net.torchscript")
        sm.save(path)
        pm = mod.PipelineManager(path, "", 1, True)
        trace_path = os.path.join(d, "trace.json")
        pm.setProfilePath(trace_path)
        g = torch.Generator().manual_seed(2)
        ins = [torch.randn(5, 1, 240, generator=g).half(), torch.zeros(2, 1, 256).half(), torch.zeros(2, 1, 256).half()]
        pm.inferenceModel(_dev(ins))
        with open(trace_path) as f:
            ev = json.load(f)["traceEvents"]
    names = [e["name"] for e in ev]
    assert any("lstm" in n for n in names) and sum("addmm" in n for n in names) == 2
    assert all(e["ph"] == "X" and e["dur"] >= 0 for e in ev)


class MlpNet(torch.nn.Module):
    """Row-wise independent: linear (tensor-core GEMM at 64 rows x 4096 outputs) + relu + linear."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(3)
        self.fc = torch.nn.Linear(256, 4096)
        self.fc2 = torch.nn.Linear(4096, 64)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc(x)))


def test_two_gpu_replicas_match_one_gpu():
    # PipelineManager(..., gpu_num=2): one runtime per device on its own thread (the reference's thread-per-GPU replicas,
    # examples/runtime/source/pipeline_manager.cpp:27-53), inputs chunked along dimension 0.  Every device sets its own
    # kernel attributes and packs its own weights; the result must equal the one-GPU run bit for bit.
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mod = _module()
    sm = torch.jit.freeze(torch.jit.script(MlpNet().half().eval()))
    g = torch.Generator().manual_seed(5)
    x = torch.randn(128, 256, generator=g).half()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "net.torchscript")
        sm.save(path)
        one = mod.PipelineManager(path, "", 1)
        two = mod.PipelineManager(path, "", 2)
        (ref,) = one.inferenceModel([x.cuda()])
        mod.reset_fallback_count()
        for _ in range(3):
            (out,) = two.inferenceModel([x.cuda()])
            assert out.shape == ref.shape
            assert torch.equal(out.cpu(), ref.cpu())
        assert mod.fallback_count() == 0
        del one, two
    add = AddNet()
    pm2, sm_add = _compile(add)
    a = torch.arange(12, dtype=torch.int64).view(4, 3)
    b = torch.ones(4, 3, dtype=torch.int64)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "add.torchscript")
        torch.jit.freeze(torch.jit.script(add.eval())).save(path)
        two = mod.PipelineManager(path, "", 2)
        (out,) = two.inferenceModel([a.cuda(), b.cuda()])
        assert torch.equal(out.cpu(), sm_add(a, b))


class TopkNet(torch.nn.Module):
    def forward(self, x):
        v, i = torch.topk(x, 3)
        return v, i


def test_topk_through_the_compiler_uses_the_device_kernel():
    mod = _module()
    pm, sm = _compile(TopkNet())
    g = torch.Generator().manual_seed(9)
    x = torch.randn(2, 300, generator=g).half()
    mod.reset_fallback_count()
    v, i = pm.inferenceModel(_dev([x]))
    assert mod.fallback_count() == 0
    rv, ri = sm(x.float())
    assert torch.equal(v.float().cpu(), rv) and torch.equal(i.cpu(), ri)
