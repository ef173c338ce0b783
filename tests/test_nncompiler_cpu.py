"""CPU: the NNCompiler module (reference front end compiled in place + this library's runtime) loads and exposes the
reference's Python surface (runtime/python/nn_runtime_py.cpp:18-25).  Skipped where the module was never built."""
import pytest


def _module():
    from pimaicompiler_b200.runtime import build as rb
    if not rb.available():
        pytest.skip("the NNCompiler module is built from the reference tree, which is not present on this machine")
    return rb.load()


def test_module_exposes_pipeline_manager():
    mod = _module()
    assert mod.__name__ == "NNCompiler"
    doc = mod.PipelineManager.__init__.__doc__
    assert "input_file" in doc and "model_type" in doc and "gpu_num" in doc
    assert hasattr(mod.PipelineManager, "inferenceModel")
    assert mod.fallback_count() == 0
