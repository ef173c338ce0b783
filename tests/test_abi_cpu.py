"""CPU: the C-ABI library loads without a GPU and exports every symbol include/pimb200.h declares."""
import ctypes

from pimaicompiler_b200 import _lib


def test_library_exports_every_declared_symbol(pimlib):
    declared = _lib.declared_symbols()
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(pimlib, name), name
    # the binding table covers the header, no more and no less
    assert sorted(_lib.SIGNATURES) == declared


def test_status_strings(pimlib):
    assert pimlib.pimb200_status_string(_lib.OK) == b"ok"
    assert b"timed" in pimlib.pimb200_status_string(_lib.ERR_TIMEOUT) or b"wait" in pimlib.pimb200_status_string(
        _lib.ERR_TIMEOUT)
    assert pimlib.pimb200_status_string(99) == b"unknown status"


def test_bad_arguments_are_rejected_before_any_launch(pimlib):
    # argument validation happens on the host, so it can be exercised without a device
    assert pimlib.pimb200_gemv_mv(None, None, None, None, 4, 4, 0, None) == _lib.ERR_BAD_ARG
    assert pimlib.pimb200_gemv_mv(1, 1, None, 1, 0, 4, 0, None) == _lib.ERR_BAD_ARG
    assert pimlib.pimb200_gemv_mv(16, 16, None, 16, 4, 4, 7, None) == _lib.ERR_BAD_ARG
    assert pimlib.pimb200_gemv_vm(None, 16, None, 16, 4, 4, 0, None) == _lib.ERR_BAD_ARG
    assert pimlib.pimb200_add_f16(16, 16, 16, 0, 8, 0, None) == _lib.ERR_BAD_ARG
    assert pimlib.pimb200_copy_2d(16, 4, 16, 8, 8, 1, None) == _lib.ERR_BAD_ARG  # pitch < row
    assert pimlib.pimb200_gemm_wx(16, 16, None, 16, 8, 8, 2, 4, 8, 0, 0, None) == _lib.ERR_BAD_ARG  # ldx < K
    h = ctypes.c_void_p()
    assert pimlib.pimb200_lstm_create(None, 4, 1, 0, 8, 8, 1, ctypes.byref(h)) == _lib.ERR_BAD_ARG
    assert pimlib.pimb200_lstm_forward(None, 16, 1, 1, None, None, 16, None, None, 0, None) == _lib.ERR_BAD_ARG
    assert pimlib.pimb200_lstm_destroy(None) == _lib.OK
    assert pimlib.pimb200_init(-1) == _lib.ERR_BAD_ARG


def test_every_exported_entry_point_is_declared(pimlib):
    # the reverse direction: no extern "C" pimb200_* symbol of the library is missing from include/*.h
    import shutil
    import subprocess
    import pytest
    nm = shutil.which("nm")
    if nm is None:
        pytest.skip("binutils nm not available")
    out = subprocess.run([nm, "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = sorted({line.split()[-1] for line in out.splitlines() if line.split() and line.split()[-1].startswith("pimb200_")})
    declared = set(_lib.declared_symbols())
    undeclared = [s for s in exported if s not in declared]
    assert not undeclared, f"exported but not declared in include/*.h: {undeclared}"
