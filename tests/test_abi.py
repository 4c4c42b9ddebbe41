"""The C-ABI library: loads, exports every symbol the header declares, and fails loudly
(no CPU fallback) when there is no usable device. No compute calls here."""
import ctypes
import os
import re

import pytest

from rllama_b200 import _ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "rllama_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rlb_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_in_tree():
    assert os.path.exists(_ffi.LIB_PATH), "run `python -m rllama_b200.build`"


def test_exports_every_declared_symbol():
    lib = ctypes.CDLL(_ffi.LIB_PATH)
    declared = header_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(lib, name), "header declares %s but the library does not export it" % name
    assert sorted(_ffi.EXPORTS) == declared


def test_header_cites_the_reference_interface():
    text = open(os.path.join(ROOT, "include", "rllama_b200.h")).read()
    assert text.count("src/tensor_opencl_support.rs") >= 10
    assert text.count("src/transformer.rs") >= 10


def test_no_cpu_fallback_without_device():
    lib = _ffi.lib()
    n = ctypes.c_int(-1)
    lib.rlb_device_count(ctypes.byref(n))
    if n.value > 0:
        pytest.skip("a CUDA device is present")
    h = ctypes.c_void_p()
    rc = lib.rlb_ctx_create(0, 0, ctypes.byref(h))
    assert rc == 3 and not h.value  # RLB_ERR_NO_DEVICE
    assert b"no CPU fallback" in lib.rlb_last_error()
    with pytest.raises(_ffi.RllamaError):
        from rllama_b200 import Cuda
        Cuda()


def test_null_arguments_are_errors_not_crashes():
    lib = _ffi.lib()
    assert lib.rlb_ctx_flush(None) == 1
    assert lib.rlb_tensor_wait(None) == 1
    assert lib.rlb_model_finalize(None) == 1
    assert lib.rlb_forward(None, None, None, 1, 0, None) == 1
    assert lib.rlb_model_create(None, None, None) == 1
