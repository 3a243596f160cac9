"""CPU-side checks of the boundary: the library builds for sm_100a, loads, and exports every
symbol the public headers declare.  No compute call is made (there is no GPU here)."""
import ctypes
import os
import re

import pytest

from flashlstm_poc_b200 import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return _lib.load()


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return set(re.findall(r"\b(flstm_[A-Za-z0-9_]+|lstm_[a-z_]+)\s*\(", text))


def test_every_declared_symbol_is_exported(lib):
    declared = _declared("flashlstm_b200/engine.h") | _declared("flashlstm/lstm_api.h") | _declared("lstm.hpp")
    assert {"flstm_engine_create", "lstm_forward", "flstm_StreamingLstmBackward"} <= declared
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    for name in _lib.ENGINE_SYMBOLS + _lib.V1_SYMBOLS + _lib.V2_SYMBOLS:
        assert name in declared, f"{name} is bound in _lib.py but not declared in include/"


def test_version_and_error_strings(lib):
    assert b"sm_100a" in lib.flstm_version()
    assert lib.flstm_last_error() is not None


def test_misuse_is_reported_not_fatal(lib):
    # null arguments are rejected before any CUDA call
    assert lib.flstm_engine_create(None, None) == 1
    assert b"null" in lib.flstm_last_error()
    assert lib.flstm_engine_forward(None, 1, None, None, None, None, None, None, None) == 1
    bufs = _lib.LstmBuffers()
    assert lib.lstm_set_execution_mode(ctypes.byref(bufs), 1) != 0  # cudaErrorInvalidValue
    assert lib.lstm_destroy_buffers(ctypes.byref(bufs)) == 0


def test_no_cpu_fallback_without_device(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    cfg = _lib.EngineConfig(1, 1, 2, 4, 4, 4, 1, 0)
    h = ctypes.c_void_p()
    st = lib.flstm_engine_create(ctypes.byref(cfg), ctypes.byref(h))
    assert st == 2 and b"no CPU path" in lib.flstm_last_error()
    from flashlstm_poc_b200.engine import Engine

    with pytest.raises(RuntimeError):
        Engine("f16", 1, 2, 4, 4, 4)


def test_extension_module_exposes_reference_entry_points(lib):
    from flashlstm_poc_b200 import _flashlstm

    assert callable(_flashlstm.streaming_lstm_forward) and callable(_flashlstm.streaming_lstm_backward)
    with pytest.raises(TypeError):
        _flashlstm.streaming_lstm_forward(1, 2, 3)  # the reference's arity is 22
    with pytest.raises(TypeError):
        _flashlstm.streaming_lstm_backward(*([0] * 29))  # and 30
