"""The C-ABI library loads, exports every symbol include/oxq.h declares, and
rejects bad arguments with a status (no GPU work is launched here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from oxydllm_b200 import _lib
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "oxq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(oxq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = _declared()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/oxq.h but not exported"


def test_bindings_cover_the_header():
    from oxydllm_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()


def test_status_strings(lib):
    assert lib.oxq_status_string(0) == b"ok"
    assert lib.oxq_status_string(-1) == b"bad shape"
    assert lib.oxq_version() >= 1


def test_argument_validation_returns_status(lib):
    from oxydllm_b200 import _lib
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(256)  # never dereferenced: validation fails first
    with pytest.raises(_lib.OxqError) as e:
        _lib.call("oxq_awq_dequant", null, null, null, 1, null, 0, 8, 16, 4, null)
    assert e.value.status == -4
    with pytest.raises(_lib.OxqError, match="not divisible by pack factor 8"):
        _lib.call("oxq_awq_dequant", one, one, one, 1, one, 0, 8, 12, 4, null)
    with pytest.raises(_lib.OxqError, match="outside 1..32"):
        _lib.call("oxq_awq_gemv", one, 2, one, one, one, 1, null, 0, one, 2, 33, 256, 128, 64, null)
    with pytest.raises(_lib.OxqError, match="must be bf16"):
        _lib.call("oxq_awq_gemv", one, 0, one, one, one, 1, null, 0, one, 2, 1, 256, 128, 64, null)
    with pytest.raises(_lib.OxqError, match="only 4/8-bit"):
        _lib.call("oxq_gptq_dequant", one, one, one, 1, one, 0, 32, 16, 16, 3, 0, null)
    with pytest.raises(_lib.OxqError, match="unsupported GGML type"):
        _lib.call("oxq_gguf_dequant", 99, one, one, 0, 4, 256, null)
    with pytest.raises(_lib.OxqError, match="multiple of the block size"):
        _lib.call("oxq_gguf_gemv", 12, one, 2, one, null, 0, one, 2, 1, 100, 8, null)
    with pytest.raises(_lib.OxqError, match="does not tile weight"):
        _lib.call("oxq_fp8_dequant", one, one, 3, 2, one, 0, 4, 4, null)
    with pytest.raises(_lib.OxqError, match="multiple of 32"):
        _lib.call("oxq_mxfp4_dequant", one, one, one, 0, 2, 48, null)
