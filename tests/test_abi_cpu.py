"""CPU-side checks of the boundary: the library loads without a driver, exports every symbol
the header declares, and the Python signature table mirrors the header."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "samb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"\b(samb_[a-z0-9_]+)\s*\(", text)


@pytest.fixture(scope="module")
def lib():
    from segment_anything_fast_b200 import build, _lib
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    from segment_anything_fast_b200 import _lib
    names = _header_functions()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/samb200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_version_and_error_strings(lib):
    assert lib.samb_abi_version() == 1
    assert lib.samb_error_string(0) == b"ok"
    assert b"shape" in lib.samb_error_string(-2)
    assert lib.samb_decode_status(0) == 0
    assert lib.samb_decode_status((0x7E << 24) | (3 << 16) | 5) == -6


def test_argument_errors_are_caught_on_the_host(lib):
    # null pointers / bad sizes must be rejected before any CUDA call (no GPU here)
    assert lib.samb_gemm_bf16(None, 8, None, 8, None, None, 0, 0, None, 8, 1, 8, 8, 0, None, None) == -1
    assert lib.samb_layernorm_bf16(None, None, None, None, 1, 8, 1e-6, 0, 0, None) == -1
    assert lib.samb_selftest_bounded_wait(None, 10, None) == -1
    assert lib.samb_mask_rle(None, 1, 8, 8, None, None, 16, None) == -1
