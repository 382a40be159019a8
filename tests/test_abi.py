"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""

from __future__ import annotations

import ctypes
from pathlib import Path
import re

import pytest

from helion_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "helion_b200.h"


def _declared() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"\b(hb200_\w+)\s*\(", text)


def test_header_declares_entry_points():
    names = _declared()
    assert "hb200_nvfp4_gemv_bf16in" in names and "hb200_abi_version" in names
    assert len(names) == len(set(names))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in _declared():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in _declared(), f"{name} is bound but not declared in the header"


def test_version_and_error_strings():
    lib = _lib.load()
    assert lib.hb200_abi_version() == _lib.ABI_VERSION
    assert lib.hb200_error_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5, -99):
        assert len(lib.hb200_error_string(code)) > 0


def test_argument_validation_happens_before_any_cuda_call():
    """Bad arguments are rejected on the host (no device needed)."""
    lib = _lib.load()
    assert lib.hb200_nvfp4_gemv_bf16in(None, None, None, None, 8, 32, 1, 1.0, None) == -1
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p16 = (p + 15) // 16 * 16
    assert lib.hb200_nvfp4_gemv_bf16in(p16, p16, p16, p16, 8, 24, 1, 1.0, None) == -1  # K % 16 != 0
    assert lib.hb200_nvfp4_gemv_bf16in(p16, p16, p16, p16, 8, 32, 33, 1.0, None) == -2  # batch > 32
    assert lib.hb200_silu_and_mul_per_block_quant(p16, p16, p16, 4, 96, 192, 96, 32, None, 0, None) == -1
    assert lib.hb200_per_token_group_fp8_quant(p16, p16, p16, 4, 96, 48, 1e-10, -448.0, 448.0, 0, 0, None) == -2
    with pytest.raises(_lib.HelionB200Error, match="invalid argument"):
        _lib.call("hb200_nvfp4_quantize", None, None, None, None, 1, 16, 16, 0, None)
