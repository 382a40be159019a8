"""ctypes binding of ``libhelion_b200.so`` (the C ABI declared in ``include/helion_b200.h``).

The library is loaded lazily on first use.  There is no fallback: if the shared
library has not been built (``python -m helion_b200.build``) or cannot be loaded,
every operator raises ``RuntimeError``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p
from ctypes import c_float
from ctypes import c_int
from ctypes import c_int64
from ctypes import c_void_p
from pathlib import Path
import threading

# HELION_B200_LIB names another build of the library (same ABI), e.g. one with different tuning constants
LIB_PATH = Path(os.environ.get("HELION_B200_LIB") or Path(__file__).resolve().parent / "libhelion_b200.so")

HB200_OK = 0
HB200_ERR_INVALID_ARGUMENT = -1
HB200_ERR_UNSUPPORTED = -2
HB200_ERR_CUDA = -3
HB200_ERR_DEVICE_TIMEOUT = -4
HB200_ERR_WORKSPACE = -5
HB200_ERR_SCRATCH_LIMIT = -6
ABI_VERSION = 1

_P = c_void_p
_I64 = c_int64

# name -> argument types (every entry point returns int unless listed in _RESTYPES)
SIGNATURES: dict[str, list] = {
    "hb200_abi_version": [],
    "hb200_error_string": [c_int],
    "hb200_nvfp4_gemv_bf16in": [_P, _P, _P, _P, _I64, _I64, _I64, c_float, _P],
    "hb200_nvfp4_gemv_bf16in_mma": [_P, _P, _P, _P, _I64, _I64, _I64, c_float, _P],
    "hb200_nvfp4_gemv_fp4in": [_P, _P, _P, _P, _P, _I64, _I64, c_float, _P],
    "hb200_silu_and_mul_per_block_quant": [_P, _P, _P, _I64, _I64, _I64, _I64, c_int, _P, c_int, _P],
    "hb200_silu_and_mul_per_block_quant_typed": [_P, _P, _P, _I64, _I64, _I64, _I64, c_int, _P, c_int, c_int, _P],
    "hb200_rms_norm_dynamic_per_token_quant": [_P, _P, _P, _P, _I64, _I64, c_float, _P, _P, c_int, c_int, _P],
    "hb200_per_token_group_fp8_quant": [_P, _P, _P, _I64, _I64, c_int, c_float, c_float, c_float, c_int, c_int, _P],
    "hb200_nvfp4_quantize": [_P, _P, _P, _P, _I64, _I64, _I64, c_int, _P],
    "hb200_nvfp4_scaled_matmul": [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, c_float, c_int, _P],
    "hb200_device_status": [c_int],
    "hb200_nvfp4_grouped_matmul": [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _P, _P, c_float, c_int, _P],
    "hb200_moe_build_schedule": [_P, _I64, _P, _I64, _P, _P, _I64, _P, _P, _P],
    "hb200_nvfp4_quantize_rows": [_P, _P, _P, _P, _I64, _I64, _I64, _P, c_int, _P, _P, c_int, _P],
    "hb200_grouped_gemm_f16": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, c_int, _P],
    "hb200_build_row_tiles": [_P, _I64, _P, _I64, _P],
    "hb200_moe_gather_rows": [_P, _P, _P, _P, _P, _P, _P, c_int, _P, _I64, _I64, _P],
    "hb200_moe_combine": [_P, _I64, _P, _P, _P, _I64, _I64, _I64, _P],
    "hb200_rms_norm_per_block_quant": [_P, _P, _P, _P, _I64, _I64, c_float, _P, _P, c_int, _I64, _I64, c_int, c_int, _P],
    "hb200_dynamic_per_token_scaled_fp8_quant": [_P, _P, _P, _I64, _I64, _P, c_int, _P],
    "hb200_moe_build_schedule_256": [_P, _I64, _P, _I64, _P, _P, _I64, _P, _P, _P],
    "hb200_nvfp4_grouped_matmul_256": [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _P, _P, c_float, c_int, _P],
    "hb200_moe_sort_pairs": [_P, c_int, _I64, _I64, _P, _P, _P, _P],
    "hb200_nvfp4_grouped_matmul_silu": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _P, _P, c_float, _P],
    "hb200_nvfp4_grouped_matmul_silu_256": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _P, _P, c_float, _P],
    "hb200_nvfp4_quantize_rows_amax": [_P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _P],
    "hb200_nvfp4_gemv_bf16in_tp": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, c_float, _P],
    "hb200_nvfp4_scaled_matmul_tp": [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, c_float, c_int, _P],
    "hb200_peer_barrier": [_P, _I64, _I64, _P, _P],
    "hb200_nvfp4_gemv_bf16in_rs": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, c_float, _P],
    "hb200_tp_reduce_partials": [_P, _P, _I64, _I64, _I64, _I64, _P],
    "hb200_dense_matmul": [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, c_int, _P],
    "hb200_ag_matmul": [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I64, ctypes.c_uint32, c_int, c_int, _P],
    "hb200_matmul_rs": [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, c_int, _P],
    "hb200_reduce_slots": [_P, _P, _I64, _I64, _I64, _I64, c_int, _P],
    "hb200_nvfp4_gemv_tc_workspace_bytes": [_I64, _I64, _I64, _I64],
    "hb200_moe_route_top_k": [_P, c_int, _I64, _I64, _I64, _P, _P, _P],
    "hb200_silu_mul_fp8": [_P, _P, _P, _I64, _I64, _I64, c_int, _P],
    "hb200_fp8_scaled_mm_workspace_bytes": [_I64, _I64, _I64],
    "hb200_fp8_scaled_mm": [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, c_int, c_int, c_int, c_int, _P,
                            _I64, _P],
    "hb200_nvfp4_gemv_bf16in_tc": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, c_float, _P, _I64, _P],
    "hb200_nvfp4_gemv_fp4in_tc": [_P, _P, _P, _P, _P, _I64, _I64, c_float, _P, _I64, _P],
    "hb200_nvfp4_gemv_bf16in_tc_builtin_scratch": [_P, _P, _P, _P, _I64, _I64, _I64, c_float, _P],
    "hb200_nvfp4_gemv_tc_builtin_scratch_reset": [_P],
    "hb200_nvfp4_gemv_tc_counter_bytes": [],
    "hb200_set_wait_budget_cycles": [_I64],
    "hb200_selftest_bounded_wait": [_P],
    "hb200_selftest_exact_reciprocal": [_P, _P],
    "hb200_build_worklist_tiles": [_P, _I64, _I64, _P, _I64, _P],
    "hb200_build_split_tiles": [_P, c_int, _I64, _I64, _I64, _P, _I64, _P],
    "hb200_nvfp4_quantize_scatter": [_P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _P],
    "hb200_rms_norm_nvfp4_quant": [_P, _P, _P, _P, _P, _I64, _I64, _I64, c_float, _P],
    "hb200_grouped_gemm_f16_direct": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, c_int, _P],
    "hb200_ep_buffer_bytes": [_I64, _I64, _I64, _I64, _I64],
    "hb200_ep_slots": [_I64, _I64, _I64, _I64, _I64],
    "hb200_ep_dispatch": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "hb200_ep_collect": [_P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "hb200_ep_gather": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "hb200_ep_return": [_P, _I64, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "hb200_ep_combine": [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
}
_RESTYPES = {"hb200_error_string": c_char_p, "hb200_nvfp4_gemv_tc_workspace_bytes": c_int64,
             "hb200_nvfp4_gemv_tc_counter_bytes": c_int64, "hb200_ep_buffer_bytes": c_int64, "hb200_ep_slots": c_int64,
             "hb200_fp8_scaled_mm_workspace_bytes": c_int64}

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class HelionB200Error(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA extension first (python -m helion_b200.build); "
                "helion_b200 has no CPU or eager fallback"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, c_int)
        version = lib.hb200_abi_version()
        if version != ABI_VERSION:
            raise RuntimeError(f"libhelion_b200.so has ABI version {version}, expected {ABI_VERSION}")
        _lib = lib
        return lib


def check(status: int, what: str) -> None:
    if status != HB200_OK:
        msg = load().hb200_error_string(status).decode()
        raise HelionB200Error(f"{what} failed with status {status}: {msg}")


def call(name: str, *args) -> None:
    """Invoke entry point ``name`` and raise on a non-zero status."""
    check(getattr(load(), name)(*args), name)
