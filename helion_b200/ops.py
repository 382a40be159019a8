"""Operator surface: the reference's Python entry points, backed by the sm_100a C ABI.

Every public function here keeps the call signature, tensor layouts, validation
order and error messages of the reference entry point named in its docstring, so
it can be swapped in for it.  The device work is registered as ``torch.library``
custom ops in the ``helion_b200`` namespace (with fake implementations for
tracing); the custom ops call ``libhelion_b200.so`` through ctypes on the current
CUDA stream.  There is no CPU or eager fallback: non-CUDA tensors raise.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch
from torch import Tensor

from . import _lib
from .layouts import fp4_storage
from .layouts import swizzled_scale_numel

_FP8 = torch.float8_e4m3fn


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "helion_b200 operators run on CUDA (sm_100a) tensors only; there is no CPU fallback "
                f"(got a tensor on {t.device})"
            )


def _ptr(t: Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------ validators
# Same checks and messages as examples/nvfp4_gemv.py:111-149.
def _check_swizzled_scales(name: str, scales: Tensor, rows: int, cols: int) -> None:
    expected = swizzled_scale_numel(rows, cols)
    if scales.numel() != expected:
        raise ValueError(
            f"{name} must contain {expected} SWIZZLE_32_4_4 scale values "
            f"for logical shape ({rows}, {cols}); got {scales.numel()}"
        )


def _check_contiguous(name: str, t: Tensor) -> None:
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _check_fp4_weight_storage(name: str, storage: Tensor) -> None:
    if storage.dim() != 2:
        raise ValueError(f"{name} must be a 2D packed FP4 tensor")
    if storage.shape[1] % 8 != 0:
        raise ValueError(f"{name} K bytes must be divisible by 8; got {storage.shape[1]}")


def _check_numel(name: str, t: Tensor, expected: int) -> None:
    if t.numel() != expected:
        raise ValueError(f"{name} must contain {expected} values; got {t.numel()}")


# ------------------------------------------------------------------ custom ops
# Workspace of the tensor-core GEMV and of scaled_mm's stream-K form (activation terms, split-K partials, tile
# arrival counters): one buffer per (device, stream), grown on demand, cached under a lock.  Calls on one stream
# are ordered, so they can share it.  Only the first _COUNTER_BYTES (the arrival counters) must be zero between
# calls; the kernels leave them zero unless a bounded wait ran out or two calls overlapped on the device
# (see device_status).
_SCALED_MM_OUT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_COUNTER_BYTES = 16384
_TC_WORKSPACES: dict[tuple[int, int | str], Tensor] = {}
_TC_RETIRED: list[Tensor] = []  # outgrown graph workspaces, kept alive for the graphs that captured them
_TC_LOCK = threading.Lock()
_TC_MIN_BYTES = 1 << 22
_TC_MIN_WEIGHT_ELEMS = int(os.environ.get("HB200_TC_MIN_ELEMS", 1 << 21))  # below this the SIMT kernel is faster alone
# a single row: measured alone (19 to 66 MB of weights) the SIMT kernel is 2 to 6 us faster; from about 130 MB on
# the tensor-core kernel wins (8192 x 28672: 36.9 against 38.9 us, 57344 x 8192: 55 against 65 us)
_TC_MIN_WEIGHT_ELEMS_1ROW = int(os.environ.get("HB200_TC_MIN_ELEMS_1ROW", 100_000_000))


def tc_workspace(device: torch.device, nbytes: int) -> Tensor:
    """The workspace for calls on the current stream of ``device``.

    While a CUDA graph is being captured the stream is the capture's own, so a look-up by stream would allocate
    (and zero-fill) inside the capture and the fill would be replayed with every step.  Captured calls therefore
    use one workspace per device that is set aside for graphs: it is allocated, outside any capture, together
    with the first ordinary workspace of the device or by :func:`reserve_graph_workspace`.  Graphs replayed
    at the same time on two streams of one device need workspaces of their own (pass them to the C ABI).
    """
    index = device.index if device.index is not None else torch.cuda.current_device()
    capturing = torch.cuda.is_current_stream_capturing()
    key = (index, "graph") if capturing else (index, _stream() or 0)
    with _TC_LOCK:
        ws = _TC_WORKSPACES.get(key)
        if ws is None or ws.numel() < nbytes:
            if capturing and ws is not None:
                raise RuntimeError(
                    f"the tensor-core workspace set aside for CUDA graphs holds {ws.numel()} bytes but this call "
                    f"needs {nbytes}: run the call once outside the capture (warm-up) or call "
                    "helion_b200.ops.reserve_graph_workspace(device, nbytes) before capturing"
                )
            # (a first use inside a capture allocates in the graph's pool: correct, but the fill is replayed)
            ws = torch.zeros(max(nbytes, _TC_MIN_BYTES), dtype=torch.uint8, device=device)
            _TC_WORKSPACES[key] = ws
        if not capturing:
            _grow_graph_workspace(index, device, nbytes)  # what ran eagerly (a warm-up) can be captured next
        return ws


def _grow_graph_workspace(index: int, device: torch.device, nbytes: int) -> None:
    """(lock held, not capturing)  Graphs captured earlier keep the address of the workspace they were captured
    with, so an outgrown one is retired, not freed."""
    gw = _TC_WORKSPACES.get((index, "graph"))
    if gw is None or gw.numel() < nbytes:
        if gw is not None:
            _TC_RETIRED.append(gw)
        _TC_WORKSPACES[(index, "graph")] = torch.zeros(max(nbytes, _TC_MIN_BYTES), dtype=torch.uint8, device=device)


def reserve_graph_workspace(device: torch.device, nbytes: int) -> None:
    """Make the workspace that captured calls on ``device`` use at least ``nbytes`` large (call outside capture)."""
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("reserve_graph_workspace must be called outside stream capture")
    index = device.index if device.index is not None else torch.cuda.current_device()
    with _TC_LOCK:
        _grow_graph_workspace(index, device, nbytes)


def device_status(reset: bool = False) -> int:
    """Sticky status of the current device's kernels (0, or ``HB200_ERR_DEVICE_TIMEOUT`` once a bounded
    device-side wait ran out); synchronises the device.  With ``reset`` a non-zero status is cleared and, because
    a kernel that gave up can leave tile arrival counters non-zero (every later call on that workspace would then
    leave tiles unwritten), the counter region of every cached workspace of the device is zeroed again."""
    status = int(_lib.load().hb200_device_status(1 if reset else 0))
    if reset and status != 0:
        index = torch.cuda.current_device()
        with _TC_LOCK:
            for (dev, _), ws in _TC_WORKSPACES.items():
                if dev == index:
                    ws[:_COUNTER_BYTES].zero_()
            for ws in _TC_RETIRED:
                if ws.device.index == index:
                    ws[:_COUNTER_BYTES].zero_()
        torch.cuda.synchronize()
    return status


def _tc_eligible(n: int, k: int, batch: int) -> bool:
    floor = _TC_MIN_WEIGHT_ELEMS_1ROW if batch == 1 else _TC_MIN_WEIGHT_ELEMS
    return k % 32 == 0 and n >= 128 and 1 <= batch <= 32 and n * k >= floor


def _gemv_path(path: str, n: int, k: int, batch: int) -> str:
    if path == "auto":
        # The tensor-core kernel streams the large matrices of a 70B-class layer faster than the SIMT one and its
        # cost barely grows with rows; small matrices (latency-bound) and K % 32 != 0 stay on SIMT.
        return "tc" if _tc_eligible(n, k, batch) else "simt"
    if path not in ("simt", "mma", "tc"):
        raise ValueError(f"path must be 'auto', 'simt', 'mma' or 'tc'; got {path!r}")
    return path


@torch.library.custom_op("helion_b200::nvfp4_gemv_bf16in", mutates_args=())
def _gemv_bf16in_op(weight_bytes: Tensor, x: Tensor, weight_scale: Tensor, alpha: float, path: str) -> Tensor:
    _require_cuda(weight_bytes, x, weight_scale)
    n, k_bytes = weight_bytes.shape
    k = k_bytes * 2
    batch = x.numel() // k if k else 1
    out = torch.empty((batch, n), dtype=torch.bfloat16, device=weight_bytes.device)
    if n and batch:
        path = _gemv_path(path, n, k, batch)
        with torch.cuda.device(weight_bytes.device):
            if path == "tc":
                need = _lib.load().hb200_nvfp4_gemv_tc_workspace_bytes(n, k, batch, 4)
                if need < 0:
                    _lib.check(int(need), "hb200_nvfp4_gemv_tc_workspace_bytes")
                ws = tc_workspace(weight_bytes.device, need)
                ptrs = (ctypes.c_void_p * 1)(out.data_ptr())
                _lib.call(
                    "hb200_nvfp4_gemv_bf16in_tc", weight_bytes.data_ptr(), x.data_ptr(), weight_scale.data_ptr(), ptrs, 1,
                    n, k, batch, n, 0, float(alpha), ws.data_ptr(), ws.numel(), _stream(),
                )
            else:
                _lib.call(
                    "hb200_nvfp4_gemv_bf16in_mma" if path == "mma" else "hb200_nvfp4_gemv_bf16in",
                    weight_bytes.data_ptr(), x.data_ptr(), weight_scale.data_ptr(), out.data_ptr(),
                    n, k, batch, float(alpha), _stream(),
                )
    return out


@_gemv_bf16in_op.register_fake
def _(weight_bytes, x, weight_scale, alpha, path):
    k = weight_bytes.shape[1] * 2
    batch = x.numel() // k if k else 1
    return weight_bytes.new_empty((batch, weight_bytes.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op("helion_b200::nvfp4_gemv_fp4in", mutates_args=())
def _gemv_fp4in_op(weight_bytes: Tensor, x_bytes: Tensor, weight_scale: Tensor, x_scale: Tensor, alpha: float,
                   path: str) -> Tensor:
    _require_cuda(weight_bytes, x_bytes, weight_scale, x_scale)
    n, k_bytes = weight_bytes.shape
    out = torch.empty((n,), dtype=torch.bfloat16, device=weight_bytes.device)
    if n:
        path = _gemv_path(path, n, k_bytes * 2, 1)
        with torch.cuda.device(weight_bytes.device):
            if path == "tc":
                need = _lib.load().hb200_nvfp4_gemv_tc_workspace_bytes(n, k_bytes * 2, 1, 1)
                if need < 0:
                    _lib.check(int(need), "hb200_nvfp4_gemv_tc_workspace_bytes")
                ws = tc_workspace(weight_bytes.device, need)
                _lib.call(
                    "hb200_nvfp4_gemv_fp4in_tc", weight_bytes.data_ptr(), x_bytes.data_ptr(), weight_scale.data_ptr(),
                    x_scale.data_ptr(), out.data_ptr(), n, k_bytes * 2, float(alpha), ws.data_ptr(), ws.numel(), _stream(),
                )
            else:
                _lib.call(
                    "hb200_nvfp4_gemv_fp4in",
                    weight_bytes.data_ptr(), x_bytes.data_ptr(), weight_scale.data_ptr(), x_scale.data_ptr(),
                    out.data_ptr(), n, k_bytes * 2, float(alpha), _stream(),
                )
    return out


@_gemv_fp4in_op.register_fake
def _(weight_bytes, x_bytes, weight_scale, x_scale, alpha, path):
    return weight_bytes.new_empty((weight_bytes.shape[0],), dtype=torch.bfloat16)


@torch.library.custom_op("helion_b200::silu_and_mul_per_block_quant", mutates_args=("out", "scales"))
def _silu_mul_quant_op(out: Tensor, input: Tensor, scales: Tensor, group_size: int, scale_ub: Tensor | None) -> None:  # noqa: A002
    _require_cuda(out, input, scales, scale_ub)
    tokens, two_i = input.shape
    with torch.cuda.device(input.device):
        _lib.call(
            "hb200_silu_and_mul_per_block_quant_typed",
            out.data_ptr(), input.data_ptr(), scales.data_ptr(), tokens, two_i // 2,
            input.stride(0), out.stride(0), group_size, _ptr(scale_ub), int(out.dtype == torch.int8),
            {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[input.dtype], _stream(),
        )


@_silu_mul_quant_op.register_fake
def _(out, input, scales, group_size, scale_ub):  # noqa: A002
    return None


@torch.library.custom_op(
    "helion_b200::rms_norm_dynamic_per_token_quant", mutates_args=("result", "scale", "residual")
)
def _rms_quant_op(
    result: Tensor, input: Tensor, weight: Tensor, scale: Tensor, epsilon: float,  # noqa: A002
    scale_ub: Tensor | None, residual: Tensor | None,
) -> None:
    _require_cuda(result, input, weight, scale, scale_ub, residual)
    tokens, hidden = input.shape
    with torch.cuda.device(input.device):
        _lib.call(
            "hb200_rms_norm_dynamic_per_token_quant",
            result.data_ptr(), input.data_ptr(), weight.data_ptr(), scale.data_ptr(), tokens, hidden,
            float(epsilon), _ptr(scale_ub), _ptr(residual), int(input.dtype == torch.float16),
            int(result.dtype == torch.int8), _stream(),
        )


@_rms_quant_op.register_fake
def _(result, input, weight, scale, epsilon, scale_ub, residual):  # noqa: A002
    return None


@torch.library.custom_op("helion_b200::rms_norm_per_block_quant", mutates_args=("result", "scale", "residual"))
def _rms_block_quant_op(
    result: Tensor, input: Tensor, weight: Tensor, scale: Tensor, epsilon: float,  # noqa: A002
    scale_ub: Tensor | None, residual: Tensor | None, group_size: int,
) -> None:
    _require_cuda(result, input, weight, scale, scale_ub, residual)
    tokens, hidden = input.shape
    with torch.cuda.device(input.device):
        _lib.call(
            "hb200_rms_norm_per_block_quant",
            result.data_ptr(), input.data_ptr(), weight.data_ptr(), scale.data_ptr(), tokens, hidden,
            float(epsilon), _ptr(scale_ub), _ptr(residual), group_size, scale.stride(0), scale.stride(1),
            int(input.dtype == torch.float16), int(result.dtype == torch.int8), _stream(),
        )


@_rms_block_quant_op.register_fake
def _(result, input, weight, scale, epsilon, scale_ub, residual, group_size):  # noqa: A002
    return None


@torch.library.custom_op("helion_b200::dynamic_per_token_scaled_fp8_quant", mutates_args=("result", "scale"))
def _dyn_token_quant_op(result: Tensor, input: Tensor, scale: Tensor, scale_ub: Tensor | None) -> None:  # noqa: A002
    _require_cuda(result, input, scale, scale_ub)
    tokens, hidden = input.shape
    with torch.cuda.device(input.device):
        _lib.call(
            "hb200_dynamic_per_token_scaled_fp8_quant",
            result.data_ptr(), input.data_ptr(), scale.data_ptr(), tokens, hidden, _ptr(scale_ub),
            int(input.dtype == torch.float16), _stream(),
        )


@_dyn_token_quant_op.register_fake
def _(result, input, scale, scale_ub):  # noqa: A002
    return None


@torch.library.custom_op("helion_b200::silu_mul_fp8", mutates_args=())
def _silu_mul_fp8_op(input: Tensor, scale: Tensor) -> Tensor:  # noqa: A002
    _require_cuda(input, scale)
    tokens, two_d = input.shape
    d = two_d // 2
    out = torch.empty((tokens, d), dtype=_FP8, device=input.device)
    if tokens and d:
        with torch.cuda.device(input.device):
            _lib.call(
                "hb200_silu_mul_fp8", out.data_ptr(), input.data_ptr(), scale.data_ptr(), tokens, d, input.stride(0),
                int(input.dtype == torch.float16), _stream(),
            )
    return out


@_silu_mul_fp8_op.register_fake
def _(input, scale):  # noqa: A002
    return torch.empty((input.shape[0], input.shape[1] // 2), dtype=_FP8, device=input.device)


@torch.library.custom_op("helion_b200::scaled_mm", mutates_args=("c",))
def _scaled_mm_op(c: Tensor, a: Tensor, b_nk: Tensor, scale_a: Tensor, scale_b: Tensor, bias: Tensor | None) -> None:
    _require_cuda(c, a, b_nk, scale_a, scale_b, bias)
    m, k = a.shape
    n = b_nk.shape[0]
    lib = _lib.load()
    with torch.cuda.device(a.device):
        need = lib.hb200_fp8_scaled_mm_workspace_bytes(m, n, k)
        ws = tc_workspace(a.device, need) if need else None
        _lib.call(
            "hb200_fp8_scaled_mm",
            a.data_ptr(), b_nk.data_ptr(), c.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(), _ptr(bias),
            m, n, k, a.stride(0), b_nk.stride(0), c.stride(0),
            int(scale_a.numel() > 1), int(scale_b.numel() > 1),
            2 if a.dtype is torch.int8 else int(a.dtype is torch.float8_e5m2), _SCALED_MM_OUT[c.dtype],
            _ptr(ws), ws.numel() if ws is not None else 0, _stream(),
        )


@_scaled_mm_op.register_fake
def _(c, a, b_nk, scale_a, scale_b, bias):
    return None


@torch.library.custom_op("helion_b200::per_token_group_fp8_quant", mutates_args=("output_q", "output_s"))
def _group_quant_op(
    input: Tensor, output_q: Tensor, output_s: Tensor, group_size: int, eps: float,  # noqa: A002
    fp8_min: float, fp8_max: float, scale_ue8m0: bool,
) -> None:
    _require_cuda(input, output_q, output_s)
    tokens, hidden = input.shape
    dtype_code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[input.dtype]
    with torch.cuda.device(input.device):
        _lib.call(
            "hb200_per_token_group_fp8_quant",
            input.data_ptr(), output_q.data_ptr(), output_s.data_ptr(), tokens, hidden, group_size,
            float(eps), float(fp8_min), float(fp8_max), int(scale_ue8m0), dtype_code, _stream(),
        )


@_group_quant_op.register_fake
def _(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0):  # noqa: A002
    return None


@torch.library.custom_op("helion_b200::nvfp4_quantize", mutates_args=())
def _nvfp4_quantize_op(x: Tensor, global_scale: Tensor | None) -> tuple[Tensor, Tensor, Tensor]:
    _require_cuda(x, global_scale)
    rows, k = x.shape
    per_token = global_scale is None
    codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    numel = swizzled_scale_numel(rows, k // 16)
    padded = rows % 128 != 0 or (k // 16) % 4 != 0
    scales = (torch.zeros if padded else torch.empty)(numel, dtype=torch.uint8, device=x.device)
    g = torch.empty((rows,), dtype=torch.float32, device=x.device) if per_token else global_scale.reshape(1).clone()
    if rows and k:
        with torch.cuda.device(x.device):
            _lib.call(
                "hb200_nvfp4_quantize", x.data_ptr(), codes.data_ptr(), scales.data_ptr(), g.data_ptr(),
                rows, k, x.stride(0), int(per_token), _stream(),
            )
    return codes, scales.view(_FP8), g


@_nvfp4_quantize_op.register_fake
def _(x, global_scale):
    rows, k = x.shape
    g = x.new_empty((rows,) if global_scale is None else (1,), dtype=torch.float32)
    return (
        x.new_empty((rows, k // 2), dtype=torch.uint8),
        x.new_empty((swizzled_scale_numel(rows, k // 16),), dtype=_FP8),
        g,
    )


def _nvfp4_row_outputs(x: Tensor, rows: int, k: int):
    codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    padded = rows % 128 != 0 or (k // 16) % 4 != 0
    scales = (torch.zeros if padded else torch.empty)(swizzled_scale_numel(rows, k // 16), dtype=torch.uint8, device=x.device)
    return codes, scales, torch.empty((rows,), dtype=torch.float32, device=x.device)


@torch.library.custom_op("helion_b200::rms_norm_nvfp4_quant", mutates_args=())
def _rms_norm_nvfp4_op(x: Tensor, weight: Tensor, epsilon: float) -> tuple[Tensor, Tensor, Tensor]:
    _require_cuda(x, weight)
    rows, k = x.shape
    codes, scales, g = _nvfp4_row_outputs(x, rows, k)
    if rows and k:
        with torch.cuda.device(x.device):
            _lib.call("hb200_rms_norm_nvfp4_quant", x.data_ptr(), weight.data_ptr(), codes.data_ptr(), scales.data_ptr(),
                      g.data_ptr(), rows, k, x.stride(0), float(epsilon), _stream())
    return codes, scales.view(_FP8), g


@torch.library.custom_op("helion_b200::silu_and_mul_nvfp4_quant", mutates_args=())
def _silu_mul_nvfp4_op(x: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    _require_cuda(x)
    rows, two_k = x.shape
    k = two_k // 2
    codes, scales, g = _nvfp4_row_outputs(x, rows, k)
    if rows and k:
        with torch.cuda.device(x.device):
            _lib.call("hb200_nvfp4_quantize_rows", x.data_ptr(), codes.data_ptr(), scales.data_ptr(), g.data_ptr(),
                      rows, k, x.stride(0), None, 1, None, None, 1, _stream())
    return codes, scales.view(_FP8), g


def _fake_nvfp4_rows(x, k):
    rows = x.shape[0]
    return (x.new_empty((rows, k // 2), dtype=torch.uint8), x.new_empty((swizzled_scale_numel(rows, k // 16),), dtype=_FP8),
            x.new_empty((rows,), dtype=torch.float32))


@_rms_norm_nvfp4_op.register_fake
def _(x, weight, epsilon):
    return _fake_nvfp4_rows(x, x.shape[1])


@_silu_mul_nvfp4_op.register_fake
def _(x):
    return _fake_nvfp4_rows(x, x.shape[1] // 2)


_OUT_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


@torch.library.custom_op("helion_b200::nvfp4_scaled_matmul", mutates_args=())
def _scaled_matmul_op(
    a_bytes: Tensor, b_bytes: Tensor, scale_a: Tensor, scale_b: Tensor, alpha: float, out_dtype: torch.dtype
) -> Tensor:
    """``a_bytes [M, K/2]`` and ``b_bytes [N, K/2]`` (both K-major, contiguous) -> ``[M, N]``."""
    _require_cuda(a_bytes, b_bytes, scale_a, scale_b)
    m, k_bytes = a_bytes.shape
    n = b_bytes.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=a_bytes.device)
    if m and n:
        with torch.cuda.device(a_bytes.device):
            _lib.call(
                "hb200_nvfp4_scaled_matmul",
                a_bytes.data_ptr(), b_bytes.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(), out.data_ptr(),
                m, n, k_bytes * 2, n, float(alpha), _OUT_DTYPES[out_dtype], _stream(),
            )
    return out


@_scaled_matmul_op.register_fake
def _(a_bytes, b_bytes, scale_a, scale_b, alpha, out_dtype):
    return a_bytes.new_empty((a_bytes.shape[0], b_bytes.shape[0]), dtype=out_dtype)


# ---------------------------------------------------------------- public entry points
def nvfp4_gemv_bf16in(
    weight_packed: Tensor, x_bf16: Tensor, weight_scale: Tensor, alpha: float = 1.0, *, backend: str | None = None,
    path: str = "auto",
) -> Tensor:
    """``weight_packed @ x_bf16`` for NVFP4 weights and a BF16 vector; returns bf16 ``[N]``.

    Drop-in for ``nvfp4_gemv_bf16in`` (examples/nvfp4_gemv.py:432-476).  ``backend`` is
    accepted for signature compatibility and ignored.  ``path`` picks the kernel: ``"simt"`` (bf16 activations
    taken exactly, fp16 products; what ``"auto"`` uses for small weights and K % 32 != 0), ``"tc"`` (tcgen05 on
    the packed weights, the activation expanded into four NVFP4 residual terms, relative error 1.2e-4; what
    ``"auto"`` uses for 1..32 rows when K % 32 == 0 and the weight has at least 2M elements) or ``"mma"``.
    """
    _check_contiguous("weight_packed", weight_packed)
    _check_contiguous("x_bf16", x_bf16)
    weight_bytes = fp4_storage(weight_packed)
    _check_fp4_weight_storage("weight_packed", weight_bytes)
    _check_numel("x_bf16", x_bf16, weight_bytes.shape[1] * 2)
    _check_swizzled_scales("weight_scale", weight_scale, weight_bytes.shape[0], weight_bytes.shape[1] // 8)
    if x_bf16.dtype is not torch.bfloat16:
        raise TypeError(f"x_bf16 must be torch.bfloat16, got {x_bf16.dtype}")
    out = _gemv_bf16in_op(weight_bytes, _aligned(x_bf16), weight_scale.reshape(-1).view(torch.uint8), alpha, path)
    return out.reshape(weight_bytes.shape[0])


def nvfp4_gemv_bf16in_batched(
    weight_packed: Tensor, x_bf16: Tensor, weight_scale: Tensor, alpha: float = 1.0, *, use_mma: bool | None = None,
    path: str = "auto",
) -> Tensor:
    """Decode-batch extension of :func:`nvfp4_gemv_bf16in`: ``x_bf16`` is ``[M, K]`` with 1 <= M <= 32,
    the result is bf16 ``[M, N]``.  ``path`` as in :func:`nvfp4_gemv_bf16in`; ``use_mma=True`` is the same as
    ``path="mma"`` (warp-level MMA on decoded weights, also for M == 1)."""
    _check_contiguous("weight_packed", weight_packed)
    _check_contiguous("x_bf16", x_bf16)
    weight_bytes = fp4_storage(weight_packed)
    _check_fp4_weight_storage("weight_packed", weight_bytes)
    if x_bf16.dim() != 2 or x_bf16.shape[1] != weight_bytes.shape[1] * 2:
        raise ValueError(f"x_bf16 must have shape [M, {weight_bytes.shape[1] * 2}]; got {tuple(x_bf16.shape)}")
    if not 1 <= x_bf16.shape[0] <= 32:
        raise ValueError(f"batch must be in 1..32; got {x_bf16.shape[0]}")
    _check_swizzled_scales("weight_scale", weight_scale, weight_bytes.shape[0], weight_bytes.shape[1] // 8)
    if x_bf16.dtype is not torch.bfloat16:
        raise TypeError(f"x_bf16 must be torch.bfloat16, got {x_bf16.dtype}")
    if use_mma:
        path = "mma"
    return _gemv_bf16in_op(weight_bytes, _aligned(x_bf16), weight_scale.reshape(-1).view(torch.uint8), alpha, path)


def nvfp4_gemv_fp4in(
    weight_packed: Tensor, x_packed: Tensor, weight_scale: Tensor, x_scale: Tensor, alpha: float = 1.0,
    *, backend: str | None = None, path: str = "auto",
) -> Tensor:
    """``weight_packed @ x_packed`` for NVFP4 weights and an NVFP4 vector; returns bf16 ``[N]``.

    Drop-in for ``nvfp4_gemv_fp4in`` (examples/nvfp4_gemv.py:479-525).
    """
    _check_contiguous("weight_packed", weight_packed)
    _check_contiguous("x_packed", x_packed)
    weight_bytes = fp4_storage(weight_packed)
    x_bytes = fp4_storage(x_packed)
    _check_fp4_weight_storage("weight_packed", weight_bytes)
    _check_numel("x_packed", x_bytes, weight_bytes.shape[1])
    scale_cols = weight_bytes.shape[1] // 8
    _check_swizzled_scales("weight_scale", weight_scale, weight_bytes.shape[0], scale_cols)
    _check_swizzled_scales("x_scale", x_scale, 1, scale_cols)
    return _gemv_fp4in_op(
        weight_bytes, _aligned(x_bytes), weight_scale.reshape(-1).view(torch.uint8),
        x_scale.reshape(-1).view(torch.uint8), alpha, path,
    )


def nvfp4_scaled_matmul(
    A_packed: Tensor, B_packed_t: Tensor, scale_a: Tensor, scale_b: Tensor,  # noqa: N803
    out_dtype: torch.dtype = torch.bfloat16, *, alpha: float = 1.0,
) -> Tensor:
    """Block-scaled FP4 x FP4 GEMM on the tensor cores: ``[M, K/2] x [K/2, N] -> [M, N]``.

    Drop-in for ``nvfp4_scaled_matmul`` (examples/nvfp4_gemm.py:331-364): ``B_packed_t`` is the transposed
    packed right-hand side (storage K-major, stride ``(1, K/2)``; anything else is re-laid out as the
    reference does), scales are flat SWIZZLE_32_4_4 e4m3 tensors for logical ``[M, K/16]`` / ``[N, K/16]``.
    ``alpha`` (keyword, default 1) is an extension that applies the operands' global scales in the epilogue.
    """
    if out_dtype not in _OUT_DTYPES:
        raise TypeError(f"unsupported output dtype for nvfp4_scaled_matmul: {out_dtype}")
    a = fp4_storage(A_packed)
    b_t = fp4_storage(B_packed_t)
    if a.dim() != 2 or b_t.dim() != 2:
        raise ValueError("nvfp4_scaled_matmul expects 2D FP4 matrices")
    m, k_bytes = a.shape
    k_bytes_b, n = b_t.shape
    if k_bytes_b != k_bytes:
        raise ValueError(
            f"B_packed_t shape {tuple(b_t.shape)} is incompatible with A_packed shape {tuple(a.shape)}"
        )
    if k_bytes % 8 != 0:
        raise ValueError(f"K must be divisible by 16, got {k_bytes * 2}")
    if a.stride() != (k_bytes, 1):
        a = a.contiguous()
    b = b_t.t()  # [N, K/2]
    if b.stride() != (k_bytes, 1):
        b = b.contiguous()
    k_groups = k_bytes // 8
    _check_swizzled_scales("scale_a", scale_a, m, k_groups)
    _check_swizzled_scales("scale_b", scale_b, n, k_groups)
    if scale_a.dtype is not _FP8:
        raise TypeError(f"scale_a must be torch.float8_e4m3fn, got {scale_a.dtype}")
    if scale_b.dtype is not _FP8:
        raise TypeError(f"scale_b must be torch.float8_e4m3fn, got {scale_b.dtype}")
    return _scaled_matmul_op(
        _aligned(a), _aligned(b), _aligned(scale_a.reshape(-1).view(torch.uint8)),
        _aligned(scale_b.reshape(-1).view(torch.uint8)), alpha, out_dtype,
    )


class HostPipelinedMatmul:
    """``host_out = (quantise(host_a) @ W^T) * alpha`` for activations that live in pinned host memory: the rows are
    cut into chunks, and the host-to-device copy of chunk i + 1, the quantiser and NVFP4 GEMM of chunk i and the
    device-to-host copy of chunk i - 1 run at the same time on three streams (PCIe is full duplex, so the two copies
    overlap each other as well as the kernels).  Every output row is what ``nvfp4_quantize`` + ``nvfp4_scaled_matmul``
    give for the whole matrix, bit for bit: rows are independent and the tensor-wide activation scale is given.

    ``weight_packed [N, K/2]`` / ``weight_scale`` are device tensors as for ``nvfp4_scaled_matmul``; ``a_global_scale``
    a one-element fp32 device tensor (the activation tensor's ``amax / (6 * 448)``); ``alpha`` the product of both
    global scales.  Buffers and streams are made once for a shape.  No counterpart in the reference (its operators
    take device tensors)."""

    def __init__(self, weight_packed: Tensor, weight_scale: Tensor, a_global_scale: Tensor, alpha: float, rows: int,
                 chunks: int = 4):
        _require_cuda(weight_packed, weight_scale, a_global_scale)
        if rows % chunks or (rows // chunks) % 256:
            raise ValueError("rows must split into chunks that are multiples of 256 rows")
        dev = weight_packed.device
        self.w, self.ws, self.ga, self.alpha = weight_packed, weight_scale, a_global_scale, float(alpha)
        self.rows, self.chunks, self.chunk = rows, chunks, rows // chunks
        self.k = weight_packed.shape[1] * 2
        self.a_buf = [torch.empty(self.chunk, self.k, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.copy_in = torch.cuda.Stream(device=dev)
        self.copy_out = torch.cuda.Stream(device=dev)
        self.a_free = [torch.cuda.Event() for _ in range(2)]

    def __call__(self, host_a: Tensor, host_out: Tensor) -> None:
        """Enqueues the whole pipeline; on return the current stream waits for the last copy to the host."""
        if host_a.shape != (self.rows, self.k) or host_a.dtype is not torch.bfloat16 or not host_a.is_pinned():
            raise ValueError("host_a must be a pinned bfloat16 [rows, K] tensor")
        if host_out.shape[0] != self.rows or not host_out.is_pinned():
            raise ValueError("host_out must be a pinned [rows, N] tensor")
        main = torch.cuda.current_stream(self.w.device)
        self.copy_in.wait_stream(main)
        self.copy_out.wait_stream(main)
        for i in range(self.chunks):
            buf, lo = self.a_buf[i % 2], i * self.chunk
            with torch.cuda.stream(self.copy_in):
                if i >= 2:
                    self.copy_in.wait_event(self.a_free[i % 2])  # the quantiser of chunk i - 2 has read this buffer
                buf.copy_(host_a[lo : lo + self.chunk], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self.copy_in)
            main.wait_event(arrived)
            codes, scales, _ = nvfp4_quantize(buf, self.ga)
            self.a_free[i % 2].record(main)
            y = nvfp4_scaled_matmul(codes, self.w.t(), scales, self.ws, host_out.dtype, alpha=self.alpha)
            done = torch.cuda.Event()
            done.record(main)
            y.record_stream(self.copy_out)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done)
                host_out[lo : lo + self.chunk].copy_(y, non_blocking=True)
        main.wait_stream(self.copy_out)


def nvfp4_w4a4_matmul(
    A_packed: Tensor, B_packed: Tensor, act_scale: Tensor, weight_scale: Tensor, alpha: float = 1.0  # noqa: N803
) -> Tensor:
    """``A_packed @ B_packed`` for NVFP4 activations ``[M, K/2]`` and NVFP4 weights stored N-major ``[K/2, N]``
    (row ``k`` in the low nibble, row ``k+1`` in the high nibble); bf16 ``[M, N]``.

    Drop-in for ``nvfp4_w4a4_matmul`` (examples/nvfp4_gemm.py:259-304).  A byte of the N-major weight holds the
    same two codes as the byte at the transposed position of the K-major weight, so the weight is transposed
    byte-wise on the device and fed to the tensor-core GEMM.
    """
    a = fp4_storage(A_packed)
    b = fp4_storage(B_packed)
    m, k_bytes_a = a.shape
    k_bytes_b, n = b.shape
    if k_bytes_a != k_bytes_b:
        raise ValueError(
            f"A_packed shape {tuple(a.shape)} is incompatible with B_packed shape {tuple(b.shape)}"
        )
    k = k_bytes_a * 2
    if k % 16 != 0:
        raise ValueError(f"K must be divisible by 16, got {k}")
    _check_swizzled_scales("act_scale", act_scale, m, k // 16)
    _check_swizzled_scales("weight_scale", weight_scale, n, k // 16)
    return _scaled_matmul_op(
        _aligned(a.contiguous()), _aligned(b.t().contiguous()), _aligned(act_scale.reshape(-1).view(torch.uint8)),
        _aligned(weight_scale.reshape(-1).view(torch.uint8)), alpha, torch.bfloat16,
    )


def nvfp4_w4a16_matmul(A: Tensor, B_packed: Tensor, weight_scale: Tensor, alpha: float = 1.0) -> Tensor:  # noqa: N803
    """``A @ B_packed`` for bf16 activations ``[M, K]`` and NVFP4 weights stored N-major ``[K/2, N]``; bf16 ``[M, N]``.

    Drop-in for ``nvfp4_w4a16_matmul`` (examples/nvfp4_gemm.py:171-210).  The weight is transposed byte-wise to
    K-major and the activations go through the decode-batch kernel 32 rows at a time (the weights are streamed
    once per 32 rows; like the reference's kernel this entry point is not the performance path for large M).
    """
    m, k = A.shape
    b = fp4_storage(B_packed)
    k_bytes, n = b.shape
    if k % 16 != 0:
        raise ValueError(f"K must be divisible by 16, got {k}")
    if k_bytes * 2 != k:
        raise ValueError(f"B_packed shape {tuple(b.shape)} is incompatible with A shape {tuple(A.shape)}")
    _check_swizzled_scales("weight_scale", weight_scale, n, k // 16)
    if A.dtype is not torch.bfloat16:
        raise TypeError(f"A must be torch.bfloat16, got {A.dtype}")
    w = b.t().contiguous()
    sc = weight_scale.reshape(-1).view(torch.uint8)
    a = A.contiguous()
    out = torch.empty(m, n, dtype=torch.bfloat16, device=A.device)
    for r0 in range(0, m, 32):
        r1 = min(m, r0 + 32)
        out[r0:r1] = _gemv_bf16in_op(w, _aligned(a[r0:r1]), sc, alpha, "auto")
    return out


def _aligned(t: Tensor) -> Tensor:
    """The kernels read activations with 16-byte loads; re-materialise odd views."""
    return t if t.data_ptr() % 16 == 0 else t.clone()


def silu_and_mul_per_block_quant(
    out: Tensor, input: Tensor, scales: Tensor, group_size: int,  # noqa: A002
    scale_ub: Tensor | None = None, is_scale_transposed: bool = False,
) -> None:
    """``out, scales <- quant_fp8_per_block(silu(input[:, :d]) * input[:, d:])`` in place.

    Drop-in for ``silu_and_mul_per_block_quant``
    (pretuned_kernels/silu_and_mul_per_block_quant/silu_and_mul_per_block_quant.py:31-122);
    the assertions are the reference's.
    """
    assert input.ndim == 2
    num_tokens, two_intermediate_size = input.shape
    assert two_intermediate_size % 2 == 0
    intermediate_size = two_intermediate_size // 2
    assert out.shape[0] == num_tokens
    assert out.shape[1] == intermediate_size
    assert out.dtype in [_FP8, torch.int8]
    if scale_ub is not None:
        assert out.dtype == _FP8
        assert scale_ub.dtype == torch.float32
    assert scales.ndim == 2 and scales.dtype == torch.float32
    assert scales.shape[0] == num_tokens
    groups_per_row = scales.shape[1]
    assert intermediate_size % group_size == 0 and intermediate_size // group_size == groups_per_row
    assert group_size in [64, 128]
    assert input.stride()[-1] == 1
    assert out.stride()[-1] == 1
    if input.dtype not in (torch.bfloat16, torch.float16, torch.float32):  # the reference converts any to fp32
        raise TypeError(f"input must be bfloat16, float16 or float32, got {input.dtype}")
    if scales.is_contiguous():
        _silu_mul_quant_op(out, input, scales, group_size, scale_ub)
    else:
        # a strided or transposed scale view (the reference writes scales by index, so any view works there):
        # the kernel writes a contiguous buffer, which is then copied into the view
        tmp = torch.empty(scales.shape, dtype=scales.dtype, device=scales.device)
        _silu_mul_quant_op(out, input, tmp, group_size, scale_ub)
        scales.copy_(tmp)


def rms_norm_dynamic_per_token_quant(
    result: Tensor, input: Tensor, weight: Tensor, scale: Tensor, epsilon: float,  # noqa: A002
    scale_ub: Tensor | None = None, residual: Tensor | None = None,
) -> None:
    """RMSNorm(weight) (+ optional residual add, written back) then per-token dynamic quantisation, in place.

    Drop-in for ``rms_norm_dynamic_per_token_quant``
    (pretuned_kernels/rms_norm_dynamic_per_token_quant/rms_norm_dynamic_per_token_quant.py:40-128).
    """
    assert input.ndim == 2
    num_tokens, hidden_size = input.shape
    assert result.dtype in [_FP8, torch.int8]
    assert result.is_contiguous() and input.is_contiguous()
    if scale_ub is not None:
        assert result.dtype == _FP8
        assert scale_ub.dtype == torch.float32
    assert input.dtype == weight.dtype
    assert scale.shape[0] == num_tokens
    assert scale.dtype == torch.float32
    if residual is not None:
        assert residual.dtype == input.dtype
        if not residual.is_contiguous():
            raise ValueError("residual must be contiguous")
    if input.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"input must be bfloat16 or float16, got {input.dtype}")
    if not (scale.is_contiguous() and weight.is_contiguous()):
        raise ValueError("scale and weight must be contiguous")
    _rms_quant_op(result, input, weight, scale, epsilon, scale_ub, residual)


def rms_norm_per_block_quant(
    result: Tensor, input: Tensor, weight: Tensor, scale: Tensor, epsilon: float,  # noqa: A002
    scale_ub: Tensor | None, residual: Tensor | None, group_size: int, is_scale_transposed: bool,
) -> None:
    """RMSNorm(weight) (+ optional residual add, written back) then one dynamic scale per ``group_size`` block.

    Drop-in for ``rms_norm_per_block_quant``
    (pretuned_kernels/rms_norm_per_block_quant/rms_norm_per_block_quant.py:38-140); ``scale`` may be a
    transposed view (``is_scale_transposed``), as there.
    """
    assert input.ndim == 2
    num_tokens, hidden_size = input.shape
    groups_per_row = scale.shape[1]
    assert hidden_size % group_size == 0 and hidden_size // group_size == groups_per_row
    assert scale.shape[0] == num_tokens
    assert scale.dtype == torch.float32
    if scale.stride(1) > 1:
        assert is_scale_transposed
    assert result.dtype in [_FP8, torch.int8]
    assert result.is_contiguous() and input.is_contiguous()
    if scale_ub is not None:
        assert result.dtype == _FP8
        assert scale_ub.dtype == torch.float32
    assert input.dtype == weight.dtype
    if residual is not None:
        assert residual.dtype == input.dtype
        if not residual.is_contiguous():
            raise ValueError("residual must be contiguous")
    assert group_size in [64, 128]
    if input.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"input must be bfloat16 or float16, got {input.dtype}")
    if not weight.is_contiguous():
        raise ValueError("weight must be contiguous")
    _rms_block_quant_op(result, input, weight, scale, epsilon, scale_ub, residual, group_size)


def dynamic_per_token_scaled_fp8_quant(
    result: Tensor, input: Tensor, scale: Tensor, scale_ub: Tensor | None = None,  # noqa: A002
) -> None:
    """Per-token dynamic FP8 quantisation ``result = fp8(input * (1 / scale))``, ``scale = amax / 448``, in place.

    Drop-in for ``dynamic_per_token_scaled_fp8_quant``
    (pretuned_kernels/dynamic_per_token_scaled_fp8_quant/dynamic_per_token_scaled_fp8_quant.py:32-72).
    """
    assert input.ndim == 2
    num_tokens, _hidden = input.shape
    assert result.shape == input.shape
    assert scale.shape[0] == num_tokens
    assert scale.dtype == torch.float32
    assert input.stride()[-1] == 1
    assert result.stride()[-1] == 1
    if input.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"input must be bfloat16 or float16, got {input.dtype}")
    if result.dtype is not _FP8:
        raise TypeError(f"result must be float8_e4m3fn, got {result.dtype}")
    if not (result.is_contiguous() and scale.is_contiguous()):
        raise ValueError("result and scale must be contiguous")
    _dyn_token_quant_op(result, input.contiguous(), scale, scale_ub)


def silu_mul_fp8(input: Tensor, scale: Tensor) -> Tensor:  # noqa: A002
    """``fp8_e4m3((silu(x[..., :d]) * x[..., d:]) / scale)`` for an input whose last dimension is ``2 * d``.

    Drop-in for ``silu_mul_fp8`` (pretuned_kernels/silu_mul_fp8/silu_mul_fp8.py:29-59): SiLU and the product are
    rounded to the input type as the reference's tile arithmetic does, the fp32 result is multiplied by the
    reciprocal of the one-element ``scale``; returns a new tensor of shape ``(*input.shape[:-1], d)``.
    """
    original_shape = input.shape
    two_d = original_shape[-1]
    d = two_d // 2
    assert scale.numel() == 1, "Scale must be a scalar Tensor"
    if two_d % 2:
        raise ValueError(f"the last dimension must be even, got {two_d}")
    if input.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"input must be bfloat16 or float16, got {input.dtype}")
    if d % 8:
        raise ValueError(f"d must be a multiple of 8 (16-byte loads of both halves), got {d}")
    input_2d = input.reshape(-1, two_d)
    if input_2d.stride(1) != 1 or input_2d.stride(0) % 8 or input_2d.data_ptr() % 16:
        input_2d = input_2d.contiguous()
    out = _silu_mul_fp8_op(input_2d, scale.reshape(1).to(torch.float32))
    return out.view(*original_shape[:-1], d)


def scaled_mm(
    c: Tensor, a: Tensor, b: Tensor, scale_a: Tensor, scale_b: Tensor, bias: Tensor | None = None,
) -> None:
    """FP8 or int8 scaled matrix multiply ``c = scale_a * (a @ b) * scale_b + bias``, in place on ``c``.

    Drop-in for ``scaled_mm`` (pretuned_kernels/scaled_mm/scaled_mm.py:18-84): ``a [M, K]`` with unit stride
    along K, ``b [K, N]`` with ``b.stride(0) == 1`` (the weight stored ``[N, K]``), scales ``[1]``, ``[1, 1]``,
    ``[M]`` / ``[M, 1]`` (``scale_a``) or ``[N]`` / ``[N, 1]`` (``scale_b``), optional ``bias [N]`` in ``c``'s dtype,
    added after the cast to that dtype.  The reference's assertions are kept.  int8 operands accumulate in int32
    (scaled_mm.py:53), converted to fp32 once after the whole K range.
    """
    M, K = a.shape  # noqa: N806
    N = b.shape[1]  # noqa: N806
    assert N > 0 and K > 0 and M > 0
    assert b.shape[0] == K
    assert a.dtype == b.dtype
    assert a.stride(1) == 1
    assert b.stride(0) == 1
    scale_a = scale_a.reshape(-1, 1) if scale_a.dim() <= 1 else scale_a
    scale_b = scale_b.reshape(-1, 1) if scale_b.dim() <= 1 else scale_b
    assert scale_a.dtype == scale_b.dtype and scale_a.is_floating_point()
    assert scale_a.shape[1] == 1 and (scale_a.shape[0] == 1 or scale_a.shape[0] == M)
    assert scale_b.shape[1] == 1 and (scale_b.shape[0] == 1 or scale_b.shape[0] == N)
    out_dtype = c.dtype
    assert out_dtype.is_floating_point
    if bias is not None:
        assert bias.numel() == N and bias.dtype == out_dtype
    if a.dtype not in (_FP8, torch.float8_e5m2, torch.int8):
        raise TypeError(f"a and b must be float8_e4m3fn, float8_e5m2 or int8, got {a.dtype}")
    if out_dtype not in _SCALED_MM_OUT:
        raise TypeError(f"c must be bfloat16, float16 or float32, got {out_dtype}")
    if c.shape != (M, N) or c.stride(1) != 1:
        raise ValueError("c must be [M, N] with unit stride along N")
    b_nk = b.t()  # [N, K], unit stride along K
    if a.stride(0) % 16 or a.data_ptr() % 16:
        a = a.contiguous()
    if b_nk.stride(0) % 16 or b_nk.data_ptr() % 16:
        b_nk = b_nk.contiguous()
    if K % 16:
        raise ValueError(f"K must be a multiple of 16 (row pitch of the TMA loads), got {K}")
    scale_a = scale_a.reshape(-1).to(torch.float32).contiguous()
    scale_b = scale_b.reshape(-1).to(torch.float32).contiguous()
    _scaled_mm_op(c, a, b_nk, scale_a, scale_b, None if bias is None else bias.reshape(-1).contiguous())


def per_token_group_fp8_quant(
    input: Tensor, output_q: Tensor, output_s: Tensor, group_size: int, eps: float,  # noqa: A002
    fp8_min: float, fp8_max: float, scale_ue8m0: bool,
    dummy_is_scale_transposed: bool = False, dummy_is_tma_aligned: bool = False,
) -> None:
    """Per-(token, group) dynamic FP8 quantisation, in place on ``output_q`` / ``output_s``.

    Drop-in for ``per_token_group_fp8_quant``
    (pretuned_kernels/per_token_group_fp8_quant/per_token_group_fp8_quant.py:29-74); the arithmetic is
    the module's fp32 reference ``_per_token_group_fp8_quant_torch`` (:77-97).
    """
    assert input.ndim == 2
    num_tokens, hidden_size = input.shape
    groups_per_row = output_s.shape[1]
    assert hidden_size % group_size == 0 and hidden_size // group_size == groups_per_row
    assert output_s.ndim == 2 and output_s.dtype == torch.float32
    if not (input.is_contiguous() and output_q.is_contiguous() and output_s.is_contiguous()):
        raise ValueError("input, output_q and output_s must be contiguous")
    if output_q.dtype is not _FP8:
        raise TypeError(f"output_q must be torch.float8_e4m3fn, got {output_q.dtype}")
    _group_quant_op(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0)


def nvfp4_quantize(x: Tensor, global_scale: Tensor | None = None) -> tuple[Tensor, Tensor, Tensor]:
    """bf16 ``[rows, K]`` -> ``(packed e2m1 [rows, K/2] uint8, swizzled e4m3 scales, global scale)``.

    With ``global_scale`` (0-dim or 1-element fp32 tensor) the whole tensor shares it; with ``None``
    each row gets its own ``row_amax / (6 * 448)`` (returned as ``[rows]``).  The code rule is the
    reference's ``quantize_fp4_e2m1`` (examples/nvfp4_gemm.py:368-381).
    """
    if x.dim() != 2:
        raise ValueError("nvfp4_quantize expects a 2D tensor")
    if x.shape[1] % 16:
        raise ValueError(f"K must be divisible by 16, got {x.shape[1]}")
    if x.dtype is not torch.bfloat16:
        raise TypeError(f"x must be torch.bfloat16, got {x.dtype}")
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    return _nvfp4_quantize_op(x, global_scale)


def _row_major_bf16(name: str, x: Tensor) -> Tensor:
    if x.dim() != 2:
        raise ValueError(f"{name} must be a 2D tensor")
    if x.dtype is not torch.bfloat16:
        raise TypeError(f"{name} must be torch.bfloat16, got {x.dtype}")
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    return x


def rms_norm_nvfp4_quant(input: Tensor, weight: Tensor, epsilon: float) -> tuple[Tensor, Tensor, Tensor]:  # noqa: A002
    """RMSNorm(weight) fused with per-token NVFP4 quantisation: bf16 ``[T, H]`` ->
    ``(packed e2m1 [T, H/2] uint8, swizzled e4m3 scales for [T, H/16], per-token global scale [T])``.

    The NVFP4 form of ``rms_norm_dynamic_per_token_quant``: the normalisation is that operator's
    (pretuned_kernels/rms_norm_dynamic_per_token_quant/rms_norm_dynamic_per_token_quant.py:131-150), the quantiser
    :func:`nvfp4_quantize`'s per-token mode; the normalised row never reaches memory.  The outputs are the activation
    operand of :func:`nvfp4_gemv_fp4in` / :func:`nvfp4_scaled_matmul` (fold the per-token scale into ``alpha`` or the
    consumer's row scale).
    """
    x = _row_major_bf16("input", input)
    if x.shape[1] % 16:
        raise ValueError(f"hidden size must be divisible by 16, got {x.shape[1]}")
    if weight.dtype is not torch.bfloat16 or weight.numel() != x.shape[1]:
        raise ValueError(f"weight must be bfloat16 with {x.shape[1]} values")
    return _rms_norm_nvfp4_op(x, _aligned(weight.reshape(-1).contiguous()), float(epsilon))


def silu_and_mul_nvfp4_quant(input: Tensor) -> tuple[Tensor, Tensor, Tensor]:  # noqa: A002
    """``y = bf16(silu(input[:, :d]) * input[:, d:])`` fused with per-token NVFP4 quantisation of ``y``:
    bf16 ``[T, 2d]`` -> ``(packed e2m1 [T, d/2], swizzled e4m3 scales for [T, d/16], per-token global scale [T])``.

    The NVFP4 form of ``silu_and_mul_per_block_quant`` (gate first:
    pretuned_kernels/silu_and_mul_per_block_quant/silu_and_mul_per_block_quant.py:97-105); ``y`` never reaches memory.
    """
    x = _row_major_bf16("input", input)
    if x.shape[1] % 32:
        raise ValueError(f"the last dimension must be 2 * d with d divisible by 16, got {x.shape[1]}")
    return _silu_mul_nvfp4_op(x)
