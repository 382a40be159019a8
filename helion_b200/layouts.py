"""Host-side data-format helpers: SWIZZLE_32_4_4 scale layout, e2m1 packing, NVFP4 quantisation.

These mirror the helper functions the reference ships next to its kernels
(``examples/nvfp4_gemv.py:60-155``, ``examples/nvfp4_gemm.py:41-61,368-424``) so that
tensors prepared for the reference can be fed to these operators unchanged.  They
are plain tensor code that runs on whatever device the input lives on; nothing
here is on the timed path.
"""

from __future__ import annotations

import torch
from torch import Tensor

FP4_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# midpoints between neighbouring magnitudes; a value exactly on one rounds down
FP4_E2M1_BOUNDARIES = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
FP4_MAX = 6.0
E4M3_MAX = 448.0


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def round_up(a: int, b: int) -> int:
    return ceil_div(a, b) * b


# ------------------------------------------------------------------ scale layout
def swizzled_scale_numel(rows: int, cols: int) -> int:
    """Bytes of the padded SWIZZLE_32_4_4 buffer for logical ``[rows, cols]`` scales."""
    return round_up(rows, 128) * round_up(cols, 4)


def swizzled_scale_offsets(row, col, cols: int):
    """Flat offset of logical scale ``(row, col)``; works on ints and tensors.

    The buffer is a sequence of 512-byte tiles (128 rows x 4 columns), ordered by
    row tile then column tile; inside a tile the byte is
    ``(row % 32) * 16 + (row % 128 // 32) * 4 + col % 4``.
    """
    tiles_per_row = ceil_div(cols, 4)
    tile = (row // 128) * tiles_per_row + col // 4
    return tile * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + col % 4


def _offset_grid(rows: int, cols: int, device) -> Tensor:
    r = torch.arange(rows, device=device, dtype=torch.int64)[:, None]
    c = torch.arange(cols, device=device, dtype=torch.int64)[None, :]
    return swizzled_scale_offsets(r, c, cols)


def swizzle_fp8_scales(scales: Tensor) -> Tensor:
    """Logical row-major ``[rows, cols]`` (or 1-D = one row) scales -> flat swizzled buffer, zero padded."""
    if scales.dim() == 1:
        scales = scales.reshape(1, -1)
    elif scales.dim() != 2:
        raise ValueError(f"expected 1D or 2D scales, got {scales.dim()}D")
    rows, cols = scales.shape
    flat = torch.zeros(swizzled_scale_numel(rows, cols), device=scales.device, dtype=scales.dtype)
    # index through a byte view: float8 tensors do not support index_put on every device
    if scales.element_size() == 1:
        flat.view(torch.uint8)[_offset_grid(rows, cols, scales.device).reshape(-1)] = scales.reshape(-1).view(torch.uint8)
    else:
        flat[_offset_grid(rows, cols, scales.device).reshape(-1)] = scales.reshape(-1)
    return flat


def unswizzle_fp8_scales(scales: Tensor, rows: int, cols: int) -> Tensor:
    """Inverse of :func:`swizzle_fp8_scales`: flat buffer -> logical ``[rows, cols]``."""
    flat = scales.reshape(-1)
    idx = _offset_grid(rows, cols, scales.device)
    if flat.element_size() == 1:
        return flat.view(torch.uint8)[idx].view(flat.dtype)
    return flat[idx]


# ---------------------------------------------------------------- e2m1 packing
def as_fp4x2(t: Tensor) -> Tensor:
    if t.dtype is torch.float4_e2m1fn_x2:
        return t
    if t.dtype is torch.uint8:
        return t.view(torch.float4_e2m1fn_x2)
    raise TypeError(f"expected uint8 or float4_e2m1fn_x2 tensor, got {t.dtype}")


def fp4_storage(t: Tensor) -> Tensor:
    """uint8 view of a packed FP4 tensor (shell dtype or raw bytes)."""
    if t.dtype is torch.float4_e2m1fn_x2:
        return t.view(torch.uint8)
    if t.dtype is torch.uint8:
        return t
    raise TypeError(f"expected uint8 or float4_e2m1fn_x2 tensor, got {t.dtype}")


def quantize_fp4_e2m1(x: Tensor) -> Tensor:
    """Float values -> 4-bit codes (bit 3 = sign, bits 0-2 = magnitude index), uint8.

    Magnitudes clamp at 6; a value exactly halfway between two magnitudes takes the
    smaller one; the sign bit is ``x < 0`` (so -0.0 encodes as 0).
    """
    mag = x.abs().clamp(max=FP4_MAX)
    idx = torch.zeros(x.shape, dtype=torch.uint8, device=x.device)
    for b in FP4_E2M1_BOUNDARIES:
        idx += (mag > b).to(torch.uint8)
    return idx | ((x < 0).to(torch.uint8) << 3)


def dequantize_fp4_codes(codes: Tensor) -> Tensor:
    """4-bit codes -> fp32 values."""
    lut = torch.tensor(FP4_E2M1_VALUES + tuple(-v for v in FP4_E2M1_VALUES), dtype=torch.float32, device=codes.device)
    return lut[codes.to(torch.int64)]


def pack_fp4_last_dim(codes: Tensor) -> Tensor:
    """``[..., K]`` codes -> ``[..., K/2]`` bytes, element 2j in the low nibble (K-major operands)."""
    if codes.shape[-1] % 2:
        raise ValueError("K dimension must be even for FP4 packing")
    pairs = codes.reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return ((pairs[..., 0] & 0xF) | (pairs[..., 1] << 4)).to(torch.uint8)


def pack_fp4(codes: Tensor) -> Tensor:
    """``[K, N]`` codes -> ``[K/2, N]`` bytes, row 2j in the low nibble (N-major weights)."""
    if codes.shape[0] % 2:
        raise ValueError("K dimension must be even for FP4 packing")
    return ((codes[0::2] & 0xF) | (codes[1::2] << 4)).to(torch.uint8)


def unpack_fp4_last_dim(packed: Tensor) -> Tensor:
    """``[..., K/2]`` bytes -> ``[..., K]`` codes."""
    b = fp4_storage(packed)
    return torch.stack((b & 0xF, b >> 4), dim=-1).reshape(*b.shape[:-1], b.shape[-1] * 2)


def unpack_fp4(packed: Tensor) -> Tensor:
    """``[K/2, N]`` bytes -> ``[K, N]`` codes."""
    b = fp4_storage(packed)
    return torch.stack((b & 0xF, b >> 4), dim=1).reshape(b.shape[0] * 2, b.shape[1])


# ------------------------------------------------------------ NVFP4 quantiser
def nvfp4_global_scale(x: Tensor) -> Tensor:
    """Per-tensor fp32 global scale ``amax / (6 * 448)`` (0-dim tensor).

    The divisor is a tensor on purpose: dividing a CUDA tensor by a Python scalar multiplies by the
    rounded reciprocal, which can differ from the true quotient in the last place."""
    amax = x.abs().amax().to(torch.float32)
    return amax / torch.tensor(FP4_MAX * E4M3_MAX, dtype=torch.float32, device=amax.device)


def nvfp4_quantize_host(x: Tensor, global_scale: Tensor | None = None, per_token: bool = False):
    """Tensor-code NVFP4 quantiser used to prepare weights (not a timed path).

    ``x`` is ``[rows, K]``; returns ``(packed [rows, K/2] uint8, swizzled e4m3 scales,
    global_scale)`` with 16-element blocks along K:  ``s = e4m3((block_amax / 6) / g)``,
    ``codes = quantize_fp4_e2m1(x / (float(s) * g))``; blocks whose decoded scale is
    zero get code 0.  ``g`` is per tensor (0-dim) or, with ``per_token``, per row.
    """
    rows, k = x.shape
    if k % 16:
        raise ValueError(f"K must be divisible by 16, got {k}")
    xf = x.to(torch.float32)
    if global_scale is None:
        if per_token:
            global_scale = xf.abs().amax(dim=-1) / torch.tensor(FP4_MAX * E4M3_MAX, dtype=torch.float32, device=xf.device)
        else:
            global_scale = nvfp4_global_scale(xf)
    g = global_scale.to(torch.float32).reshape(-1, 1, 1) if per_token else global_scale.to(torch.float32)
    blocks = xf.reshape(rows, k // 16, 16)
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    # (tensor divisors: dividing a CUDA tensor by a Python scalar multiplies by the rounded reciprocal)
    sf = (amax / torch.tensor(FP4_MAX, dtype=torch.float32, device=xf.device)) / g
    sf = torch.where(g > 0, sf, torch.zeros_like(sf))
    s8 = sf.to(torch.float8_e4m3fn)
    denom = s8.to(torch.float32) * g
    v = torch.where(denom > 0, blocks / denom, torch.zeros_like(blocks))
    codes = quantize_fp4_e2m1(v).reshape(rows, k)
    return pack_fp4_last_dim(codes), swizzle_fp8_scales(s8.reshape(rows, k // 16)), global_scale


def nvfp4_dequantize_host(packed: Tensor, scales: Tensor, global_scale=1.0) -> Tensor:
    """``[rows, K/2]`` bytes + swizzled scales (+ global scale) -> fp32 ``[rows, K]``."""
    b = fp4_storage(packed)
    rows, kb = b.shape
    vals = dequantize_fp4_codes(unpack_fp4_last_dim(b)).reshape(rows, kb // 8, 16)
    s = unswizzle_fp8_scales(scales, rows, kb // 8).to(torch.float32)
    out = (vals * s[:, :, None]).reshape(rows, kb * 2)
    if isinstance(global_scale, Tensor) and global_scale.dim() >= 1:
        return out * global_scale.reshape(-1, 1).to(torch.float32)
    return out * global_scale
