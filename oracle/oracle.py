"""CPU oracle for the quantized-inference operators -- TEST INFRASTRUCTURE ONLY.

This module restates, in plain tensor code on the CPU, what the reference's own
PyTorch reference functions compute for each operator on the hot path.  It is the
checker for the CUDA kernels: only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it.  Nothing
under ``helion_b200/`` imports it and no product path falls back to it.

Parity pin: every function below is checked in ``tests/test_oracle_golden.py``
against fixtures in ``tests/golden/*.npz`` that were produced by running the
reference's functions (imported from the reference checkout) on seeded inputs and,
for the FP8 operators, by running the reference's KERNELS themselves in the
reference's CPU interpreter; ``tests/golden/make_golden.py`` is the generating script.  Pieces the reference
does not contain (the NVFP4 quantiser with a global scale, the NVFP4 MoE
pipeline) are compositions of pinned pieces and say so in their docstring.

Float arithmetic is done with torch CPU ops because the reference's functions are
torch code: dtype casts (bf16, float8_e4m3fn) and their rounding are then the
reference's by construction.  Integer/byte work (nibble decode, swizzle offsets)
is restated from the formulas.
"""

from __future__ import annotations

import torch
from torch import Tensor

E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E2M1_BOUNDARIES = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
FP8_MAX = 448.0
FP8_MIN_SCALE = 1.0 / (448.0 * 512.0)


# ------------------------------------------------------------------- formats
def swizzled_offsets(rows: int, cols: int) -> Tensor:
    """int64 ``[rows, cols]`` flat offsets of SWIZZLE_32_4_4 (examples/nvfp4_gemv.py:68-79)."""
    r = torch.arange(rows, dtype=torch.int64)[:, None]
    c = torch.arange(cols, dtype=torch.int64)[None, :]
    col_tiles = (cols + 3) // 4
    return ((r // 128) * col_tiles + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4


def swizzled_numel(rows: int, cols: int) -> int:
    """examples/nvfp4_gemv.py:64-65."""
    return ((rows + 127) // 128 * 128) * ((cols + 3) // 4 * 4)


def swizzle_scales(logical: Tensor) -> Tensor:
    """Logical ``[rows, cols]`` e4m3 scales -> flat zero-padded buffer (examples/nvfp4_gemv.py:82-101)."""
    rows, cols = logical.shape
    out = torch.zeros(swizzled_numel(rows, cols), dtype=torch.uint8)
    out[swizzled_offsets(rows, cols).reshape(-1)] = logical.contiguous().view(torch.uint8).reshape(-1)
    return out.view(logical.dtype)


def unswizzle_scales(flat: Tensor, rows: int, cols: int) -> Tensor:
    """examples/nvfp4_gemv.py:104-108."""
    return flat.reshape(-1).view(torch.uint8)[swizzled_offsets(rows, cols)].view(flat.dtype)


def dequant_e2m1(nibbles: Tensor) -> Tensor:
    """4-bit codes -> fp32: sign * {0,.5,1,1.5,2,3,4,6} (examples/nvfp4_gemv.py:528-536,
    test/test_quantized_ops.py:18-26)."""
    lut = torch.tensor(E2M1_MAGNITUDES + tuple(-m for m in E2M1_MAGNITUDES), dtype=torch.float32)
    return lut[(nibbles.to(torch.int64) & 0xF)]


def _bytes(t: Tensor) -> Tensor:
    return t.view(torch.uint8) if t.dtype is not torch.uint8 else t


def unpack_k_major(packed: Tensor) -> Tensor:
    """``[R, K/2]`` bytes -> fp32 ``[R, K]``; low nibble is the even k (examples/nvfp4_gemv.py:548-556,
    examples/nvfp4_gemm.py:411-424 with last_dim=True)."""
    b = _bytes(packed).to(torch.int32)
    lo, hi = dequant_e2m1(b & 0xF), dequant_e2m1((b >> 4) & 0xF)
    return torch.stack((lo, hi), dim=-1).reshape(b.shape[0], b.shape[1] * 2)


def unpack_n_major(packed: Tensor) -> Tensor:
    """``[K/2, N]`` bytes -> fp32 ``[K, N]``; low nibble is the even row (examples/nvfp4_gemm.py:384-393,411-424)."""
    b = _bytes(packed).to(torch.int32)
    lo, hi = dequant_e2m1(b & 0xF), dequant_e2m1((b >> 4) & 0xF)
    return torch.stack((lo, hi), dim=1).reshape(b.shape[0] * 2, b.shape[1])


def quantize_fp4_e2m1(x: Tensor) -> Tensor:
    """fp32 -> 4-bit codes: magnitude index = number of boundaries strictly below min(|x|, 6)
    (torch.bucketize, right=False), sign bit = x < 0 (examples/nvfp4_gemm.py:368-381)."""
    mag = x.abs().clamp(max=6.0)
    idx = torch.bucketize(mag, torch.tensor(E2M1_BOUNDARIES, dtype=mag.dtype)).to(torch.uint8)
    return idx | ((x < 0).to(torch.uint8) << 3)


def pack_k_major(codes: Tensor) -> Tensor:
    """examples/nvfp4_gemm.py:396-408."""
    r, k = codes.shape
    p = codes.reshape(r, k // 2, 2)
    return ((p[:, :, 0] & 0xF) | (p[:, :, 1] << 4)).to(torch.uint8)


def dequant_scaled_k_major(packed: Tensor, scales_swizzled: Tensor) -> Tensor:
    """fp32 ``[R, K]`` = e2m1 values times their block scale (no global scale)."""
    vals = unpack_k_major(packed)
    rows, k = vals.shape
    s = unswizzle_scales(scales_swizzled, rows, k // 16).to(torch.float32)
    return (vals.reshape(rows, k // 16, 16) * s[:, :, None]).reshape(rows, k)


# ---------------------------------------------------------------------- GEMV
def nvfp4_gemv_bf16in(weight_packed: Tensor, x_bf16: Tensor, weight_scale: Tensor, alpha: float = 1.0) -> Tensor:
    """examples/nvfp4_gemv.py:539-557: fp32 products, times the fp32 block scale, summed over K in fp32,
    times alpha, rounded to bf16.  Returns ``[N]``."""
    w = unpack_k_major(weight_packed)
    n, k = w.shape
    s = unswizzle_scales(weight_scale, n, k // 16).to(torch.float32).repeat_interleave(16, dim=1)
    prod = w * x_bf16.to(torch.float32).reshape(1, k)
    # the reference sums pairs (lo*x0 + hi*x1) first, then scales, then reduces
    pair = prod.reshape(n, k // 2, 2)
    pair = (pair[:, :, 0] + pair[:, :, 1]) * s[:, ::2]
    return (pair.sum(-1) * alpha).to(torch.bfloat16)


def nvfp4_gemv_fp4in(
    weight_packed: Tensor, x_packed: Tensor, weight_scale: Tensor, x_scale: Tensor, alpha: float = 1.0
) -> Tensor:
    """examples/nvfp4_gemv.py:560-590: as above with an e2m1 activation and scale = w_scale * x_scale."""
    w = unpack_k_major(weight_packed)
    n, k = w.shape
    x = unpack_k_major(_bytes(x_packed).reshape(1, -1))
    ws = unswizzle_scales(weight_scale, n, k // 16).to(torch.float32)
    xs = unswizzle_scales(x_scale, 1, k // 16).to(torch.float32)
    s = (ws * xs).repeat_interleave(8, dim=1)
    pair = (w * x).reshape(n, k // 2, 2)
    pair = (pair[:, :, 0] + pair[:, :, 1]) * s
    return (pair.sum(-1) * alpha).to(torch.bfloat16)


def nvfp4_gemm_bf16in(weight_packed: Tensor, x_bf16: Tensor, weight_scale: Tensor, alpha: float = 1.0) -> Tensor:
    """Decode batch ``[M, K] x [N, K]^T``: dequantise -> fp32 matmul -> * alpha -> bf16, the semantics of
    reference_nvfp4_w4a16_matmul (examples/nvfp4_gemm.py:428-443) with a K-major weight."""
    w = dequant_scaled_k_major(weight_packed, weight_scale)
    return (torch.matmul(x_bf16.to(torch.float32), w.t()) * alpha).to(torch.bfloat16)


# ---------------------------------------------------------------------- GEMM
def nvfp4_w4a16_matmul(a: Tensor, b_packed_n_major: Tensor, weight_scale: Tensor, alpha: float = 1.0) -> Tensor:
    """examples/nvfp4_gemm.py:428-443 (B is ``[K/2, N]``, scales logical ``[N, K/16]``)."""
    b = unpack_n_major(b_packed_n_major)
    k, n = b.shape
    s = unswizzle_scales(weight_scale, n, k // 16).to(torch.float32)  # [N, K/16]
    b = b * s.t().repeat_interleave(16, dim=0)
    return (torch.matmul(a.to(torch.float32), b) * alpha).to(torch.bfloat16)


def nvfp4_w4a4_matmul(
    a_packed: Tensor, b_packed_n_major: Tensor, act_scale: Tensor, weight_scale: Tensor, alpha: float = 1.0
) -> Tensor:
    """examples/nvfp4_gemm.py:446-475."""
    a = dequant_scaled_k_major(a_packed, act_scale)
    b = unpack_n_major(b_packed_n_major)
    k, n = b.shape
    s = unswizzle_scales(weight_scale, n, k // 16).to(torch.float32)
    b = b * s.t().repeat_interleave(16, dim=0)
    return (torch.matmul(a, b) * alpha).to(torch.bfloat16)


def nvfp4_scaled_matmul(
    a_packed: Tensor, b_packed_k_major: Tensor, scale_a: Tensor, scale_b: Tensor, out_dtype=torch.bfloat16,
    alpha: float = 1.0,
) -> Tensor:
    """Block-scaled ``A[M,K] @ B[N,K]^T`` as dequantise-then-fp32-matmul.  The reference's own entry point
    (examples/nvfp4_gemm.py:331-364) defers to torch._scaled_mm, which has no CPU path; its independent
    pin is reference_nvfp4_w4a4_matmul (:446-475), whose arithmetic this follows with a K-major B."""
    a = dequant_scaled_k_major(a_packed, scale_a)
    b = dequant_scaled_k_major(b_packed_k_major, scale_b)
    return (torch.matmul(a, b.t()) * alpha).to(out_dtype)


# ----------------------------------------------------------- NVFP4 quantiser
def nvfp4_quantize(x: Tensor, global_scale: Tensor | None = None, per_token: bool = False):
    """bf16/fp32 ``[R, K]`` -> (packed ``[R, K/2]``, swizzled e4m3 scales, fp32 global scale).

    Composition (the reference has no such function; its pieces are quantize_fp4_e2m1,
    pack_fp4_last_dim and swizzle_fp8_scales): ``g = amax / (6*448)`` per tensor or per row,
    ``s = e4m3((block_amax / 6) / g)`` per 16 elements, ``codes = quantize_fp4_e2m1(x / (float(s) * g))``,
    code 0 where the decoded scale (or g) is zero.
    """
    rows, k = x.shape
    xf = x.to(torch.float32)
    if global_scale is None:
        global_scale = (xf.abs().amax(dim=-1) if per_token else xf.abs().amax()) / (6.0 * 448.0)
    g = global_scale.to(torch.float32).reshape(-1, 1, 1) if per_token else global_scale.to(torch.float32).reshape(())
    blocks = xf.reshape(rows, k // 16, 16)
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    sf = (amax / 6.0) / g
    sf = torch.where(g > 0, sf, torch.zeros_like(sf))
    s8 = sf.to(torch.float8_e4m3fn)
    denom = s8.to(torch.float32) * g
    v = torch.where(denom > 0, blocks / denom, torch.zeros_like(blocks))
    codes = quantize_fp4_e2m1(v).reshape(rows, k)
    return pack_k_major(codes), swizzle_scales(s8.reshape(rows, k // 16)), global_scale.to(torch.float32)


# ------------------------------------------------------------ quant producers
def silu_and_mul_per_block_quant(x: Tensor, group_size: int, scale_ub: Tensor | None = None):
    """_silu_and_mul_per_block_quant_torch
    (pretuned_kernels/silu_and_mul_per_block_quant/silu_and_mul_per_block_quant.py:125-153).
    Returns ``(codes float8_e4m3fn [T, I], scales fp32 [T, I/group])``."""
    t, two_i = x.shape
    i = two_i // 2
    a = x[:, :i].to(torch.float32)
    b = x[:, i:].to(torch.float32)
    y = (a * torch.sigmoid(a) * b).reshape(t, i // group_size, group_size)
    s = y.abs().amax(dim=-1)
    if scale_ub is not None:
        s = s.clamp(max=float(scale_ub))
    s = (s * (1.0 / FP8_MAX)).clamp(min=FP8_MIN_SCALE)
    q = (y / s[:, :, None]).clamp(-FP8_MAX, FP8_MAX)
    return q.reshape(t, i).to(torch.float8_e4m3fn), s


def rms_norm_dynamic_per_token_quant(
    x: Tensor, weight: Tensor, epsilon: float, scale_ub: Tensor | None = None, residual: Tensor | None = None,
    rms_ulp_nudge: Tensor | None = None,
):
    """_rms_norm_dynamic_per_token_quant_torch
    (pretuned_kernels/rms_norm_dynamic_per_token_quant/rms_norm_dynamic_per_token_quant.py:131-163).
    Returns ``(codes [T, H], scale [T, 1], new_residual or None)``.

    ``rms_ulp_nudge`` (int32 ``[T]``, test hook) moves each row's fp32 ``rms`` by that many units in the
    last place before it is used, to decide whether a mismatch is explained by summation order."""
    xf = x.to(torch.float32)
    new_res = None
    if residual is not None:
        xf = xf + residual.to(torch.float32)
        new_res = xf.to(residual.dtype)
    rms = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + epsilon)
    if rms_ulp_nudge is not None:
        rms = (rms.view(torch.int32) + rms_ulp_nudge.reshape(-1, 1).to(torch.int32)).view(torch.float32)
    normed = (xf * rms).to(x.dtype) * weight[None, :]
    s = normed.to(torch.float32).abs().amax(dim=-1, keepdim=True)
    if scale_ub is not None:
        s = s.clamp(max=float(scale_ub))
    s = (s * (1.0 / FP8_MAX)).clamp(min=FP8_MIN_SCALE)
    q = (normed.to(torch.float32) / s).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, s, new_res


def dynamic_per_token_scaled_fp8_quant(x: Tensor, scale_ub: Tensor | None = None):
    """_dynamic_per_token_scaled_fp8_quant_torch
    (pretuned_kernels/dynamic_per_token_scaled_fp8_quant/dynamic_per_token_scaled_fp8_quant.py:77-99):
    per-row ``s = clamp(amax * (1/448), min=1/(448*512))``, ``q = fp8(clamp(x * (1/s)))`` -- a multiply by
    the reciprocal, not a division.  Returns ``(codes [T, H], scale [T, 1])``."""
    xf = x.to(torch.float32)
    s = xf.abs().amax(dim=-1)
    if scale_ub is not None:
        s = s.clamp(max=float(scale_ub))
    s = (s * (1.0 / FP8_MAX)).clamp(min=FP8_MIN_SCALE)
    y = xf * (1.0 / s[:, None])
    return y.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), s[:, None]


def rms_norm_per_block_quant(
    x: Tensor, weight: Tensor, epsilon: float, group_size: int, scale_ub: Tensor | None = None,
    residual: Tensor | None = None, rms_ulp_nudge: Tensor | None = None,
):
    """_rms_norm_per_block_quant_torch
    (pretuned_kernels/rms_norm_per_block_quant/rms_norm_per_block_quant.py:134-173): RMSNorm as in
    rms_norm_dynamic_per_token_quant, then one scale per ``group_size`` block of the hidden dimension and a
    true division.  Returns ``(codes [T, H], scale [T, H/group], new_residual or None)``; ``rms_ulp_nudge`` as in
    :func:`rms_norm_dynamic_per_token_quant`."""
    t, h = x.shape
    xf = x.to(torch.float32)
    new_res = None
    if residual is not None:
        xf = xf + residual.to(torch.float32)
        new_res = xf.to(residual.dtype)
    rms = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + epsilon)
    if rms_ulp_nudge is not None:
        rms = (rms.view(torch.int32) + rms_ulp_nudge.reshape(-1, 1).to(torch.int32)).view(torch.float32)
    normed = ((xf * rms).to(x.dtype) * weight[None, :]).to(torch.float32).reshape(t, h // group_size, group_size)
    s = normed.abs().amax(dim=-1)
    if scale_ub is not None:
        s = s.clamp(max=float(scale_ub))
    s = (s * (1.0 / FP8_MAX)).clamp(min=FP8_MIN_SCALE)
    q = (normed / s[:, :, None]).clamp(-FP8_MAX, FP8_MAX).reshape(t, h).to(torch.float8_e4m3fn)
    return q, s, new_res


def silu_mul_fp8(x: Tensor, scale: Tensor) -> Tensor:
    """silu_mul_fp8 (pretuned_kernels/silu_mul_fp8/silu_mul_fp8.py:29-59): SiLU and the product in the input
    type (torch rounds each to it), the result in fp32 times ``1 / scale``, cast to e4m3.  Values beyond the
    e4m3 range are clamped to +-448 first (the kernel's conversion saturates; torch's cast would give NaN)."""
    d = x.shape[-1] // 2
    a, b = x[..., :d], x[..., d:]
    result = (torch.nn.functional.silu(a) * b).to(torch.float32)
    inv = 1.0 / scale.reshape(()).to(torch.float32)
    return (result * inv).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def scaled_mm(
    a: Tensor, b: Tensor, scale_a: Tensor, scale_b: Tensor, bias: Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
) -> Tensor:
    """scaled_mm (pretuned_kernels/scaled_mm/scaled_mm.py:18-84): fp32 accumulation of ``a [M, K] @ b [K, N]``
    (FP8 operands, products exact), ``scale_a * acc`` then ``scale_b.T * acc`` in fp32, the cast to the output
    type, and only then the bias, added in the output type.  The accumulation runs in fp64 and is rounded to
    fp32 once: the reference leaves the summation order to the tiling.  For int8 operands the reference accumulates
    in int32 and converts to fp32 once (scaled_mm.py:53,66); fp64 holds those sums exactly, so this is that value."""
    m, _k = a.shape
    n = b.shape[1]
    acc = (a.to(torch.float64) @ b.to(torch.float64)).to(torch.float32)
    sa = scale_a.reshape(-1, 1).to(torch.float32)
    sb = scale_b.reshape(-1, 1).to(torch.float32)
    assert sa.shape[0] in (1, m) and sb.shape[0] in (1, n)
    acc = sa * acc
    acc = sb.T * acc
    c = acc.to(out_dtype)
    if bias is not None:
        c = c + bias.reshape(1, -1).to(out_dtype)
    return c


def rms_norm_row_rms(x: Tensor, epsilon: float, residual: Tensor | None = None) -> Tensor:
    """The fp32 ``rms`` factor of each row as the function above computes it (test helper)."""
    xf = x.to(torch.float32)
    if residual is not None:
        xf = xf + residual.to(torch.float32)
    return torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + epsilon)


def per_token_group_fp8_quant(
    x: Tensor, group_size: int, eps: float, fp8_min: float, fp8_max: float, scale_ue8m0: bool
):
    """_per_token_group_fp8_quant_torch
    (pretuned_kernels/per_token_group_fp8_quant/per_token_group_fp8_quant.py:77-97)."""
    t, h = x.shape
    xf = x.reshape(t, h // group_size, group_size).to(torch.float32)
    s = xf.abs().amax(dim=-1).clamp(min=eps) / fp8_max
    if scale_ue8m0:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    q = (xf / s[:, :, None]).clamp(fp8_min, fp8_max).to(torch.float8_e4m3fn)
    return q.reshape(t, h), s


# ------------------------------------------------------- grouped / MoE GEMM
def moe_matmul_ogs(a: Tensor, w: Tensor, top1_expert: Tensor) -> Tensor:
    """moe_matmul_ogs_reference (examples/moe_matmul_ogs.py:128-151): ``C[t] = A[t] @ W[e(t)]``;
    rows of experts nobody picked are left untouched (zero here)."""
    t, _ = a.shape
    n = w.shape[2]
    out = torch.zeros(t, n, dtype=torch.promote_types(a.dtype, w.dtype))
    for e in range(w.shape[0]):
        idx = (top1_expert == e).nonzero(as_tuple=True)[0]
        if idx.numel():
            out[idx] = (a[idx].to(torch.float32) @ w[e].to(torch.float32)).to(out.dtype)
    return out


def grouped_gemm_jagged(a_packed: Tensor, b: Tensor, group_offsets: Tensor) -> Tensor:
    """``torch.cat([A_i @ B])`` with a shared B (examples/grouped_gemm.py:52-104): equals A_packed @ B."""
    return (a_packed.to(torch.float32) @ b.to(torch.float32)).to(torch.promote_types(a_packed.dtype, b.dtype))


def grouped_gemm_worklist(a_packed: Tensor, b_grouped: Tensor, worklist: Tensor) -> Tensor:
    """``A[sum(align(M_g)), K] @ B[G, N, K]^T`` over ``(group, start, valid_m, store_m)`` rows
    (pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224; rows past valid_m read as
    zero, rows past store_m are not written)."""
    out = torch.zeros(a_packed.shape[0], b_grouped.shape[1], dtype=a_packed.dtype)
    for g, start, valid_m, store_m in worklist.tolist():
        rows = a_packed[start : start + store_m].to(torch.float32).clone()
        rows[valid_m:] = 0
        out[start : start + store_m] = (rows @ b_grouped[g].to(torch.float32).t()).to(out.dtype)
    return out


def moe_route(logits: Tensor, top_k: int):
    """Router of the MoE configuration: softmax over experts in fp32, top-k, weights used as produced
    (no renormalisation).  Returns ``(weights fp32 [T, k], experts int64 [T, k])``."""
    probs = torch.softmax(logits.to(torch.float32), dim=-1)
    w, e = torch.topk(probs, top_k, dim=-1)
    return w, e


def moe_sort(experts: Tensor, num_experts: int):
    """Stable sort of the flattened (token, slot) pairs by expert, as
    moe_matmul_ogs_helion_kernel_args_gen does for top-1 (examples/moe_matmul_ogs.py:89-124).
    Returns ``(sorted_pair_idx int32 [T*k], counts int32 [E], offsets int32 [E+1])``."""
    flat = experts.reshape(-1)
    order = torch.argsort(flat, stable=True).to(torch.int32)
    counts = torch.bincount(flat, minlength=num_experts).to(torch.int32)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0)
    return order, counts, offsets


def nvfp4_moe(
    x: Tensor, logits: Tensor, top_k: int,
    w_gu_packed: Tensor, w_gu_scale: list[Tensor] | Tensor, w_gu_global: Tensor,
    w_d_packed: Tensor, w_d_scale: list[Tensor] | Tensor, w_d_global: Tensor,
    return_pairs: bool = False, routing: tuple[Tensor, Tensor] | None = None,
):
    """NVFP4 MoE layer (composition; the reference has no NVFP4 MoE): route, then per expert
    quantise the gathered bf16 rows per token to NVFP4, ``h = deq(A) @ deq(W_gu)^T`` in fp32,
    ``y = silu(h[:, :I]) * h[:, I:]`` (gate first, as silu_and_mul_per_block_quant), requantise y per
    token, ``o = bf16(deq(y) @ deq(W_d)^T)``, and accumulate ``out[t] += weight * o`` in fp32; bf16 result.
    The per-expert loop is moe_matmul_ogs_reference's (examples/moe_matmul_ogs.py:128-151), which returns every
    expert's output rows in the activation dtype: ``o`` is rounded to bf16 before the routing-weighted sum.

    Weights: ``w_gu_packed [E, 2I, H/2]``, ``w_d_packed [E, H, I/2]``; scales are per-expert swizzled
    buffers; ``*_global`` are per-expert fp32 global scales ``[E]``.  The intermediate ``h`` is rounded to
    bf16 before SiLU-mul and ``y`` to bf16 before requantisation, as a bf16 activation pipeline does.
    Experts no token was routed to are never touched (their entries may be ``None`` in the scale lists).

    ``routing = (weights [T, k], experts [T, k])`` replaces the router (to compare the expert arithmetic
    alone when two routers disagree on a near-tie).  With ``return_pairs`` the result is
    ``(out, pairs)`` where ``pairs`` holds, per (token, slot) pair in expert order, the intermediate the
    second GEMM consumes: ``tok``, ``slot``, ``expert``, ``y`` (bf16 ``[P, I]``), ``codes`` (uint8 nibbles
    ``[P, I]``), ``scales`` (e4m3 ``[P, I/16]``, logical layout) and ``g`` (fp32 ``[P]``).
    """
    t, hdim = x.shape
    e_count = len(w_gu_packed)  # a tensor [E, ...] or a list with None for experts that are not needed
    inter = next(w for w in w_gu_packed if w is not None).shape[0] // 2
    weights, experts = moe_route(logits, top_k) if routing is None else routing
    out = torch.zeros(t, hdim, dtype=torch.float32)
    keep: dict[str, list[Tensor]] = {k: [] for k in ("tok", "slot", "expert", "y", "codes", "scales", "g")}
    for e in range(e_count):
        tok, slot = (experts == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        ap, asc, ag = nvfp4_quantize(x[tok], per_token=True)
        a = dequant_scaled_k_major(ap, asc) * ag.reshape(-1, 1)
        wgu = dequant_scaled_k_major(w_gu_packed[e], w_gu_scale[e]) * w_gu_global[e]
        h = (a @ wgu.t()).to(torch.bfloat16).to(torch.float32)
        y = (torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]).to(torch.bfloat16)
        yp, ysc, yg = nvfp4_quantize(y, per_token=True)
        if return_pairs:
            keep["tok"].append(tok)
            keep["slot"].append(slot)
            keep["expert"].append(torch.full_like(tok, e))
            keep["y"].append(y)
            keep["codes"].append(unpack_codes_k_major(yp))
            keep["scales"].append(unswizzle_scales(ysc, y.shape[0], inter // 16))
            keep["g"].append(yg)
        yq = dequant_scaled_k_major(yp, ysc) * yg.reshape(-1, 1)
        wd = dequant_scaled_k_major(w_d_packed[e], w_d_scale[e]) * w_d_global[e]
        o = (yq @ wd.t()).to(torch.bfloat16).to(torch.float32)
        out.index_add_(0, tok, o * weights[tok, slot].reshape(-1, 1))
    if return_pairs:
        return out.to(torch.bfloat16), {k: torch.cat(v) for k, v in keep.items()}
    return out.to(torch.bfloat16)


def unpack_codes_k_major(packed: Tensor) -> Tensor:
    """``[R, K/2]`` packed bytes -> ``[R, K]`` 4-bit codes (uint8), low nibble = even k."""
    b = _bytes(packed)
    return torch.stack((b & 0xF, b >> 4), dim=-1).reshape(b.shape[0], -1)


def nvfp4_moe_down(
    codes: Tensor, scales: Tensor, g: Tensor, tok: Tensor, slot: Tensor, expert: Tensor, weights: Tensor,
    w_d_packed: Tensor, w_d_scale: list[Tensor] | Tensor, w_d_global: Tensor, tokens: int,
) -> Tensor:
    """Second half of :func:`nvfp4_moe` from a given quantised intermediate (``codes [P, I]`` nibbles,
    ``scales [P, I/16]`` e4m3 logical, ``g [P]``): ``o = deq(y) @ deq(W_d)^T``, routing-weighted sum per token
    in fp32 over bf16 expert rows, bf16 result.  Used to show that an output difference comes from the
    intermediate's codes alone."""
    p, inter = codes.shape
    hdim = next(w for w in w_d_packed if w is not None).shape[0]
    yq = dequant_e2m1(codes) * scales.to(torch.float32).repeat_interleave(16, dim=1) * g.reshape(-1, 1)
    out = torch.zeros(tokens, hdim, dtype=torch.float32)
    for e in expert.unique().tolist():
        sel = (expert == e).nonzero(as_tuple=True)[0]
        wd = dequant_scaled_k_major(w_d_packed[e], w_d_scale[e]) * w_d_global[e]
        o = (yq[sel] @ wd.t()).to(torch.bfloat16).to(torch.float32)
        out.index_add_(0, tok[sel], o * weights[tok[sel], slot[sel]].reshape(-1, 1))
    return out.to(torch.bfloat16)
