"""NVFP4 mixture-of-experts layer on the grouped tcgen05 GEMM.

The reference ships a top-1 bf16/fp16 expert GEMM (``moe_matmul_ogs``,
examples/moe_matmul_ogs.py:31-124) whose argument generator sorts tokens by expert
on the host side of the stream and reads ``max_T_per_expert`` back.  This module is
the NVFP4, top-k form of that operator: routing (softmax, top-k, stable sort by
expert) stays in tensor code on the device, the schedule is built by a kernel, and
nothing synchronises with the host.

Pipeline for tokens ``x [T, H]``:
  route -> per-token NVFP4 quantisation of the gathered rows -> grouped GEMM with
  ``W_gu [E, 2I, H]`` (bf16 out) -> fused SiLU-mul + per-token NVFP4 quantisation ->
  grouped GEMM with ``W_d [E, H, I]`` (routing weight folded into the row scale) ->
  combine over the top-k slots.
"""

from __future__ import annotations

import os

from dataclasses import dataclass

import torch
from torch import Tensor

from . import _lib
from .layouts import ceil_div
from .layouts import nvfp4_global_scale
from .layouts import swizzled_scale_numel
from .ops import _require_cuda
from .ops import _stream


@dataclass
class GroupedNvfp4Weight:
    """Expert weights ``[E, N, K]`` quantised to NVFP4: packed codes ``[E, N, K/2]`` (uint8), one swizzled
    e4m3 scale buffer per expert back to back (``[E, swizzled_scale_numel(N, K/16)]``) and one fp32 global
    scale per expert ``[E]``."""

    packed: Tensor
    scales: Tensor
    global_scale: Tensor
    # rows interleave gate and up in blocks of 128 (see interleave_gate_up); lets the first expert GEMM
    # apply SiLU-mul in its epilogue
    gate_up_interleaved: bool = False

    @property
    def experts(self) -> int:
        return self.packed.shape[0]

    @property
    def n(self) -> int:
        return self.packed.shape[1]

    @property
    def k(self) -> int:
        return self.packed.shape[2] * 2


def quantize_expert_weights(w: Tensor) -> GroupedNvfp4Weight:
    """``[E, N, K]`` float weights -> :class:`GroupedNvfp4Weight` with a global scale per expert (on ``w``'s device,
    through the CUDA quantiser)."""
    from .ops import nvfp4_quantize

    e, n, k = w.shape
    packed = torch.empty(e, n, k // 2, dtype=torch.uint8, device=w.device)
    scales = torch.empty(e, swizzled_scale_numel(n, k // 16), dtype=torch.uint8, device=w.device)
    gs = torch.empty(e, dtype=torch.float32, device=w.device)
    for i in range(e):
        wb = w[i].to(torch.bfloat16)  # the quantiser consumes bf16; the global scale must see the same values
        g = nvfp4_global_scale(wb).reshape(1)
        c, s, _ = nvfp4_quantize(wb, g)
        packed[i], scales[i], gs[i] = c, s.view(torch.uint8), g[0]
    return GroupedNvfp4Weight(packed, scales.view(torch.float8_e4m3fn), gs)


def interleave_gate_up(w: GroupedNvfp4Weight) -> GroupedNvfp4Weight:
    """Reorder the rows of a gate||up weight ``[E, 2I, K]`` (gate rows first, as the reference's
    silu_and_mul kernels expect) into blocks of 128 gate rows followed by the 128 up rows of the same
    outputs, codes and scale tiles alike (a 128-row block is one scale row-tile, so whole tiles move)."""
    if w.gate_up_interleaved:
        return w
    e, n, kb = w.packed.shape
    inter = n // 2
    if n % 256:
        raise ValueError(f"gate||up rows ({n}) must be a multiple of 256 to interleave in blocks of 128")
    packed = w.packed.view(e, 2, inter // 128, 128, kb).permute(0, 2, 1, 3, 4).reshape(e, n, kb).contiguous()
    tile_bytes = w.scales.numel() // (e * (n // 128))
    scales = (w.scales.view(torch.uint8).view(e, 2, inter // 128, tile_bytes).permute(0, 2, 1, 3)
              .reshape(e, -1).contiguous().view(torch.float8_e4m3fn))
    return GroupedNvfp4Weight(packed, scales, w.global_scale, True)


_ROUTE_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


@torch.library.custom_op("helion_b200::moe_route_top_k", mutates_args=())
def _route_top_k_op(logits: Tensor, top_k: int) -> tuple[Tensor, Tensor]:
    _require_cuda(logits)
    tokens, experts = logits.shape
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=logits.device)
    chosen = torch.empty((tokens, top_k), dtype=torch.int64, device=logits.device)
    with torch.cuda.device(logits.device):
        _lib.call("hb200_moe_route_top_k", logits.data_ptr(), _ROUTE_DTYPES[logits.dtype], tokens, experts, top_k,
                  weights.data_ptr(), chosen.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return weights, chosen


@_route_top_k_op.register_fake
def _(logits, top_k):
    return (logits.new_empty((logits.shape[0], top_k), dtype=torch.float32),
            logits.new_empty((logits.shape[0], top_k), dtype=torch.int64))


def route_top_k(router_logits: Tensor, top_k: int) -> tuple[Tensor, Tensor]:
    """softmax over experts in fp32, then top-k, in one kernel; weights are used as produced (not renormalised).

    Returns ``(weights [T, top_k] fp32, experts [T, top_k] int64)`` in descending order of weight, as
    ``torch.topk(torch.softmax(logits.float(), -1), top_k)`` does.
    """
    if router_logits.dim() != 2:
        raise ValueError("router_logits must be [tokens, experts]")
    tokens, experts = router_logits.shape
    if not 0 < top_k <= experts:
        raise ValueError(f"top_k must be in 1..{experts}, got {top_k}")
    if router_logits.dtype not in _ROUTE_DTYPES:
        router_logits = router_logits.to(torch.float32)
    if experts > 1024:
        raise ValueError(f"at most 1024 experts are supported, got {experts}")
    return _route_top_k_op(router_logits.contiguous(), top_k)


@dataclass
class MoeSchedule:
    max_tiles: int
    tile_info: Tensor       # int32 [max_tiles, 2]
    padded_offsets: Tensor  # int32 [E + 1]
    sorted_pairs: Tensor    # int32 [T * top_k]
    row_of_sorted: Tensor   # int32 [T * top_k]
    row_of_pair: Tensor     # int32 [T * top_k]
    pad: int = 128          # every expert's rows are padded to a multiple of this (128, or 256 for CTA-pair tiles)


def _max_tiles(pairs: int, num_experts: int, pad: int) -> int:
    # bound that does not depend on the routing (in 128-row units; even for 256-row padding)
    max_tiles = ceil_div(pairs, 128) + num_experts * (pad // 128)
    return max_tiles + max_tiles % (pad // 128)


@torch.library.custom_op("helion_b200::moe_build_schedule", mutates_args=())
def _build_schedule_op(flat: Tensor, num_experts: int, pad: int) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    _require_cuda(flat)
    pairs = flat.numel()
    dev = flat.device
    # stable counting sort + per-expert counts in three small launches (no radix sort, no host read)
    sorted_pairs = torch.empty(pairs, dtype=torch.int32, device=dev)
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    scratch = torch.empty(max(1, ceil_div(pairs, 1024)) * num_experts, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("hb200_moe_sort_pairs", flat.data_ptr(), int(flat.dtype is torch.int64), pairs, num_experts,
                  sorted_pairs.data_ptr(), counts.data_ptr(), scratch.data_ptr(), _stream())
    max_tiles = _max_tiles(pairs, num_experts, pad)
    tile_info = torch.empty(max_tiles, 2, dtype=torch.int32, device=dev)
    padded_offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    row_of_sorted = torch.empty(pairs, dtype=torch.int32, device=dev)
    row_of_pair = torch.empty(pairs, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "hb200_moe_build_schedule" if pad == 128 else "hb200_moe_build_schedule_256",
            counts.data_ptr(), num_experts, sorted_pairs.data_ptr(), pairs,
            padded_offsets.data_ptr(), tile_info.data_ptr(), max_tiles, row_of_sorted.data_ptr(),
            row_of_pair.data_ptr(), _stream(),
        )
    return tile_info, padded_offsets, sorted_pairs, row_of_sorted, row_of_pair


@_build_schedule_op.register_fake
def _(flat, num_experts, pad):
    pairs = flat.numel()
    i32 = dict(dtype=torch.int32)
    return (flat.new_empty((_max_tiles(pairs, num_experts, pad), 2), **i32), flat.new_empty((num_experts + 1,), **i32),
            flat.new_empty((pairs,), **i32), flat.new_empty((pairs,), **i32), flat.new_empty((pairs,), **i32))


def build_schedule(experts_per_token: Tensor, num_experts: int, pad: int = 128) -> MoeSchedule:
    """Sort the (token, slot) pairs by expert (stable, as examples/moe_matmul_ogs.py:107-109 does for
    top-1) and lay the experts out in groups padded to ``pad`` rows (128, or 256 for the CTA-pair grouped
    GEMM); all on the device."""
    if pad not in (128, 256):
        raise ValueError(f"pad must be 128 or 256, got {pad}")
    flat = experts_per_token.reshape(-1).contiguous()
    if flat.dtype not in (torch.int64, torch.int32):
        flat = flat.to(torch.int64)
    tile_info, padded_offsets, sorted_pairs, row_of_sorted, row_of_pair = _build_schedule_op(flat, num_experts, pad)
    return MoeSchedule(tile_info.shape[0], tile_info, padded_offsets, sorted_pairs, row_of_sorted, row_of_pair, pad)


def _quantize_rows(x: Tensor, k: int, sched: MoeSchedule, src_div: int, item_scale: Tensor | None, silu_mul: bool,
                   gather: bool):
    rows = sched.max_tiles * 128
    dev = x.device
    codes = torch.empty(rows, k // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(swizzled_scale_numel(rows, k // 16), dtype=torch.uint8, device=dev)
    gscale = torch.zeros(rows, dtype=torch.float32, device=dev)
    items = sched.sorted_pairs.numel()
    with torch.cuda.device(dev):
        _lib.call(
            "hb200_nvfp4_quantize_rows", x.data_ptr(), codes.data_ptr(), scales.data_ptr(), gscale.data_ptr(),
            items, k, x.stride(0),
            sched.sorted_pairs.data_ptr() if gather else sched.row_of_sorted.data_ptr(), src_div,
            sched.row_of_sorted.data_ptr(), None if item_scale is None else item_scale.data_ptr(),
            int(silu_mul), _stream(),
        )
    return codes, scales, gscale


def _quantize_and_gather(x: Tensor, sched: MoeSchedule, top_k: int, fused: bool = True):
    """Quantise every token row once (per-token global scale) and place its packed row at the rows of all its
    (token, slot) pairs in the expert-sorted padded layout -- an eighth of the arithmetic of quantising every pair.
    ``fused``: one kernel that writes the top-k copies itself (K % 64 == 0, K <= 4096); otherwise the quantiser
    followed by a row-gather kernel (same bytes)."""
    from .ops import nvfp4_quantize

    t, k = x.shape
    if k % 32:
        return _quantize_rows(x, k, sched, top_k, None, False, gather=True)
    rows = sched.max_tiles * 128
    dev = x.device
    codes = torch.empty(rows, k // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(swizzled_scale_numel(rows, k // 16), dtype=torch.uint8, device=dev)
    gscale = torch.zeros(rows, dtype=torch.float32, device=dev)
    if fused and k % 64 == 0 and k <= 4096 and top_k <= 32 and x.stride(0) % 8 == 0:
        with torch.cuda.device(dev):
            _lib.call("hb200_nvfp4_quantize_scatter", x.data_ptr(), codes.data_ptr(), scales.data_ptr(), gscale.data_ptr(),
                      sched.row_of_pair.data_ptr(), t, top_k, k, x.stride(0), _stream())
        return codes, scales, gscale
    codes_t, scales_t, g_t = nvfp4_quantize(x)
    with torch.cuda.device(dev):
        _lib.call(
            "hb200_moe_gather_rows", codes_t.data_ptr(), scales_t.data_ptr(), g_t.data_ptr(), codes.data_ptr(),
            scales.data_ptr(), gscale.data_ptr(), sched.sorted_pairs.data_ptr(), top_k,
            sched.row_of_sorted.data_ptr(), sched.sorted_pairs.numel(), k, _stream(),
        )
    return codes, scales, gscale


def grouped_matmul(a_codes: Tensor, a_scales: Tensor, w: GroupedNvfp4Weight, sched: MoeSchedule,
                   row_scale: Tensor | None, out_dtype: torch.dtype = torch.bfloat16) -> Tensor:
    """``out[r] = row_scale[r] * w.global_scale[g(r)] * A[r] @ W[g(r)]^T`` over the padded row layout."""
    rows = sched.max_tiles * 128
    out = torch.empty(rows, w.n, dtype=out_dtype, device=a_codes.device)
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out_dtype]
    with torch.cuda.device(a_codes.device):
        _lib.call(
            "hb200_nvfp4_grouped_matmul_256" if sched.pad == 256 else "hb200_nvfp4_grouped_matmul",
            a_codes.data_ptr(), w.packed.data_ptr(), a_scales.data_ptr(),
            w.scales.data_ptr(), out.data_ptr(), sched.tile_info.data_ptr(), sched.max_tiles, w.n, w.k,
            w.experts, w.n, None if row_scale is None else row_scale.data_ptr(), w.global_scale.data_ptr(),
            1.0, code, _stream(),
        )
    return out


def grouped_matmul_silu(a_codes: Tensor, a_scales: Tensor, w: GroupedNvfp4Weight, sched: MoeSchedule,
                        row_scale: Tensor | None) -> tuple[Tensor, Tensor]:
    """First expert GEMM with SiLU-mul in the epilogue (``w`` gate/up interleaved): returns
    ``y = bf16(silu(gate) * up) [rows, N/2]`` and every row's ``max |y|``."""
    if not w.gate_up_interleaved:
        raise ValueError("the SiLU-mul epilogue needs a gate/up weight interleaved with interleave_gate_up()")
    rows = sched.max_tiles * 128
    y = torch.empty(rows, w.n // 2, dtype=torch.bfloat16, device=a_codes.device)
    row_amax = torch.empty(rows, dtype=torch.float32, device=a_codes.device)
    with torch.cuda.device(a_codes.device):
        _lib.call(
            "hb200_nvfp4_grouped_matmul_silu_256" if sched.pad == 256 else "hb200_nvfp4_grouped_matmul_silu", a_codes.data_ptr(), w.packed.data_ptr(), a_scales.data_ptr(),
            w.scales.data_ptr(), y.data_ptr(), row_amax.data_ptr(), sched.tile_info.data_ptr(), sched.max_tiles, w.n,
            w.k, w.experts, w.n // 2, None if row_scale is None else row_scale.data_ptr(),
            w.global_scale.data_ptr(), 1.0, _stream(),
        )
    return y, row_amax


def _quantize_rows_amax(y: Tensor, row_amax: Tensor, k: int, sched: MoeSchedule, item_scale: Tensor | None):
    rows = sched.max_tiles * 128
    dev = y.device
    codes = torch.empty(rows, k // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(swizzled_scale_numel(rows, k // 16), dtype=torch.uint8, device=dev)
    gscale = torch.zeros(rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call(
            "hb200_nvfp4_quantize_rows_amax", y.data_ptr(), codes.data_ptr(), scales.data_ptr(), gscale.data_ptr(),
            row_amax.data_ptr(), sched.sorted_pairs.numel(), k, y.stride(0), sched.row_of_sorted.data_ptr(),
            None if item_scale is None else item_scale.data_ptr(), _stream(),
        )
    return codes, scales, gscale


@torch.library.custom_op("helion_b200::nvfp4_moe", mutates_args=())
def _nvfp4_moe_op(x: Tensor, router_logits: Tensor, top_k: int, gu_packed: Tensor, gu_scales: Tensor,
                  gu_global: Tensor, gu_interleaved: bool, d_packed: Tensor, d_scales: Tensor, d_global: Tensor) -> Tensor:
    return _nvfp4_moe_impl(x, router_logits, top_k, GroupedNvfp4Weight(gu_packed, gu_scales, gu_global, gu_interleaved),
                           GroupedNvfp4Weight(d_packed, d_scales, d_global), None)


@_nvfp4_moe_op.register_fake
def _(x, router_logits, top_k, gu_packed, gu_scales, gu_global, gu_interleaved, d_packed, d_scales, d_global):
    return x.new_empty(x.shape)


def nvfp4_moe(x: Tensor, router_logits: Tensor, top_k: int, w_gate_up: GroupedNvfp4Weight,
              w_down: GroupedNvfp4Weight, *, intermediates: dict | None = None) -> Tensor:
    """NVFP4 MoE layer: ``x [T, H]`` bf16, ``router_logits [T, E]`` -> bf16 ``[T, H]``
    (``torch.ops.helion_b200.nvfp4_moe`` on the bundles' tensors).

    The top-k, NVFP4 form of ``moe_matmul_ogs`` (examples/moe_matmul_ogs.py:31-124): softmax-then-top-k routing
    weights used without renormalisation, per-token NVFP4 activations, SiLU-mul between the two expert GEMMs
    (gate rows first), routing-weighted sum over the top-k slots in slot order.

    ``intermediates`` (a dict, filled in place) receives what the second expert GEMM consumes, for parity
    checks: the routing (``weights``, ``experts``), the schedule (``sched``) and, over the padded row layout,
    the re-quantised SiLU-mul output (``a2`` packed codes, ``sf2`` swizzled scales, ``g2`` per-row global scales)
    and ``y`` (bf16 SiLU-mul output) when the fused epilogue produced it.
    """
    _require_cuda(x, router_logits)
    if x.dtype is not torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous 2D bfloat16 tensor")
    h = x.shape[1]
    e = w_gate_up.experts
    inter = w_gate_up.n // 2
    if w_gate_up.k != h or w_down.k != inter or w_down.n != h or w_down.experts != e:
        raise ValueError("expert weight shapes do not match the activations")
    if intermediates is not None:
        return _nvfp4_moe_impl(x, router_logits, top_k, w_gate_up, w_down, intermediates)
    return _nvfp4_moe_op(x, router_logits, top_k, w_gate_up.packed, w_gate_up.scales, w_gate_up.global_scale,
                         w_gate_up.gate_up_interleaved, w_down.packed, w_down.scales, w_down.global_scale)


def _row_padding(pairs: int, experts: int, n1: int, n2: int) -> int:
    """Rows every expert is padded to: 128, or 256 (CTA-pair tiles) when ``HB200_MOE_PAD=256`` asks for it and both
    GEMMs' N are multiples of 256.  Both layouts give the same output bit for bit.  Measured on 8192 tokens x 128
    experts x top-8 (512 rows per expert): pairs move a third fewer operand bytes into every SM, but their one
    accumulator stage costs a drain per tile and the 256-row padding an eighth more rows, and the step is 3 % slower."""
    if os.environ.get("HB200_MOE_PAD") == "256" and n1 % 256 == 0 and n2 % 256 == 0:
        return 256
    return 128


def _nvfp4_moe_impl(x: Tensor, router_logits: Tensor, top_k: int, w_gate_up: GroupedNvfp4Weight,
                    w_down: GroupedNvfp4Weight, intermediates: dict | None) -> Tensor:
    t, h = x.shape
    e = w_gate_up.experts
    inter = w_gate_up.n // 2
    weights, experts = route_top_k(router_logits, top_k)
    sched = build_schedule(experts, e, _row_padding(t * top_k, e, w_gate_up.n, h))
    a1, sf1, g1 = _quantize_and_gather(x, sched, top_k)
    y = None
    if w_gate_up.gate_up_interleaved:
        # SiLU-mul in the GEMM's epilogue: the [rows, 2I] intermediate never reaches memory
        y, row_amax = grouped_matmul_silu(a1, sf1, w_gate_up, sched, g1)
        a2, sf2, g2 = _quantize_rows_amax(y, row_amax, inter, sched, None)
    else:
        h1 = grouped_matmul(a1, sf1, w_gate_up, sched, g1)
        a2, sf2, g2 = _quantize_rows(h1, inter, sched, 1, None, True, gather=False)
    # every expert's output rows in bf16, as moe_matmul_ogs returns them; the routing weights enter in the combine
    o = grouped_matmul(a2, sf2, w_down, sched, g2)
    out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _lib.call("hb200_moe_combine", o.data_ptr(), o.stride(0), sched.row_of_pair.data_ptr(),
                  weights.reshape(-1).data_ptr(), out.data_ptr(), t, top_k, h, _stream())
    if intermediates is not None:
        intermediates.update(weights=weights, experts=experts, sched=sched, a2=a2, sf2=sf2, g2=g2, y=y)
    return out
