"""Multi-GPU forms of the operators, one process per GPU over ``torch.distributed``.

Two partitionings, both from the shape of the work itself:

* column tensor parallelism for GEMV / GEMM: rank r owns rows ``[r*N/g, (r+1)*N/g)`` of the K-major
  weight and its scale tiles (``N/g`` must be a multiple of 128 so the 128-row scale tiles never
  straddle ranks); activations are replicated; the bf16 outputs are all-gathered.
* expert parallelism for the MoE layer: rank r owns experts ``[r*E/g, (r+1)*E/g)``; tokens start
  data-parallel, are dispatched to the ranks that own their experts with an all-to-all, and the
  expert outputs travel back with the mirrored all-to-all before the routing-weighted combine.

The collectives are the process group's (NCCL on GPUs, gloo in the CPU tests of the host logic).
The reference has no counterpart: its only multi-GPU code are fused matmul+collective example
kernels on symmetric memory (examples/distributed/), none for these operators.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
from torch import Tensor
import torch.distributed as dist


# ------------------------------------------------------------------ sharding helpers
def shard_range(n: int, world: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """Row range of ``rank`` when ``n`` rows are split evenly over ``world`` ranks."""
    if n % world:
        raise ValueError(f"{n} rows do not split evenly over {world} ranks")
    per = n // world
    if per % multiple:
        raise ValueError(f"rows per rank ({per}) must be a multiple of {multiple}")
    return rank * per, (rank + 1) * per


def shard_weight_rows(packed: Tensor, scales: Tensor, world: int, rank: int) -> tuple[Tensor, Tensor]:
    """Slice a K-major NVFP4 weight ``[N, K/2]`` and its swizzled scales to the rows of ``rank``.

    Because the scale buffer is ordered by 128-row tile, a row range that starts and ends on a multiple
    of 128 is a contiguous byte range of it.
    """
    n, kb = packed.shape
    lo, hi = shard_range(n, world, rank)
    col_tiles = -(-(kb // 8) // 4)
    flat = scales.reshape(-1)
    return packed[lo:hi], flat[(lo // 128) * col_tiles * 512 : (hi // 128) * col_tiles * 512]


def all_gather_columns(y_local: Tensor, group=None) -> Tensor:
    """``[M, N/g]`` per rank -> ``[M, N]`` on every rank (rank-major column blocks)."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    m, n_local = y_local.shape
    buf = torch.empty(world * m, n_local, dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(buf, y_local.contiguous(), group=group)
    return buf.reshape(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)


def column_parallel_gemv(weight_local: Tensor, scale_local: Tensor, x: Tensor, alpha: float = 1.0, group=None) -> Tensor:
    """``x [M, K]`` (replicated, 1 <= M <= 32) against this rank's weight rows; returns the gathered ``[M, N]``."""
    from . import ops

    if x.shape[0] == 1:
        y = ops.nvfp4_gemv_bf16in(weight_local, x.reshape(-1), scale_local, alpha).reshape(1, -1)
    else:
        y = ops.nvfp4_gemv_bf16in_batched(weight_local, x, scale_local, alpha)
    return all_gather_columns(y, group)


def column_parallel_matmul(a_packed: Tensor, scale_a: Tensor, b_local: Tensor, scale_b_local: Tensor,
                           alpha: float = 1.0, out_dtype: torch.dtype = torch.bfloat16, group=None) -> Tensor:
    """Block-scaled GEMM with B's rows (the output columns) split over the ranks; A is replicated."""
    from . import ops

    y = ops.nvfp4_scaled_matmul(a_packed, b_local.t(), scale_a, scale_b_local, out_dtype, alpha=alpha)
    return all_gather_columns(y, group)


# ------------------------------------------------------------------ expert parallelism
@dataclass
class DispatchPlan:
    """Who sends what in the dispatch all-to-all, for one rank."""

    order: Tensor            # int64 [P]: local (token, slot) pairs sorted by expert (hence by owner rank)
    send_counts: list[int]   # pairs going to each rank
    recv_counts: list[int]   # pairs arriving from each rank
    local_expert: Tensor     # int64 [sum(recv_counts)]: expert index, local to this rank, of every received row


def plan_dispatch(experts: Tensor, num_experts: int, group=None) -> DispatchPlan:
    """Sort this rank's (token, slot) pairs by expert and exchange the per-rank counts and expert ids.

    ``experts`` is ``[T_local, top_k]`` with global expert ids.  Counts are exchanged with a fixed-size
    all-to-all and read on the host (the variable-size all-to-all needs them as Python ints).
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
    per = num_experts // world
    flat = experts.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    owner_counts = torch.bincount(flat // per, minlength=world)
    recv = torch.empty_like(owner_counts)
    if world > 1:
        dist.all_to_all_single(recv, owner_counts, group=group)
    else:
        recv.copy_(owner_counts)
    send_counts = owner_counts.tolist()
    recv_counts = recv.tolist()
    ids_send = (flat[order] - (flat[order] // per) * per).contiguous()
    ids_recv = torch.empty(sum(recv_counts), dtype=torch.int64, device=experts.device)
    if world > 1:
        dist.all_to_all_single(ids_recv, ids_send, recv_counts, send_counts, group=group)
    else:
        ids_recv.copy_(ids_send)
    del rank
    return DispatchPlan(order, send_counts, recv_counts, ids_recv)


def exchange_rows(rows: Tensor, send_counts: list[int], recv_counts: list[int], group=None) -> Tensor:
    """Variable-size all-to-all of row blocks (rows sorted by destination rank)."""
    out = torch.empty(sum(recv_counts), rows.shape[1], dtype=rows.dtype, device=rows.device)
    if dist.get_world_size(group) == 1:
        out.copy_(rows)
    else:
        dist.all_to_all_single(out, rows.contiguous(), recv_counts, send_counts, group=group)
    return out


ExpertFn = Callable[[Tensor, Tensor], Tensor]  # (rows [R, H], local expert id [R]) -> rows [R, H]


def expert_parallel_moe(x: Tensor, router_logits: Tensor, top_k: int, num_experts: int, expert_fn: ExpertFn,
                        group=None) -> Tensor:
    """MoE layer over expert-parallel ranks.  ``x [T_local, H]`` are this rank's tokens; ``expert_fn`` applies
    this rank's experts to the rows it receives (no routing weight).  Returns bf16 ``[T_local, H]``."""
    from .moe import route_top_k

    weights, experts = route_top_k(router_logits, top_k)
    plan = plan_dispatch(experts, num_experts, group)
    token_of_pair = plan.order // top_k
    rows = exchange_rows(x[token_of_pair], plan.send_counts, plan.recv_counts, group)
    o = expert_fn(rows, plan.local_expert)
    back = exchange_rows(o, plan.recv_counts, plan.send_counts, group)
    # `back` is in sorted-pair order; weight every row and sum the top_k rows of each token in fp32
    w_sorted = weights.reshape(-1)[plan.order].to(torch.float32)
    out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
    out.index_add_(0, token_of_pair, back.to(torch.float32) * w_sorted[:, None])
    return out.to(torch.bfloat16)


def make_nvfp4_expert_fn(w_gate_up, w_down) -> ExpertFn:
    """``expert_fn`` running this rank's NVFP4 experts (``GroupedNvfp4Weight`` bundles of the local experts)
    through the grouped tcgen05 GEMMs."""
    from . import moe as M

    def fn(rows: Tensor, local_expert: Tensor) -> Tensor:
        if rows.shape[0] == 0:
            return rows.new_empty(0, w_down.n)
        sched = M.build_schedule(local_expert.reshape(-1, 1), w_gate_up.experts)
        a1, sf1, g1 = M._quantize_rows(rows.contiguous(), w_gate_up.k, sched, 1, None, False, gather=True)
        h1 = M.grouped_matmul(a1, sf1, w_gate_up, sched, g1)
        a2, sf2, g2 = M._quantize_rows(h1, w_down.k, sched, 1, None, True, gather=False)
        o = M.grouped_matmul(a2, sf2, w_down, sched, g2)
        return o[sched.row_of_pair.long()]

    return fn
