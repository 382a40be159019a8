"""bf16 / fp16 grouped GEMM entry points with the reference's call signatures, on the tcgen05 ``kind::f16`` kernel.

* :func:`moe_matmul_ogs` -- ``examples/moe_matmul_ogs.py:31-85`` (top-1 expert GEMM over sorted tokens)
* :func:`moe_matmul_ogs_helion_kernel_args_gen` -- ``examples/moe_matmul_ogs.py:89-124``, without the host read
* :func:`grouped_gemm_jagged` / :func:`grouped_gemm_jagged_persistent` -- ``examples/grouped_gemm.py:52-225``
* :func:`grouped_gemm_deepgemm` -- ``pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224``

The kernel wants both operands K-major.  The reference's ``W [E, K, N]`` and ``B [K, N]`` are N-major, so these
wrappers transpose them on the device first (a copy the caller can avoid by keeping weights K-major and calling
:func:`grouped_matmul_f16` directly).
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _lib
from .layouts import ceil_div
from .ops import _require_cuda
from .ops import _stream


def _pad_k(t: Tensor, k_pad: int) -> Tensor:
    return t if t.shape[-1] == k_pad else torch.nn.functional.pad(t, (0, k_pad - t.shape[-1]))


@torch.library.custom_op("helion_b200::grouped_matmul_f16_out", mutates_args=("out",))
def grouped_matmul_f16_out(out: Tensor, a: Tensor, b: Tensor, row_tiles: Tensor) -> None:
    """In-place form of :func:`grouped_matmul_f16`: rows of ``out [R, N]`` that no tile stores keep their contents."""
    _require_cuda(out, a, b, row_tiles)
    if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype is not a.dtype or out.dtype is not a.dtype:
        raise TypeError(f"operands and output must all be bfloat16 or all float16, got {a.dtype}, {b.dtype}, {out.dtype}")
    g, n, k = b.shape
    if a.shape[1] != k:
        raise ValueError("K dimension mismatch between A and B")
    if out.dim() != 2 or out.shape[1] != n or out.stride(1) != 1 or out.shape[0] < a.shape[0]:
        raise ValueError(f"out must be [>= {a.shape[0]}, {n}] with unit stride along N")
    k_pad = ceil_div(k, 8) * 8
    a = _pad_k(a, k_pad).contiguous()
    b = _pad_k(b, k_pad).contiguous()
    if a.shape[0] and n and row_tiles.shape[0]:
        with torch.cuda.device(a.device):
            _lib.call(
                "hb200_grouped_gemm_f16", a.data_ptr(), b.data_ptr(), out.data_ptr(), row_tiles.data_ptr(),
                row_tiles.shape[0], a.shape[0], n, k_pad, g, out.stride(0), int(a.dtype is torch.bfloat16), _stream(),
            )


@grouped_matmul_f16_out.register_fake
def _(out, a, b, row_tiles):
    return None


@torch.library.custom_op("helion_b200::grouped_matmul_f16", mutates_args=())
def grouped_matmul_f16(a: Tensor, b: Tensor, row_tiles: Tensor, out_rows: int | None = None) -> Tensor:
    """``out[r] = a[r] @ b[g(r)].T`` over the row tiles; ``a [R, K]``, ``b [G, N, K]`` (both K-major, same 2-byte
    dtype), ``row_tiles`` int32 ``[T, 4]`` = (group, first row, valid rows, rows to store) on the device.
    Rows no tile stores are zero."""
    rows = a.shape[0] if out_rows is None else out_rows
    out = torch.zeros(max(rows, a.shape[0]), b.shape[1], dtype=a.dtype, device=a.device)
    grouped_matmul_f16_out(out, a, b, row_tiles)
    return out[:rows] if rows != out.shape[0] else out


@grouped_matmul_f16.register_fake
def _(a, b, row_tiles, out_rows=None):
    return a.new_empty((a.shape[0] if out_rows is None else out_rows, b.shape[1]))


def row_tiles_from_split_sizes(split_sizes: Tensor, total_rows: int) -> Tensor:
    """Device-side tile list for groups given by per-group row counts ``split_sizes [G]`` (int32 or int64 on the
    device, any stride): group g owns rows ``[P_g, P_g + size_g)`` with ``P`` the raw running sum, clipped to the
    rows that exist (oversized and negative sizes are clipped, never trusted)."""
    _require_cuda(split_sizes)
    if split_sizes.dim() != 1 or split_sizes.dtype not in (torch.int32, torch.int64):
        raise ValueError("split_sizes must be a 1D int32 or int64 tensor")
    groups = split_sizes.numel()
    max_tiles = ceil_div(total_rows, 128) + groups
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=split_sizes.device)
    with torch.cuda.device(split_sizes.device):
        _lib.call("hb200_build_split_tiles", split_sizes.data_ptr(), int(split_sizes.dtype is torch.int64),
                  split_sizes.stride(0), groups, total_rows, tiles.data_ptr(), max_tiles, _stream())
    return tiles


def grouped_gemm_split_sizes(a: Tensor, b_grouped: Tensor, split_sizes: Tensor, out: Tensor | None = None) -> Tensor:
    """``out[rows of group g] = a[rows of group g] @ b_grouped[g].T`` with the groups given as device-resident row
    counts, the metadata form of the reference's grouped tcgen05 kernels
    (test/test_cute_grouped_gemm_split_sizes.py:620-745).  Nothing is read back, so a captured call can be
    replayed after ``split_sizes`` changed; with ``out`` given, rows no group covers keep their contents."""
    tiles = row_tiles_from_split_sizes(split_sizes, a.shape[0])
    if out is None:
        return grouped_matmul_f16(a, b_grouped, tiles)
    grouped_matmul_f16_out(out, a, b_grouped, tiles)
    return out


def row_tiles_from_offsets(group_offsets: Tensor, total_rows: int) -> Tensor:
    """Device-side tile list for groups delimited by ``group_offsets [G + 1]`` (int32 on the device)."""
    _require_cuda(group_offsets)
    groups = group_offsets.numel() - 1
    max_tiles = ceil_div(total_rows, 128) + groups
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=group_offsets.device)
    with torch.cuda.device(group_offsets.device):
        _lib.call("hb200_build_row_tiles", group_offsets.to(torch.int32).contiguous().data_ptr(), groups,
                  tiles.data_ptr(), max_tiles, _stream())
    return tiles


def moe_matmul_ogs_helion_kernel_args_gen(A: Tensor, W: Tensor, top1_expert_per_token: Tensor):  # noqa: N803
    """Same tuple as the reference's generator; ``max_T_per_expert`` is the bound ``T`` so nothing is read back."""
    e = W.size(0)
    sorted_to_orig = torch.argsort(top1_expert_per_token, stable=True).to(torch.int32)
    counts = torch.zeros(e, dtype=torch.int32, device=A.device)
    counts.index_add_(0, top1_expert_per_token.reshape(-1), torch.ones_like(top1_expert_per_token, dtype=torch.int32))
    offsets = torch.zeros(e + 1, dtype=torch.int32, device=A.device)
    offsets[1:] = torch.cumsum(counts, 0, dtype=torch.int32)
    return A, W, counts, offsets, sorted_to_orig, int(A.shape[0])


@torch.library.custom_op("helion_b200::moe_matmul_ogs", mutates_args=())
def moe_matmul_ogs(A: Tensor, W: Tensor, expert_token_counts: Tensor, expert_token_offsets: Tensor,  # noqa: N803
                   sorted_to_orig_token_idx: Tensor, max_T_per_expert: int) -> Tensor:  # noqa: N803
    """``C[t] = A[t] @ W[e(t)]`` with ``W [E, K, N]``; tokens of expert ``e`` are
    ``sorted_to_orig_token_idx[offsets[e] : offsets[e] + counts[e]]``.  Rows no expert owns stay zero."""
    del expert_token_counts, max_T_per_expert  # implied by the offsets
    t, k = A.shape
    e, k2, n = W.shape
    if k != k2:
        raise ValueError("K dimension mismatch between A and W")
    dtype = torch.promote_types(A.dtype, W.dtype)
    a_sorted = A.to(dtype).index_select(0, sorted_to_orig_token_idx.long())
    w_k_major = W.to(dtype).transpose(1, 2).contiguous()
    tiles = row_tiles_from_offsets(expert_token_offsets, t)
    out_sorted = grouped_matmul_f16(a_sorted, w_k_major, tiles)
    c = torch.zeros(t, n, dtype=dtype, device=A.device)
    c.index_copy_(0, sorted_to_orig_token_idx.long(), out_sorted)
    return c


@moe_matmul_ogs.register_fake
def _(A, W, expert_token_counts, expert_token_offsets, sorted_to_orig_token_idx, max_T_per_expert):  # noqa: N803
    return A.new_empty((A.shape[0], W.shape[2]), dtype=torch.promote_types(A.dtype, W.dtype))


@torch.library.custom_op("helion_b200::grouped_gemm_jagged", mutates_args=())
def grouped_gemm_jagged(A_packed: Tensor, B: Tensor, group_offsets: Tensor) -> Tensor:  # noqa: N803
    """``torch.cat([A_i @ B])`` for row groups of ``A_packed`` and one shared ``B [K, N]``."""
    total_m, k = A_packed.shape
    k2, n = B.shape
    assert k == k2, "K dimension mismatch between A_packed and B"
    dtype = torch.promote_types(A_packed.dtype, B.dtype)
    tiles = row_tiles_from_offsets(group_offsets, total_m)
    return grouped_matmul_f16(A_packed.to(dtype), B.to(dtype).t().contiguous().unsqueeze(0), _single_group(tiles))


@grouped_gemm_jagged.register_fake
def _(A_packed, B, group_offsets):  # noqa: N803
    return A_packed.new_empty((A_packed.shape[0], B.shape[1]), dtype=torch.promote_types(A_packed.dtype, B.dtype))


def _single_group(tiles: Tensor) -> Tensor:
    """All groups share one B: point every used tile at group 0."""
    t = tiles.clone()
    t[:, 0] = torch.where(t[:, 0] >= 0, torch.zeros_like(t[:, 0]), t[:, 0])
    return t


grouped_gemm_jagged_persistent = grouped_gemm_jagged


@torch.library.custom_op("helion_b200::grouped_gemm_deepgemm", mutates_args=())
def grouped_gemm_deepgemm(a_packed: Tensor, b_grouped: Tensor, worklist: Tensor) -> Tensor:
    """``A[sum(align(M_g)), K] @ B[G, N, K].T`` over ``worklist [W, 4]`` = (group, start, valid_m, store_m).

    The items are cut into 128-row tiles on the device (``hb200_build_worklist_tiles``): item ``i`` owns the
    tile slots ``[start_i / 128 + i, ...)``, which never collide for items whose row ranges do not overlap, so
    ``ceil(m_total / 128) + W`` slots suffice and nothing is read back to the host.
    """
    m_total, k = a_packed.shape
    _groups, n, k2 = b_grouped.shape
    assert k == k2, "K dimension mismatch between A and B"
    assert worklist.size(1) == 4
    _require_cuda(a_packed, b_grouped, worklist)
    wl = worklist.to(torch.int32).contiguous()
    items = wl.shape[0]
    max_tiles = ceil_div(m_total, 128) + items
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=wl.device)
    with torch.cuda.device(wl.device):
        _lib.call("hb200_build_worklist_tiles", wl.data_ptr(), items, m_total, tiles.data_ptr(), max_tiles, _stream())
    return grouped_matmul_f16(a_packed, b_grouped, tiles, out_rows=m_total)


@grouped_gemm_deepgemm.register_fake
def _(a_packed, b_grouped, worklist):
    return a_packed.new_empty((a_packed.shape[0], b_grouped.shape[1]))
