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


def grouped_matmul_f16(a: Tensor, b: Tensor, row_tiles: Tensor, out_rows: int | None = None) -> Tensor:
    """``out[r] = a[r] @ b[g(r)].T`` over the row tiles; ``a [R, K]``, ``b [G, N, K]`` (both K-major, same 2-byte
    dtype), ``row_tiles`` int32 ``[T, 4]`` = (group, first row, valid rows, rows to store) on the device."""
    _require_cuda(a, b, row_tiles)
    if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype is not a.dtype:
        raise TypeError(f"operands must both be bfloat16 or float16, got {a.dtype} and {b.dtype}")
    g, n, k = b.shape
    if a.shape[1] != k:
        raise ValueError("K dimension mismatch between A and B")
    k_pad = ceil_div(k, 8) * 8
    a = _pad_k(a, k_pad).contiguous()
    b = _pad_k(b, k_pad).contiguous()
    rows = a.shape[0] if out_rows is None else out_rows
    out = torch.zeros(rows, n, dtype=a.dtype, device=a.device)
    if rows and n and row_tiles.shape[0]:
        with torch.cuda.device(a.device):
            _lib.call(
                "hb200_grouped_gemm_f16", a.data_ptr(), b.data_ptr(), out.data_ptr(), row_tiles.data_ptr(),
                row_tiles.shape[0], a.shape[0], n, k_pad, g, n, int(a.dtype is torch.bfloat16), _stream(),
            )
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


def grouped_gemm_jagged(A_packed: Tensor, B: Tensor, group_offsets: Tensor) -> Tensor:  # noqa: N803
    """``torch.cat([A_i @ B])`` for row groups of ``A_packed`` and one shared ``B [K, N]``."""
    total_m, k = A_packed.shape
    k2, n = B.shape
    assert k == k2, "K dimension mismatch between A_packed and B"
    dtype = torch.promote_types(A_packed.dtype, B.dtype)
    tiles = row_tiles_from_offsets(group_offsets, total_m)
    return grouped_matmul_f16(A_packed.to(dtype), B.to(dtype).t().contiguous().unsqueeze(0), _single_group(tiles))


def _single_group(tiles: Tensor) -> Tensor:
    """All groups share one B: point every used tile at group 0."""
    t = tiles.clone()
    t[:, 0] = torch.where(t[:, 0] >= 0, torch.zeros_like(t[:, 0]), t[:, 0])
    return t


grouped_gemm_jagged_persistent = grouped_gemm_jagged


def grouped_gemm_deepgemm(a_packed: Tensor, b_grouped: Tensor, worklist: Tensor) -> Tensor:
    """``A[sum(align(M_g)), K] @ B[G, N, K].T`` over ``worklist [W, 4]`` = (group, start, valid_m, store_m)."""
    m_total, k = a_packed.shape
    _groups, n, k2 = b_grouped.shape
    assert k == k2, "K dimension mismatch between A and B"
    assert worklist.size(1) == 4
    # split every work item into 128-row tiles (tensor code on the device; the item count is static)
    wl = worklist.to(torch.int32)
    max_store = m_total  # bound on store_m without reading the worklist
    per_item = ceil_div(max_store, 128) if wl.shape[0] == 1 else None
    if per_item is None:
        # store_m of an item never exceeds the distance to the next item's start in a valid worklist,
        # so ceil(m_total / 128) + W tiles suffice overall; build them per item with a fixed fan-out.
        per_item = ceil_div(m_total, 128)
    i = torch.arange(per_item, dtype=torch.int32, device=wl.device)[None, :]
    start = wl[:, 1:2] + i * 128
    valid = (wl[:, 2:3] - i * 128).clamp(min=0, max=128)
    store = (wl[:, 3:4] - i * 128).clamp(min=0, max=128)
    group = torch.where(store > 0, wl[:, 0:1].expand_as(store), torch.full_like(store, -1))
    tiles = torch.stack((group, start, valid, store), dim=-1).reshape(-1, 4).contiguous()
    return grouped_matmul_f16(a_packed, b_grouped, tiles, out_rows=m_total)
