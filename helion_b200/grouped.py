"""bf16 / fp16 grouped GEMM entry points with the reference's call signatures, on the tcgen05 ``kind::f16`` kernel.

* :func:`moe_matmul_ogs` -- ``examples/moe_matmul_ogs.py:31-85`` (top-1 expert GEMM over sorted tokens)
* :func:`moe_matmul_ogs_helion_kernel_args_gen` -- ``examples/moe_matmul_ogs.py:89-124``, without the host read
* :func:`grouped_gemm_jagged` / :func:`grouped_gemm_jagged_persistent` -- ``examples/grouped_gemm.py:52-225``
* :func:`grouped_gemm_deepgemm` -- ``pretuned_kernels/grouped_gemm_deepgemm/grouped_gemm_deepgemm.py:172-224``
* :func:`grouped_gemm` (direct mode, per-group N and K) -- ``pretuned_kernels/grouped_gemm/grouped_gemm.py:213-327``

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


# ------------------------------------------------------------------ direct mode (heterogeneous groups)
@torch.library.custom_op("helion_b200::grouped_gemm_direct", mutates_args=("outputs",))
def grouped_gemm_direct(group_a: list[Tensor], group_b: list[Tensor], outputs: list[Tensor]) -> None:
    """``outputs[i] <- group_a[i] @ group_b[i].T`` (fp32 accumulate) for groups with their own M, N and K:
    ``group_a[i] [M_i, K_i]``, ``group_b[i] [N_i, K_i]``, ``outputs[i] [M_i, N_i]``, all fp16 or all bf16, unit stride
    along the last dimension, any row pitch, anywhere in device memory.  One launch per eight groups; nothing is
    allocated or copied (K_i % 8 == 0)."""
    import ctypes

    groups = len(group_a)
    if len(group_b) != groups or len(outputs) != groups:
        raise ValueError("group_a, group_b and outputs must have one entry per group")
    if groups == 0:
        return
    _require_cuda(*group_a, *group_b, *outputs)
    dtype = group_a[0].dtype
    if dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"operands must be bfloat16 or float16, got {dtype}")
    for a, b, o in zip(group_a, group_b, outputs):
        if a.dtype is not dtype or b.dtype is not dtype or o.dtype is not dtype:
            raise TypeError("all operands and outputs must share one 2-byte dtype")
        if a.dim() != 2 or b.dim() != 2 or o.dim() != 2 or a.shape[1] != b.shape[1] or o.shape != (a.shape[0], b.shape[0]):
            raise ValueError(f"group shapes do not form A[M,K] @ B[N,K].T -> [M,N]: {tuple(a.shape)}, {tuple(b.shape)}, {tuple(o.shape)}")
        if (a.numel() and a.stride(1) != 1) or (b.numel() and b.stride(1) != 1) or (o.numel() and o.stride(1) != 1):
            raise ValueError("operands and outputs need unit stride along their last dimension")

    def arr(ctype, values):
        return (ctype * groups)(*values)

    pitch = lambda t: t.stride(0) if t.shape[0] > 1 else max(t.shape[1], 1)  # noqa: E731
    args = (
        arr(ctypes.c_void_p, [t.data_ptr() for t in group_a]), arr(ctypes.c_void_p, [t.data_ptr() for t in group_b]),
        arr(ctypes.c_void_p, [t.data_ptr() for t in outputs]),
        arr(ctypes.c_int64, [t.shape[0] for t in group_a]), arr(ctypes.c_int64, [t.shape[0] for t in group_b]),
        arr(ctypes.c_int64, [t.shape[1] for t in group_a]),
        arr(ctypes.c_int64, [pitch(t) for t in group_a]), arr(ctypes.c_int64, [pitch(t) for t in group_b]),
        arr(ctypes.c_int64, [pitch(t) for t in outputs]),
    )
    with torch.cuda.device(group_a[0].device):
        _lib.call("hb200_grouped_gemm_f16_direct", *args, groups, int(dtype is torch.bfloat16), _stream())


@grouped_gemm_direct.register_fake
def _(group_a, group_b, outputs):
    return None


_DIRECT_PLANS: dict[tuple, tuple] = {}


def grouped_gemm(a_placeholder: Tensor, b_placeholder: Tensor, layout: Tensor, n_sizes: Tensor, k_sizes: Tensor,
                 out_placeholder: Tensor, direct_pointers: Tensor, direct_strides: Tensor,
                 problem_signature: tuple[int, ...]) -> Tensor:
    """Grouped ``A_g[M_g, K_g] @ B_g[N_g, K_g].T`` with direct runtime metadata: drop-in for ``grouped_gemm``
    (pretuned_kernels/grouped_gemm/grouped_gemm.py:213-253) as ``_prepare_helion`` (:261-327) calls it.

    ``direct_pointers`` (int64 ``[G, 3]``: A, B, out) and ``direct_strides`` (int32 ``[G, 3, 2]``) are the device
    tables the reference builds from host values; ``problem_signature`` = ``(G, M_0, N_0, K_0, M_1, ...)`` carries
    the real per-group sizes (the placeholders, ``layout``, ``n_sizes`` and ``k_sizes`` repeat them in forms this
    kernel does not need).  The tables are read back once per (table, signature) and the launch plan is cached, so
    later calls -- including captured ones -- touch no host-device copy; the first call must come before capture.
    Operand dtype is the placeholders'.  Returns ``out_placeholder``.
    """
    import ctypes

    del layout, n_sizes, k_sizes  # the padded row layout and the size vectors restate problem_signature
    groups = int(problem_signature[0])
    sizes = [tuple(int(v) for v in problem_signature[1 + 3 * g : 4 + 3 * g]) for g in range(groups)]
    dtype = a_placeholder.dtype
    if dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"operands must be bfloat16 or float16, got {dtype}")
    if direct_pointers.shape != (groups, 3) or direct_pointers.dtype is not torch.int64:
        raise ValueError(f"direct_pointers must be int64 [{groups}, 3]")
    if direct_strides.shape != (groups, 3, 2):
        raise ValueError(f"direct_strides must be [{groups}, 3, 2]")
    _require_cuda(direct_pointers, direct_strides)
    key = (direct_pointers.data_ptr(), direct_pointers._version, direct_strides.data_ptr(), direct_strides._version,
           tuple(problem_signature), dtype)
    plan = _DIRECT_PLANS.get(key)
    if plan is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("grouped_gemm reads its pointer table back on the first call: call it once before capturing")
        ptrs = direct_pointers.cpu().tolist()
        strides = direct_strides.cpu().tolist()
        for g, st in enumerate(strides):
            if any(s[1] != 1 for s in st if sizes[g][0] and sizes[g][1] and sizes[g][2]):
                raise ValueError("grouped_gemm needs unit stride along K (A, B) and N (out)")

        def arr(ctype, values):
            return (ctype * groups)(*values)

        plan = (
            arr(ctypes.c_void_p, [p[0] for p in ptrs]), arr(ctypes.c_void_p, [p[1] for p in ptrs]),
            arr(ctypes.c_void_p, [p[2] for p in ptrs]),
            arr(ctypes.c_int64, [s[0] for s in sizes]), arr(ctypes.c_int64, [s[1] for s in sizes]),
            arr(ctypes.c_int64, [s[2] for s in sizes]),
            arr(ctypes.c_int64, [max(st[0][0], sz[2]) for st, sz in zip(strides, sizes)]),
            arr(ctypes.c_int64, [max(st[1][0], sz[2]) for st, sz in zip(strides, sizes)]),
            arr(ctypes.c_int64, [max(st[2][0], sz[1]) for st, sz in zip(strides, sizes)]),
        )
        if len(_DIRECT_PLANS) > 256:
            _DIRECT_PLANS.clear()
        _DIRECT_PLANS[key] = plan
    with torch.cuda.device(direct_pointers.device):
        _lib.call("hb200_grouped_gemm_f16_direct", *plan, groups, int(dtype is torch.bfloat16), _stream())
    return out_placeholder
