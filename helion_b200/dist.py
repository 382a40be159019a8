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


def shard_weight_k(packed: Tensor, scales: Tensor, world: int, rank: int) -> tuple[Tensor, Tensor]:
    """Slice a K-major NVFP4 weight ``[N, K/2]`` and its swizzled scales to the K range of ``rank`` (row parallelism:
    ``K / world`` must be a multiple of 64 so that whole scale column tiles move).  The scale buffer is ordered by
    (row tile, column tile), so a K range is one contiguous run of 512-byte tiles inside every row tile."""
    n, kb = packed.shape
    k = 2 * kb
    if k % world or (k // world) % 64:
        raise ValueError(f"K ({k}) must split into {world} shards that are multiples of 64")
    k_local = k // world
    col_tiles, local_tiles = -(-(k // 16) // 4), k_local // 64
    row_tiles = -(-n // 128)
    tiles = scales.reshape(-1).view(torch.uint8).reshape(row_tiles, col_tiles, 512)
    part = tiles[:, rank * local_tiles : (rank + 1) * local_tiles].reshape(-1)
    return packed[:, rank * (k_local // 2) : (rank + 1) * (k_local // 2)].contiguous(), part.contiguous().view(scales.dtype)


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


# ------------------------------------------------------------------ fused matmul + collective
@torch.library.custom_op("helion_b200::dense_matmul_out", mutates_args=("out",))
def _dense_matmul_op(a: Tensor, b_nk: Tensor, out: Tensor) -> None:
    from . import _lib
    from .ops import _require_cuda

    _require_cuda(a, b_nk, out)
    m, k = a.shape
    n = b_nk.shape[0]
    with torch.cuda.device(a.device):
        _lib.call("hb200_dense_matmul", a.data_ptr(), b_nk.data_ptr(), out.data_ptr(), m, n, k, a.stride(0),
                  b_nk.stride(0), out.stride(0), int(a.dtype is torch.bfloat16),
                  torch.cuda.current_stream(a.device).cuda_stream)


@_dense_matmul_op.register_fake
def _(a, b_nk, out):
    return None


def dense_matmul(a: Tensor, b: Tensor, out: Tensor | None = None) -> Tensor:
    """``a [M, K] @ b [K, N]`` in bf16 or fp16 on CTA pairs (256 x 256 tiles, fp32 accumulate); the one-GPU form of
    the two fused kernels below (``torch.ops.helion_b200.dense_matmul_out`` on the K-major operands).  ``b`` is taken
    K-major (``b.stride(0) == 1``, the weight stored ``[N, K]``); anything else is copied into that layout first."""
    if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype != a.dtype:
        raise TypeError("dense_matmul takes bfloat16 or float16 operands of one type")
    m, k = a.shape
    if b.shape[0] != k:
        raise ValueError(f"b {tuple(b.shape)} does not match a {tuple(a.shape)}")
    n = b.shape[1]
    b_nk = _k_major(b)
    if a.stride(1) != 1 or a.stride(0) % 8 or _misaligned(a):
        a = a.contiguous()
    if out is None:
        out = torch.empty(m, n, dtype=a.dtype, device=a.device)
    _dense_matmul_op(a, b_nk, out)
    return out


def _k_major(b: Tensor) -> Tensor:
    """``b [K, N]`` -> its ``[N, K]`` storage with unit stride along K (a view when ``b`` already is K-major)."""
    b_nk = b.t()
    if b_nk.stride(1) != 1 or b_nk.stride(0) % 8 or _misaligned(b_nk):
        b_nk = b_nk.contiguous()
    return b_nk


def _misaligned(t: Tensor) -> bool:
    """Whether ``t`` starts off a 16-byte boundary (from the storage offset: no data pointer is read, so that shapes
    trace under fake tensors; allocations themselves are at least 256-byte aligned)."""
    return (t.storage_offset() * t.element_size()) % 16 != 0


class FusedMatmulCollectives:
    """All-gather + matmul and matmul + reduce-scatter as single kernels over peer memory, the B200 forms of
    ``helion_all_gather_matmul`` (examples/distributed/all_gather_matmul.py:145-196) and
    ``helion_matmul_reduce_scatter`` (examples/distributed/matmul_reduce_scatter.py:118-140).

    The reference gathers with the copy engine on a second stream and lets a Triton matmul wait on progress
    flags; ``all_gather_matmul`` does the same around the tcgen05 GEMM (which takes the row tiles in arrival
    order), or, with ``gather="kernel"``, lets two warps of every CTA of the GEMM push the shard to the peers and
    count arrivals on the destination: one kernel, nothing else on the stream.  For the
    reduce-scatter the GEMM's epilogue stores every tile into the owner's receive buffer; a barrier kernel and
    a slot reduction (rank order, fp32) follow.  Symmetric buffers are allocated on first use per shape.
    """

    def __init__(self, device: torch.device, group=None):
        self._tp = TensorParallel(device, group)
        self.device, self.world, self.rank = device, self._tp.world, self._tp.rank
        self._gather = {}
        self._recv = {}

    def all_gather_matmul(self, a_shared: Tensor, b: Tensor, splits_per_rank: int = 1,
                          gather: str = "kernel") -> tuple[Tensor, Tensor]:
        """``a_shared [M / world, K]`` (this rank's rows), ``b [K, N]`` -> ``(gathered a [M, K], gathered a @ b)``.
        The gathered copy lives in a symmetric buffer that the next call with the same shape overwrites.

        ``gather="kernel"`` (default): one kernel does everything, two warps of every CTA of the GEMM push the shard to
        the peers.  ``gather="copy_engine"`` (the reference's structure): the shard is staged in symmetric memory, and
        on a second stream the copy engines pull every peer's shard chunk by chunk into this rank's gather buffer, a
        stream memory write after each chunk raising its progress counter; the GEMM kernel waits on the counters.
        Measured at M = 4096, N = 6656, K = 16384: 744-756 against 786-807 us on two GPUs, 777 against 822 us on four
        (one chunk per rank; more chunks cost more fences than they gain in overlap)."""
        from . import _lib
        from .ops import _require_cuda

        _require_cuda(a_shared, b)
        if a_shared.dtype not in (torch.bfloat16, torch.float16) or b.dtype != a_shared.dtype:
            raise TypeError("all_gather_matmul takes bfloat16 or float16 operands of one type")
        if gather not in ("copy_engine", "kernel"):
            raise ValueError(f"gather must be 'copy_engine' or 'kernel', got {gather!r}")
        rows, k = a_shared.shape
        if b.shape[0] != k:
            raise ValueError(f"b {tuple(b.shape)} does not match a_shared {tuple(a_shared.shape)}")
        n = b.shape[1]
        if rows % splits_per_rank or (rows // splits_per_rank) % 256:
            raise ValueError("rows per rank must split into chunks that are multiples of 256 rows")
        a_shared = a_shared.contiguous()
        b_nk = _k_major(b)
        world, rank = self.world, self.rank
        push = gather == "kernel" or world == 1
        key = (rows, k, a_shared.dtype, splits_per_rank, push)
        st = self._gather.get(key)
        if st is None:
            buf, buf_ptrs = self._tp._symmetric(world * rows * k, a_shared.dtype)
            if push:
                prog, prog_ptrs = self._tp._symmetric(max(64, world * splits_per_rank), torch.int32)
                st = dict(buf=buf.view(world * rows, k), buf_ptrs=buf_ptrs, prog=prog, prog_ptrs=prog_ptrs, calls=0)
            else:
                # only this rank writes its own counters (stream memory writes behind the copies): a plain tensor;
                # the shards are pulled from symmetric staging buffers, through views of every peer's buffer
                prog = torch.zeros(max(64, world * splits_per_rank), dtype=torch.uint32, device=self.device)
                prog_ptrs = (self._tp._ct.c_void_p * world)()
                prog_ptrs[rank] = prog.data_ptr()
                stage, _ = self._tp._symmetric(rows * k, a_shared.dtype)
                hdl = self._tp._handles[-1]
                st = dict(buf=buf.view(world * rows, k), buf_ptrs=buf_ptrs, prog=prog, prog_ptrs=prog_ptrs, calls=0,
                          stage=stage.view(rows, k), hdl=hdl,
                          peers=[hdl.get_buffer(r, (rows, k), a_shared.dtype, 0) for r in range(world)],
                          side=torch.cuda.Stream(device=self.device, priority=-1))
            self._tp._sync_all()  # the counters are zero everywhere before the first call
            self._gather[key] = st
        st["calls"] += 1
        calls = st["calls"]
        c = torch.empty(world * rows, n, dtype=a_shared.dtype, device=self.device)
        main = torch.cuda.current_stream(self.device)
        if not push:
            st["stage"].copy_(a_shared)
        # nobody overwrites a gather buffer that its owner's previous call still reads; every staged shard is complete
        self._tp.barrier()
        if not push:
            side, chunk = st["side"], rows // splits_per_rank
            side.wait_stream(main)
            with torch.cuda.stream(side):
                for step in range(1, world):
                    src = (rank - step) % world  # the order in which the GEMM takes the tiles
                    for ci in range(splits_per_rank):
                        dst_rows = st["buf"][src * rows + ci * chunk : src * rows + (ci + 1) * chunk]
                        dst_rows.copy_(st["peers"][src][ci * chunk : (ci + 1) * chunk])
                        st["hdl"].stream_write_value32(st["prog"], src * splits_per_rank + ci, calls)
                st["buf"][rank * rows : (rank + 1) * rows].copy_(st["stage"])  # the GEMM reads these rows from the shard
        with torch.cuda.device(self.device):
            _lib.call("hb200_ag_matmul", (st["stage"] if not push else a_shared).data_ptr(), st["buf_ptrs"], st["prog_ptrs"],
                      b_nk.data_ptr(), c.data_ptr(), rows, n, k, b_nk.stride(0), c.stride(0), world, rank,
                      splits_per_rank, calls, int(push), int(a_shared.dtype is torch.bfloat16), main.cuda_stream)
        if not push:
            main.wait_stream(side)
        return st["buf"], c

    def matmul_reduce_scatter(self, a: Tensor, b: Tensor) -> Tensor:
        """``a [M, K_local]``, ``b [K_local, N]`` (this rank's K shard) -> rows ``[rank M / world, +M / world)`` of the
        sum over ranks of ``a @ b``.  Every partial product is rounded to the operand type before it travels, and
        the owner adds the partials in rank order in fp32, as the reference kernel does."""
        from . import _lib
        from .ops import _require_cuda

        _require_cuda(a, b)
        if a.dtype not in (torch.bfloat16, torch.float16) or b.dtype != a.dtype:
            raise TypeError("matmul_reduce_scatter takes bfloat16 or float16 operands of one type")
        m, k = a.shape
        if b.shape[0] != k:
            raise ValueError(f"b {tuple(b.shape)} does not match a {tuple(a.shape)}")
        n = b.shape[1]
        if m % (256 * self.world):
            raise ValueError("M must be a multiple of 256 rows per rank")
        rows = m // self.world
        if a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16:
            a = a.contiguous()
        b_nk = _k_major(b)
        key = (m, n, a.dtype)
        st = self._recv.get(key)
        if st is None:
            ring = [self._tp._symmetric(m * n, a.dtype) for _ in range(2)]
            self._tp._sync_all()
            st = self._recv[key] = dict(ring=ring, turn=0)
        slots, slot_ptrs = st["ring"][st["turn"]]
        st["turn"] ^= 1  # two buffers alternate: a peer may push the next step while this rank still reduces
        out = torch.empty(rows, n, dtype=a.dtype, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        is_bf16 = int(a.dtype is torch.bfloat16)
        with torch.cuda.device(self.device):
            _lib.call("hb200_matmul_rs", a.data_ptr(), b_nk.data_ptr(), slot_ptrs, m, n, k, a.stride(0), b_nk.stride(0),
                      self.world, self.rank, is_bf16, stream)
            self._tp.barrier()
            _lib.call("hb200_reduce_slots", slots.data_ptr(), out.data_ptr(), self.world, rows, n, out.stride(0), is_bf16,
                      stream)
        return out


# ------------------------------------------------------------------ fused column parallelism
class GatheredOutput:
    """A ring of ``[rows, n_total]`` output buffers in symmetric memory, mapped into every rank.

    Two buffers alternate so that a rank may still read the result of one step while its peers already
    push the next one; ``hb200_peer_barrier`` after every step is the only synchronisation needed.
    """

    def __init__(self, locals_: list[Tensor], ptr_arrays: list):
        self.locals = locals_
        self.ptr_arrays = ptr_arrays
        self.turn = 0

    def next(self):
        i = self.turn
        self.turn = (i + 1) % len(self.locals)
        return self.locals[i], self.ptr_arrays[i]


class TensorParallel:
    """Column-parallel GEMV / GEMM whose kernels store their output slice straight into every rank's buffer
    over NVLink, followed by a barrier kernel: no collective call and no host involvement per step, so a whole
    step can be captured in a CUDA graph.  With one rank (or no process group) it degenerates to the plain
    kernels writing a local buffer.

    The symmetric allocation and the peer mapping come from ``torch.distributed._symmetric_memory``
    (the allocator the reference's distributed examples use, examples/distributed/all_gather_matmul.py:90-130).
    """

    def __init__(self, device: torch.device, group=None):
        import ctypes

        self._ct = ctypes
        self.device = device
        self.group = group
        active = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if active else 1
        self.rank = dist.get_rank(group) if active else 0
        self._handles = []  # keeps the rendezvous handles (and so the peer mappings) alive
        flags = self._symmetric(64, torch.int32)
        self.flag_ptrs = flags[1]
        self._flags = flags[0]
        self._epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self._sync_all()

    # -- allocation
    def _symmetric(self, numel: int, dtype: torch.dtype):
        """Zeroed symmetric tensor of ``numel`` elements -> (local tensor, ctypes array of per-rank pointers)."""
        ct = self._ct
        if self.world == 1:
            t = torch.zeros(numel, dtype=dtype, device=self.device)
            ptrs = [t.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm_mem

            t = symm_mem.empty(numel, dtype=dtype, device=self.device)
            t.zero_()
            g = self.group if self.group is not None else dist.group.WORLD
            hdl = symm_mem.rendezvous(t, g.group_name)
            self._handles.append(hdl)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
        arr = (ct.c_void_p * len(ptrs))(*ptrs)
        return t, arr

    def _sync_all(self):
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def gathered_output(self, rows: int, n_total: int, dtype: torch.dtype = torch.bfloat16, buffers: int = 2) -> GatheredOutput:
        locals_, arrays = [], []
        for _ in range(buffers):
            t, arr = self._symmetric(rows * n_total, dtype)
            locals_.append(t.view(rows, n_total))
            arrays.append(arr)
        self._sync_all()  # every rank's zero-fill is done before anybody pushes
        return GatheredOutput(locals_, arrays)

    # -- steps
    def barrier(self) -> None:
        from . import _lib

        _lib.call("hb200_peer_barrier", self.flag_ptrs, self.world, self.rank, self._epoch.data_ptr(),
                  torch.cuda.current_stream(self.device).cuda_stream)

    def gemv(self, weight_local: Tensor, scale_local: Tensor, x: Tensor, out: GatheredOutput, alpha: float = 1.0,
             barrier: bool = True) -> Tensor:
        """``x [M, K]`` bf16 (replicated, 1 <= M <= 32) against this rank's weight rows; every rank ends up with
        the full ``[M, N]`` in its buffer (returned)."""
        from . import _lib

        m, k = x.shape
        n_local = weight_local.shape[0]
        buf, ptrs = out.next()
        if buf.shape[0] < m or buf.shape[1] != n_local * self.world or buf.dtype != torch.bfloat16:
            raise ValueError("output ring does not match [M, N_local * world] bf16")
        if weight_local.shape[1] * 2 != k:
            raise ValueError("weight and activation disagree on K")
        from . import ops

        stream = torch.cuda.current_stream(self.device).cuda_stream
        # With peers, a single row stays on the SIMT kernel: the barrier kernel between two GEMVs breaks the
        # dependent-launch chain that hides the tensor-core path's activation expansion, and the slices are small
        # (measured on two GPUs, decode layer: 112 us against 142 us).
        if (m >= 2 or self.world == 1) and ops._gemv_path("auto", n_local, k, m) == "tc":
            need = _lib.load().hb200_nvfp4_gemv_tc_workspace_bytes(n_local, k, m, 4)
            ws = ops.tc_workspace(self.device, need)
            _lib.call("hb200_nvfp4_gemv_bf16in_tc", weight_local.data_ptr(), x.data_ptr(), scale_local.data_ptr(), ptrs,
                      self.world, n_local, k, m, buf.shape[1], self.rank * n_local, float(alpha), ws.data_ptr(),
                      ws.numel(), stream)
        else:
            _lib.call("hb200_nvfp4_gemv_bf16in_tp", weight_local.data_ptr(), x.data_ptr(), scale_local.data_ptr(), ptrs,
                      self.world, n_local, k, m, buf.shape[1], self.rank * n_local, float(alpha), stream)
        if barrier:
            self.barrier()
        return buf[:m]

    def scatter_buffers(self, rows: int, n_total: int, buffers: int = 2) -> GatheredOutput:
        """Ring of fp32 ``[world, rows, n_total / world]`` partial-sum buffers for :meth:`gemv_row_parallel`."""
        if n_total % self.world:
            raise ValueError(f"{n_total} output columns do not split evenly over {self.world} ranks")
        locals_, arrays = [], []
        for _ in range(buffers):
            t, arr = self._symmetric(self.world * rows * (n_total // self.world), torch.float32)
            locals_.append(t.view(self.world, rows, n_total // self.world))
            arrays.append(arr)
        self._sync_all()
        return GatheredOutput(locals_, arrays)

    def gemv_row_parallel(self, weight_kshard: Tensor, scale_kshard: Tensor, x_kshard: Tensor, partials: GatheredOutput,
                          alpha: float = 1.0) -> Tensor:
        """Row-parallel projection with a fused reduce-scatter: this rank holds the weight's K shard ``[N, K/world/2]``
        (see :func:`shard_weight_k`) and ``x_kshard [M, K/world]`` (1 <= M <= 32); every rank ends up with its own
        ``[M, N/world]`` column slice of ``x @ W.T`` (bf16): partial sums go straight from the kernel into the owning
        rank's buffer, a barrier kernel, then the owner adds them in rank order."""
        from . import _lib

        m, k_local = x_kshard.shape
        n = weight_kshard.shape[0]
        buf, ptrs = partials.next()
        if buf.shape != (self.world, m, n // self.world) or buf.dtype is not torch.float32:
            raise ValueError("partial-sum ring does not match [world, M, N / world] fp32")
        if weight_kshard.shape[1] * 2 != k_local:
            raise ValueError("weight shard and activation shard disagree on K")
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            _lib.call("hb200_nvfp4_gemv_bf16in_rs", weight_kshard.data_ptr(), x_kshard.data_ptr(), scale_kshard.data_ptr(),
                      ptrs, self.world, self.rank, n, k_local, m, float(alpha), stream)
        self.barrier()
        out = torch.empty(m, n // self.world, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            _lib.call("hb200_tp_reduce_partials", buf.data_ptr(), out.data_ptr(), self.world, m, n // self.world,
                      out.stride(0), stream)
        return out

    def matmul(self, a_packed: Tensor, scale_a: Tensor, b_local: Tensor, scale_b_local: Tensor, out: GatheredOutput,
               alpha: float = 1.0, barrier: bool = True) -> Tensor:
        """Block-scaled GEMM, B's rows ``[N_local, K/2]`` (output columns) owned by this rank, A replicated."""
        from . import _lib

        m, kb = a_packed.shape
        n_local = b_local.shape[0]
        buf, ptrs = out.next()
        if buf.shape[0] != m or buf.shape[1] != n_local * self.world:
            raise ValueError("output ring does not match [M, N_local * world]")
        if buf.dtype not in (torch.bfloat16, torch.float16):
            raise TypeError("fused column-parallel matmul writes bf16 or fp16")
        _lib.call("hb200_nvfp4_scaled_matmul_tp", a_packed.data_ptr(), b_local.data_ptr(), scale_a.data_ptr(),
                  scale_b_local.data_ptr(), ptrs, self.world, self.rank, m, n_local, 2 * kb, buf.shape[1],
                  self.rank * n_local, float(alpha), 0 if buf.dtype == torch.bfloat16 else 1,
                  torch.cuda.current_stream(self.device).cuda_stream)
        if barrier:
            self.barrier()
        return buf


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


Router = Callable[[Tensor, int], tuple[Tensor, Tensor]]       # (logits, top_k) -> (weights [T, k], experts [T, k])
Combine = Callable[[Tensor, Tensor, Tensor, int], Tensor]      # (rows [P, H], row_of_pair [P], weights [P], T) -> [T, H]


def combine_rows(back: Tensor, row_of_pair: Tensor, pair_weight: Tensor, tokens: int) -> Tensor:
    """``out[t] = bf16(sum_s w[t*k+s] * back[row_of_pair[t*k+s]])`` in fp32 and slot order (``hb200_moe_combine``)."""
    from . import _lib

    top_k = row_of_pair.numel() // tokens
    hidden = back.shape[1]
    if not back.is_cuda or back.dtype is not torch.bfloat16 or hidden % 8:
        raise ValueError("combine_rows wants CUDA bfloat16 rows with hidden % 8 == 0")
    back = back.contiguous()
    out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=back.device)
    with torch.cuda.device(back.device):
        _lib.call("hb200_moe_combine", back.data_ptr(), back.stride(0), row_of_pair.to(torch.int32).data_ptr(),
                  pair_weight.to(torch.float32).contiguous().data_ptr(), out.data_ptr(), tokens, top_k, hidden,
                  torch.cuda.current_stream(back.device).cuda_stream)
    return out


def expert_parallel_moe(x: Tensor, router_logits: Tensor, top_k: int, num_experts: int, expert_fn: ExpertFn,
                        group=None, *, router: Router | None = None, combine: Combine | None = None) -> Tensor:
    """MoE layer over expert-parallel ranks with the process group's all-to-all as the data plane.
    ``x [T_local, H]`` are this rank's tokens; ``expert_fn`` applies this rank's experts to the rows it receives
    (no routing weight).  Returns bf16 ``[T_local, H]``.  ``router`` and ``combine`` default to the CUDA kernels
    (``moe.route_top_k``, :func:`combine_rows`); host-logic tests inject tensor-code stand-ins."""
    if router is None:
        from .moe import route_top_k as router
    if combine is None:
        combine = combine_rows
    weights, experts = router(router_logits, top_k)
    plan = plan_dispatch(experts, num_experts, group)
    token_of_pair = plan.order // top_k
    rows = exchange_rows(x[token_of_pair], plan.send_counts, plan.recv_counts, group)
    o = expert_fn(rows, plan.local_expert)
    back = exchange_rows(o, plan.recv_counts, plan.send_counts, group)
    # `back` is in sorted-pair order: row p belongs to pair order[p]
    pairs = plan.order.numel()
    row_of_pair = torch.empty(pairs, dtype=torch.int32, device=x.device)
    row_of_pair[plan.order] = torch.arange(pairs, dtype=torch.int32, device=x.device)
    return combine(back, row_of_pair, weights.reshape(-1), x.shape[0])


def make_nvfp4_expert_fn(w_gate_up, w_down) -> ExpertFn:
    """``expert_fn`` running this rank's NVFP4 experts (``GroupedNvfp4Weight`` bundles of the local experts)
    through the grouped tcgen05 GEMMs."""
    from . import moe as M

    def fn(rows: Tensor, local_expert: Tensor) -> Tensor:
        if rows.shape[0] == 0:
            return rows.new_empty(0, w_down.n)
        sched = M.build_schedule(local_expert.reshape(-1, 1), w_gate_up.experts)
        a1, sf1, g1 = M._quantize_rows(rows.contiguous(), w_gate_up.k, sched, 1, None, False, gather=True)
        if w_gate_up.gate_up_interleaved:
            y, row_amax = M.grouped_matmul_silu(a1, sf1, w_gate_up, sched, g1)
            a2, sf2, g2 = M._quantize_rows_amax(y, row_amax, w_down.k, sched, None)
        else:
            h1 = M.grouped_matmul(a1, sf1, w_gate_up, sched, g1)
            a2, sf2, g2 = M._quantize_rows(h1, w_down.k, sched, 1, None, True, gather=False)
        o = M.grouped_matmul(a2, sf2, w_down, sched, g2)
        return o[sched.row_of_pair.long()]

    return fn


# ------------------------------------------------------------------ expert parallelism over peer memory
class ExpertParallel:
    """NVFP4 MoE layer over expert-parallel ranks whose exchange is done by this library's own kernels over peer
    memory (``csrc/moe_ep.cu``): tokens travel as NVFP4 rows (codes, block scales, one global scale per token: about
    2.3 KB per (token, expert) pair at hidden 4096 instead of 8 KB in bf16), every expert rank returns ONE
    routing-weighted, pre-reduced 2-byte row per (token, rank), receive areas have a capacity that follows from the
    shapes, and nothing is read on the host: a step is a fixed sequence of launches and two barrier kernels.

    ``tokens`` is the number of tokens per rank (fixed at construction: the symmetric buffer is sized from it).
    Rank r owns experts ``[r E / W, (r + 1) E / W)``; weights are :class:`moe.GroupedNvfp4Weight` bundles of the local
    experts, the gate/up bundle interleaved with :func:`moe.interleave_gate_up`.

    Numerics: every (token, slot) pair is computed exactly as on one GPU; the sum over a token's slots is taken per
    expert rank first (fp32, slot order; it travels as fp16 values with a power-of-two row factor, 11 significant
    bits) and over ranks second, so results agree with the one-GPU layer up to a last-place flip of the bf16
    result, not bit for bit.
    """

    def __init__(self, device: torch.device, tokens: int, hidden: int, top_k: int, num_experts: int, group=None,
                 *, _emulate: tuple[int, int, list[Tensor]] | None = None):
        import ctypes

        from . import _lib

        self.device = device
        self.tokens, self.hidden, self.top_k, self.experts = tokens, hidden, top_k, num_experts
        if _emulate is not None:
            # several "ranks" on one GPU for tests: buffers are ordinary tensors, phases are run rank after rank
            # by the caller and no barrier kernel is launched (nothing may wait for a launch that has not started)
            self.world, self.rank, buffers = _emulate
            self._tp = None
        else:
            self._tp = TensorParallel(device, group)
            self.world, self.rank = self._tp.world, self._tp.rank
        lib = _lib.load()
        nbytes = int(lib.hb200_ep_buffer_bytes(self.world, tokens, hidden, top_k, num_experts))
        if nbytes < 0:
            _lib.check(nbytes, "hb200_ep_buffer_bytes")
        self.slots = int(lib.hb200_ep_slots(self.world, tokens, hidden, top_k, num_experts))
        self.e_local = num_experts // self.world
        if _emulate is not None:
            if any(b.numel() < nbytes for b in buffers):
                raise ValueError(f"emulated exchange buffers must hold {nbytes} bytes")
            self._buf = buffers[self.rank]
            self.bases = (ctypes.c_void_p * self.world)(*[b.data_ptr() for b in buffers])
        else:
            self._buf, self.bases = self._tp._symmetric(nbytes, torch.uint8)
            self._tp._sync_all()
        self._state = None

    @staticmethod
    def buffer_bytes(world: int, tokens: int, hidden: int, top_k: int, num_experts: int) -> int:
        from . import _lib

        return int(_lib.load().hb200_ep_buffer_bytes(world, tokens, hidden, top_k, num_experts))

    def _shape_args(self):
        return (self.world, self.rank, self.tokens, self.hidden, self.top_k, self.experts)

    def _barrier(self):
        if self._tp is not None:
            self._tp.barrier()

    # -- phases (a rank's phases run in this order; ranks meet at the barriers)
    def dispatch(self, x: Tensor, router_logits: Tensor) -> None:
        """Route, quantise every token once, sort the (token, slot) pairs by expert and push them to their ranks."""
        from . import _lib
        from . import moe as M
        from . import ops

        if x.shape != (self.tokens, self.hidden) or x.dtype is not torch.bfloat16 or not x.is_contiguous():
            raise ValueError(f"x must be a contiguous bfloat16 [{self.tokens}, {self.hidden}] tensor")
        weights, experts = M.route_top_k(router_logits, self.top_k)
        codes_t, scales_t, g_t = ops.nvfp4_quantize(x)
        flat = experts.reshape(-1)
        pairs = flat.numel()
        dev = x.device
        sorted_pairs = torch.empty(pairs, dtype=torch.int32, device=dev)
        counts = torch.empty(self.experts, dtype=torch.int32, device=dev)
        scratch = torch.empty(max(1, -(-pairs // 1024)) * self.experts, dtype=torch.int32, device=dev)
        route_local = torch.empty(pairs, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        with torch.cuda.device(dev):
            _lib.call("hb200_moe_sort_pairs", flat.data_ptr(), 1, pairs, self.experts, sorted_pairs.data_ptr(),
                      counts.data_ptr(), scratch.data_ptr(), stream)
            _lib.call("hb200_ep_dispatch", codes_t.data_ptr(), scales_t.data_ptr(), g_t.data_ptr(),
                      weights.data_ptr(), flat.data_ptr(), sorted_pairs.data_ptr(), counts.data_ptr(),
                      route_local.data_ptr(), self.bases, *self._shape_args(), stream)
        self._state = route_local

    def run_experts(self, w_gate_up, w_down) -> None:
        """Sort what arrived by expert, run the two grouped GEMMs (SiLU-mul between them) and push one pre-reduced
        row per (source, token) back."""
        from . import _lib
        from . import moe as M
        from .layouts import ceil_div
        from .layouts import swizzled_scale_numel

        if w_gate_up.experts != self.e_local or w_down.experts != self.e_local:
            raise ValueError(f"this rank owns {self.e_local} experts")
        if w_gate_up.k != self.hidden or w_down.n != self.hidden or w_down.k != w_gate_up.n // 2:
            raise ValueError("expert weight shapes do not match the activations")
        dev = self.device
        slots, h, inter = self.slots, self.hidden, w_down.k
        stream = torch.cuda.current_stream(dev).cuda_stream
        i32 = dict(dtype=torch.int32, device=dev)
        expert_of_slot = torch.empty(slots, **i32)
        sorted_slots = torch.empty(slots, **i32)
        counts = torch.empty(self.e_local, **i32)
        scratch = torch.empty(max(1, ceil_div(slots, 1024)) * self.e_local, **i32)
        max_tiles = ceil_div(slots, 128) + self.e_local
        rows = max_tiles * 128
        tile_info = torch.empty(max_tiles, 2, **i32)
        padded_offsets = torch.empty(self.e_local + 1, **i32)
        row_of_sorted = torch.empty(slots, **i32)
        row_of_slot = torch.full((slots,), -1, **i32)
        a1 = torch.empty(rows, h // 2, dtype=torch.uint8, device=dev)
        sf1 = torch.empty(swizzled_scale_numel(rows, h // 16), dtype=torch.uint8, device=dev)
        g1 = torch.zeros(rows, dtype=torch.float32, device=dev)
        w_row = torch.zeros(rows, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.call("hb200_ep_collect", self._buf.data_ptr(), expert_of_slot.data_ptr(), *self._shape_args(), stream)
            _lib.call("hb200_moe_sort_pairs", expert_of_slot.data_ptr(), 0, slots, self.e_local, sorted_slots.data_ptr(),
                      counts.data_ptr(), scratch.data_ptr(), stream)
            _lib.call("hb200_moe_build_schedule", counts.data_ptr(), self.e_local, sorted_slots.data_ptr(), slots,
                      padded_offsets.data_ptr(), tile_info.data_ptr(), max_tiles, row_of_sorted.data_ptr(),
                      row_of_slot.data_ptr(), stream)
            _lib.call("hb200_ep_gather", self._buf.data_ptr(), sorted_slots.data_ptr(), row_of_sorted.data_ptr(),
                      a1.data_ptr(), sf1.data_ptr(), g1.data_ptr(), w_row.data_ptr(), *self._shape_args(), stream)
        sched = M.MoeSchedule(max_tiles, tile_info, padded_offsets, sorted_slots, row_of_sorted, row_of_slot, 128)
        if w_gate_up.gate_up_interleaved:
            y, row_amax = M.grouped_matmul_silu(a1, sf1, w_gate_up, sched, g1)
            a2, sf2, g2 = M._quantize_rows_amax(y, row_amax, inter, sched, None)
        else:
            h1 = M.grouped_matmul(a1, sf1, w_gate_up, sched, g1)
            a2, sf2, g2 = M._quantize_rows(h1, inter, sched, 1, None, True, gather=False)
        o = M.grouped_matmul(a2, sf2, w_down, sched, g2)
        with torch.cuda.device(dev):
            _lib.call("hb200_ep_return", o.data_ptr(), o.stride(0), row_of_slot.data_ptr(), w_row.data_ptr(), self.bases,
                      *self._shape_args(), stream)

    def combine(self) -> Tensor:
        """Add, per token, the rows the expert ranks returned (rank order, fp32); bf16 ``[tokens, hidden]``."""
        from . import _lib

        if self._state is None:
            raise RuntimeError("combine() follows dispatch() and run_experts()")
        out = torch.empty(self.tokens, self.hidden, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            _lib.call("hb200_ep_combine", self._buf.data_ptr(), self._state.data_ptr(), out.data_ptr(),
                      *self._shape_args(), torch.cuda.current_stream(self.device).cuda_stream)
        self._state = None
        return out

    def moe(self, x: Tensor, router_logits: Tensor, w_gate_up, w_down) -> Tensor:
        """One MoE layer step: ``x [tokens, hidden]`` bf16 and ``router_logits [tokens, E]`` of this rank's tokens."""
        self.dispatch(x, router_logits)
        self._barrier()  # every rank's rows, counts and tables have arrived
        self.run_experts(w_gate_up, w_down)
        self._barrier()  # every rank's returned rows have arrived
        return self.combine()

    def phase_times(self, x: Tensor, router_logits: Tensor, w_gate_up, w_down) -> dict:
        """Microseconds of every phase of one step on this rank (CUDA events, a device synchronisation and a host
        barrier between phases, so the figures do not add up to the pipelined step time)."""
        def timed(fn):
            if self._tp is not None:
                self._tp._sync_all()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            r = fn()
            b.record()
            torch.cuda.synchronize(self.device)
            return a.elapsed_time(b) * 1e3, r

        out = {}
        out["dispatch"], _ = timed(lambda: self.dispatch(x, router_logits))
        out["barrier_1"], _ = timed(self._barrier)
        out["experts_and_return"], _ = timed(lambda: self.run_experts(w_gate_up, w_down))
        out["barrier_2"], _ = timed(self._barrier)
        out["combine"], _ = timed(self.combine)
        return out
