"""Column-parallel forms whose kernels store their output slice into every rank's buffer.

On one GPU the "peers" are further buffers on the same device: each rank's call runs to completion before
the next one starts, so nothing waits on anything.  The barrier kernel is only ever launched with one rank
here; the two-rank run over real peer mappings needs two GPUs and is skipped otherwise.
"""

from __future__ import annotations

import ctypes
import os
import socket

import pytest
import torch

import helion_b200 as hb
from helion_b200 import _lib
from helion_b200 import dist as D
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def device_status_ok():
    torch.cuda.synchronize()
    return _lib.load().hb200_device_status(1) == 0


def ptr_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def random_weight(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
    scales = O.swizzle_scales((torch.rand(n, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
    return codes.to(DEV), scales.to(DEV)


@pytest.mark.parametrize("batch", [1, 4, 17])
@pytest.mark.parametrize("world", [2, 4])
def test_gemv_slices_land_in_every_buffer(batch, world):
    n, k = 1024, 2048
    codes, scales = random_weight(n, k, 7 + batch)
    x = torch.randn(batch, k, generator=torch.Generator().manual_seed(batch)).to(torch.bfloat16).to(DEV)
    full = hb.nvfp4_gemv_bf16in_batched(codes, x, scales, 0.5) if batch > 1 else \
        hb.nvfp4_gemv_bf16in(codes, x.reshape(-1), scales, 0.5).reshape(1, -1)
    bufs = [torch.full((batch, n), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    ptrs = ptr_array(bufs)
    stream = torch.cuda.current_stream().cuda_stream
    for rank in range(world):
        w_r, s_r = D.shard_weight_rows(codes, scales, world, rank)
        n_local = n // world
        _lib.call("hb200_nvfp4_gemv_bf16in_tp", w_r.data_ptr(), x.data_ptr(), s_r.data_ptr(), ptrs, world, n_local, k,
                  batch, n, rank * n_local, 0.5, stream)
    assert device_status_ok()
    for b in bufs:
        # a slice is computed with the split-K plan of its own size, so allow the last bf16 place
        torch.testing.assert_close(b.float(), full.float(), rtol=1e-2, atol=1e-2 * float(full.float().abs().mean()))
    for b in bufs[1:]:
        assert torch.equal(b, bufs[0])
    # the slices themselves are bit-identical to the plain entry point on the same shard
    w0, s0 = D.shard_weight_rows(codes, scales, world, 1)
    y0 = hb.nvfp4_gemv_bf16in_batched(w0, x, s0, 0.5) if batch > 1 else \
        hb.nvfp4_gemv_bf16in(w0, x.reshape(-1), s0, 0.5).reshape(1, -1)
    assert torch.equal(bufs[0][:, n // world : 2 * (n // world)], y0)


@pytest.mark.parametrize("batch,world", [(2, 2), (8, 4), (1, 2)])
def test_tensor_core_gemv_slices_land_in_every_buffer(batch, world):
    n, k = 2048, 4096
    codes, scales = random_weight(n, k, 31 + batch)
    x = torch.randn(batch, k, generator=torch.Generator().manual_seed(batch)).to(torch.bfloat16).to(DEV)
    bufs = [torch.full((batch, n), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    ptrs = ptr_array(bufs)
    stream = torch.cuda.current_stream().cuda_stream
    n_local = n // world
    need = _lib.load().hb200_nvfp4_gemv_tc_workspace_bytes(n_local, k, batch, 4)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    for rank in range(world):
        w_r, s_r = D.shard_weight_rows(codes, scales, world, rank)
        _lib.call("hb200_nvfp4_gemv_bf16in_tc", w_r.data_ptr(), x.data_ptr(), s_r.data_ptr(), ptrs, world, n_local, k,
                  batch, n, rank * n_local, 0.5, ws.data_ptr(), need, stream)
    assert device_status_ok()
    for b in bufs[1:]:
        assert torch.equal(b, bufs[0])
    want = torch.cat([hb.nvfp4_gemv_bf16in_batched(*D.shard_weight_rows(codes, scales, world, r)[:1], x,
                                                   D.shard_weight_rows(codes, scales, world, r)[1], 0.5, path="tc")
                      for r in range(world)], dim=1)
    assert torch.equal(bufs[0], want)


@pytest.mark.parametrize("m,n,k,world", [(256, 1024, 512, 2), (512, 1024, 1024, 4), (300, 1024, 256, 2), (256, 1040, 256, 2)])
def test_matmul_slices_land_in_every_buffer(m, n, k, world):
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, generator=g).to(DEV)
    sa = O.swizzle_scales((torch.rand(m, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn)).to(DEV)
    n_local = n // world
    shards = [random_weight(n_local, k, 100 * r + m) for r in range(world)]
    bufs = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    ptrs = ptr_array(bufs)
    stream = torch.cuda.current_stream().cuda_stream
    for rank, (b, sb) in enumerate(shards):
        _lib.call("hb200_nvfp4_scaled_matmul_tp", a.data_ptr(), b.data_ptr(), sa.data_ptr(), sb.data_ptr(), ptrs, world,
                  rank, m, n_local, k, n, rank * n_local, 0.25, 0, stream)
    assert device_status_ok()
    want = torch.cat([hb.nvfp4_scaled_matmul(a, b.t(), sa, sb, alpha=0.25) for b, sb in shards], dim=1)
    for buf in bufs:
        assert torch.equal(buf, want)


@pytest.mark.parametrize("batch,world", [(1, 2), (4, 4), (17, 2), (1, 8)])
def test_row_parallel_partials_reduce_to_the_full_product(batch, world):
    """K-sharded projection with the fused reduce-scatter, ranks emulated one after the other on one GPU: every
    rank's kernel stores its fp32 partials into the owners' buffers, then each owner adds them in rank order."""
    n, k = 1024, 4096
    codes, scales = random_weight(n, k, 17 + batch)
    x = torch.randn(batch, k, generator=torch.Generator().manual_seed(batch)).to(torch.bfloat16).to(DEV)
    full = hb.nvfp4_gemv_bf16in_batched(codes, x, scales, 0.5, path="simt" if batch == 1 else "mma")
    cols = n // world
    bufs = [torch.full((world, batch, cols), float("nan"), dtype=torch.float32, device=DEV) for _ in range(world)]
    ptrs = ptr_array(bufs)
    stream = torch.cuda.current_stream().cuda_stream
    k_local = k // world
    for rank in range(world):
        w_r, s_r = D.shard_weight_k(codes, scales, world, rank)
        x_r = x[:, rank * k_local : (rank + 1) * k_local].contiguous()
        _lib.call("hb200_nvfp4_gemv_bf16in_rs", w_r.data_ptr(), x_r.data_ptr(), s_r.data_ptr(), ptrs, world, rank, n,
                  k_local, batch, 0.5, stream)
    assert device_status_ok()
    for rank in range(world):
        assert torch.isfinite(bufs[rank]).all()  # every slot was written by its source rank
        out = torch.empty(batch, cols, dtype=torch.bfloat16, device=DEV)
        _lib.call("hb200_tp_reduce_partials", bufs[rank].data_ptr(), out.data_ptr(), world, batch, cols, cols, stream)
        want = full[:, rank * cols : (rank + 1) * cols]
        # the K range is summed in `world` pieces instead of one: the last bf16 place may move
        torch.testing.assert_close(out.float(), want.float(), rtol=1e-2, atol=1e-2 * float(full.float().abs().mean()))
        # and the owner's sum is exactly the fp32 sum of the partials in rank order
        acc = torch.zeros(batch, cols, device=DEV)
        for r in range(world):
            acc += bufs[rank][r]
        assert torch.equal(out, acc.to(torch.bfloat16))


def test_shard_weight_k_moves_whole_scale_tiles():
    n, k = 256, 512
    g = torch.Generator().manual_seed(2)
    packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
    logical = (torch.rand(n, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn)
    scales = O.swizzle_scales(logical)
    for r in range(4):
        p, s = D.shard_weight_k(packed, scales, 4, r)
        assert torch.equal(p, packed[:, r * 64 : (r + 1) * 64])
        assert torch.equal(s.view(torch.uint8), O.swizzle_scales(logical[:, r * 8 : (r + 1) * 8]).view(torch.uint8))
    with pytest.raises(ValueError, match="multiples of 64"):
        D.shard_weight_k(packed, scales, 16, 0)


def test_matmul_tp_rejects_what_the_pair_kernel_cannot_take():
    a = torch.zeros(128, 64, dtype=torch.uint8, device=DEV)
    s = torch.zeros(128 * 8, dtype=torch.uint8, device=DEV)
    out = torch.zeros(128, 256, dtype=torch.bfloat16, device=DEV)
    rc = _lib.load().hb200_nvfp4_scaled_matmul_tp(a.data_ptr(), a.data_ptr(), s.data_ptr(), s.data_ptr(), ptr_array([out]),
                                                  1, 0, 128, 128, 128, 256, 0, 1.0, 0, None)
    assert rc == _lib.HB200_ERR_UNSUPPORTED
    rc = _lib.load().hb200_nvfp4_scaled_matmul_tp(a.data_ptr(), a.data_ptr(), s.data_ptr(), s.data_ptr(), ptr_array([out]),
                                                  1, 3, 128, 128, 128, 256, 0, 1.0, 0, None)
    assert rc == _lib.HB200_ERR_INVALID_ARGUMENT


def test_single_rank_context_and_barrier():
    tp = D.TensorParallel(torch.device(DEV))
    assert tp.world == 1
    n, k, m = 512, 1024, 256
    codes, scales = random_weight(n, k, 3)
    x = torch.randn(4, k, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    ring = tp.gathered_output(4, n)
    for _ in range(3):
        y = tp.gemv(codes, scales, x, ring, 1.0)
        assert torch.equal(y, hb.nvfp4_gemv_bf16in_batched(codes, x, scales, 1.0))
    g = torch.Generator().manual_seed(5)
    a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, generator=g).to(DEV)
    sa = O.swizzle_scales((torch.rand(m, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn)).to(DEV)
    ring2 = tp.gathered_output(m, n)
    y = tp.matmul(a, sa, codes, scales, ring2, 1.0)
    assert torch.equal(y, hb.nvfp4_scaled_matmul(a, codes.t(), sa, scales))
    assert device_status_ok()
    assert int(tp._epoch.item()) == 4  # one barrier per step


def _two_rank_worker(rank: int, world: int, port: int, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        tp = D.TensorParallel(dev)
        n, k, m = 2048, 1024, 512
        g = torch.Generator().manual_seed(11)
        codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
        scales = O.swizzle_scales((torch.rand(n, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
        a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, generator=g).to(dev)
        sa = O.swizzle_scales((torch.rand(m, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn)).to(dev)
        x = torch.randn(8, k, generator=g).to(torch.bfloat16).to(dev)
        w_r, s_r = D.shard_weight_rows(codes.to(dev), scales.to(dev), world, rank)
        ring_v, ring_m = tp.gathered_output(8, n), tp.gathered_output(m, n)
        ok = True
        for _ in range(4):
            yv = tp.gemv(w_r, s_r, x, ring_v, 1.0)
            ok &= bool(torch.equal(yv, D.column_parallel_gemv(w_r, s_r, x, 1.0)))
            ym = tp.matmul(a, sa, w_r, s_r, ring_m, 1.0)
            ok &= bool(torch.equal(ym, D.column_parallel_matmul(a, sa, w_r, s_r)))
        # row-parallel projection with the fused reduce-scatter against the one-GPU product
        full = hb.nvfp4_gemv_bf16in_batched(codes.to(dev), x, scales.to(dev), 1.0, path="mma")
        w_k, s_k = D.shard_weight_k(codes.to(dev), scales.to(dev), world, rank)
        x_k = x[:, rank * (k // world) : (rank + 1) * (k // world)].contiguous()
        ring_p = tp.scatter_buffers(8, n)
        for _ in range(4):
            yk = tp.gemv_row_parallel(w_k, s_k, x_k, ring_p, 1.0)
            want = full[:, rank * (n // world) : (rank + 1) * (n // world)]
            ok &= bool(torch.allclose(yk.float(), want.float(), rtol=1e-2, atol=1e-2 * float(full.float().abs().mean())))
        torch.cuda.synchronize()
        ok &= _lib.load().hb200_device_status(1) == 0
        result[rank] = int(ok)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_over_peer_memory():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = mp.get_context("spawn").Array("i", [0, 0])
    mp.spawn(_two_rank_worker, args=(2, port, result), nprocs=2, join=True)
    assert list(result) == [1, 1]
