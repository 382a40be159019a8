"""Dense bf16 / fp16 GEMM on CTA pairs, all-gather + matmul and matmul + reduce-scatter as single kernels.

With one rank the fused kernels still run inside one launch: the push CTAs copy the shard into the gather buffer
while the compute CTAs work on it; the reduce-scatter stores into slot 0 and reduces one slot.  The arrival counters
and the waits on them need a peer: that run, over real peer mappings, needs two GPUs and is skipped otherwise.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch

from helion_b200 import _lib
from helion_b200 import dist as D

pytestmark = pytest.mark.gpu
DEV = "cuda"


def status_ok():
    torch.cuda.synchronize()
    return _lib.load().hb200_device_status(1) == 0


def close(got, a, b):
    """fp32 accumulation of exact products: within one place of the output type plus an accumulation slack."""
    ref = a.double() @ b.double()
    mag = a.double().abs() @ b.double().abs()
    ulp = 2.0**-8 if got.dtype is torch.bfloat16 else 2.0**-11
    return bool(((got.double() - ref).abs() <= 1.01 * ulp * ref.abs() + 2.0**-18 * mag + 1e-30).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k,n", [(256, 64, 256), (512, 4096, 768), (300, 200, 264), (1000, 1032, 520), (4096, 1024, 2048)])
def test_dense_matmul(m, k, n, dtype):
    g = torch.Generator().manual_seed(m + k + n)
    a = torch.randn(m, k, generator=g).to(dtype).to(DEV)
    b = (torch.randn(n, k, generator=g) / k**0.5).to(dtype).to(DEV).t()  # [K, N], K-major
    c = D.dense_matmul(a, b)
    assert status_ok()
    assert close(c, a, b)
    c2 = D.dense_matmul(a, b.contiguous())  # N-major b: re-laid out, same values
    assert torch.equal(c, c2)


def test_dense_matmul_rejects_what_it_does_not_take():
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(TypeError):
        D.dense_matmul(a, torch.zeros(64, 256, dtype=torch.float16, device=DEV))
    with pytest.raises(ValueError):
        D.dense_matmul(a, torch.zeros(32, 256, dtype=torch.bfloat16, device=DEV))
    lib = _lib.load()
    c = torch.empty(128, 256, dtype=torch.bfloat16, device=DEV)
    # fewer than 256 rows: the pair kernel does not take it
    assert lib.hb200_dense_matmul(a.data_ptr(), a.data_ptr(), c.data_ptr(), 128, 256, 64, 64, 64, 256, 1, None) == _lib.HB200_ERR_UNSUPPORTED


@pytest.mark.parametrize("splits", [1, 2, 4])
def test_all_gather_matmul_with_one_rank(splits):
    rows, k, n = 1024, 512, 768
    fm = D.FusedMatmulCollectives(torch.device(DEV, torch.cuda.current_device()))
    g = torch.Generator().manual_seed(splits)
    b = (torch.randn(n, k, generator=g) / k**0.5).to(torch.bfloat16).to(DEV).t()
    for step in range(3):
        a = torch.randn(rows, k, generator=g).to(torch.bfloat16).to(DEV)
        gathered, c = fm.all_gather_matmul(a, b, splits_per_rank=splits)
        assert status_ok()
        assert torch.equal(gathered, a)
        assert torch.equal(c, D.dense_matmul(a, b))
        assert close(c, a, b)


def test_matmul_reduce_scatter_with_one_rank():
    m, k, n = 512, 1024, 512
    fm = D.FusedMatmulCollectives(torch.device(DEV, torch.cuda.current_device()))
    g = torch.Generator().manual_seed(3)
    for step in range(3):  # two receive buffers alternate
        a = torch.randn(m, k, generator=g).to(torch.float16).to(DEV)
        b = (torch.randn(n, k, generator=g) / k**0.5).to(torch.float16).to(DEV).t()
        out = fm.matmul_reduce_scatter(a, b)
        assert status_ok()
        assert torch.equal(out, D.dense_matmul(a, b))


def test_shapes_the_fused_kernels_do_not_take():
    fm = D.FusedMatmulCollectives(torch.device(DEV, torch.cuda.current_device()))
    b = torch.zeros(256, 512, dtype=torch.bfloat16, device=DEV).t()
    with pytest.raises(ValueError):
        fm.all_gather_matmul(torch.zeros(384, 256, dtype=torch.bfloat16, device=DEV), b, splits_per_rank=2)  # 192-row chunks
    with pytest.raises(ValueError):
        fm.matmul_reduce_scatter(torch.zeros(384, 256, dtype=torch.bfloat16, device=DEV), b)


def _two_rank_worker(rank: int, world: int, port: int, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        fm = D.FusedMatmulCollectives(dev)
        ok = True
        # all-gather + matmul against the unfused form: gather with the process group, then the same GEMM kernel
        rows, k, n = 1024, 2048, 1536
        g = torch.Generator().manual_seed(31)
        b = (torch.randn(n, k, generator=g) / k**0.5).to(torch.bfloat16).to(dev).t()
        for step in range(6):
            full = torch.randn(world * rows, k, generator=g).to(torch.bfloat16).to(dev)
            shard = full[rank * rows : (rank + 1) * rows].contiguous()
            # the copy engines pull the shards on a second stream, or the GEMM's own warps push them
            gathered, c = fm.all_gather_matmul(shard, b, splits_per_rank=2, gather=("copy_engine", "kernel")[step % 2])
            torch.cuda.synchronize()
            ok &= bool(torch.equal(gathered, full))
            ok &= bool(torch.equal(c, D.dense_matmul(full, b)))
        # matmul + reduce-scatter against: every rank's rounded partial, gathered, summed in rank order in fp32
        m, k_local, n = 1024, 1024, 768
        for step in range(3):
            a = torch.randn(m, world * k_local, generator=g).to(torch.bfloat16).to(dev)
            bb = (torch.randn(n, world * k_local, generator=g) / (world * k_local) ** 0.5).to(torch.bfloat16).to(dev)
            a_l = a[:, rank * k_local : (rank + 1) * k_local].contiguous()
            b_l = bb[:, rank * k_local : (rank + 1) * k_local].contiguous().t()
            out = fm.matmul_reduce_scatter(a_l, b_l)
            partial = D.dense_matmul(a_l, b_l)
            parts = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(parts, partial)
            want = sum(p.float() for p in parts)  # rank order
            rows_r = m // world
            ok &= bool(torch.equal(out, want[rank * rows_r : (rank + 1) * rows_r].to(torch.bfloat16)))
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
