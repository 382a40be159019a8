"""Expert-parallel NVFP4 MoE over the library's own exchange kernels.

On one GPU the "ranks" are objects that share ordinary device buffers and whose phases are run rank after rank
(every launch completes before the next one that depends on it starts; the barrier kernel is never launched for more
ranks than there are GPUs).  The run over real peer mappings needs two GPUs and is skipped otherwise.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch

from helion_b200 import _lib
from helion_b200 import dist as D
from helion_b200 import moe as M

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(y, ref):
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    assert torch.isfinite(y).all()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    return float(((y - ref).abs() / torch.maximum(ref.abs(), floor)).max())


def status_ok():
    torch.cuda.synchronize()
    return _lib.load().hb200_device_status(1) == 0


def make_problem(world, t_local, h, inter, e, seed, dev=DEV):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(world * t_local, h, generator=g).to(torch.bfloat16).to(dev)
    logits = torch.randn(world * t_local, e, generator=g).to(dev)
    w_gu = M.quantize_expert_weights((torch.randn(e, 2 * inter, h, generator=g) * 0.02).to(dev))
    w_d = M.quantize_expert_weights((torch.randn(e, h, inter, generator=g) * 0.02).to(dev))
    return x, logits, w_gu, w_d


def shard(bundle, world, rank):
    per = bundle.experts // world
    sl = slice(rank * per, (rank + 1) * per)
    return M.GroupedNvfp4Weight(bundle.packed[sl].contiguous(), bundle.scales[sl].contiguous(),
                                bundle.global_scale[sl].contiguous(), bundle.gate_up_interleaved)


@pytest.mark.parametrize("world,t_local,h,inter,e,k", [(2, 64, 256, 128, 8, 2), (4, 40, 256, 256, 8, 4), (2, 200, 512, 384, 16, 8),
                                                      (1, 96, 256, 128, 4, 2)])
def test_emulated_ranks_match_the_one_gpu_layer(world, t_local, h, inter, e, k):
    x, logits, w_gu, w_d = make_problem(world, t_local, h, inter, e, seed=world + k)
    w_gu_i = M.interleave_gate_up(w_gu)
    single = M.nvfp4_moe(x, logits, k, w_gu_i, w_d)
    nbytes = D.ExpertParallel.buffer_bytes(world, t_local, h, k, e)
    buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    ranks = [D.ExpertParallel(torch.device(DEV, torch.cuda.current_device()), t_local, h, k, e, _emulate=(world, r, buffers))
             for r in range(world)]
    for step in range(2):  # twice: the buffers are reused from step to step
        for r, ep in enumerate(ranks):
            ep.dispatch(x[r * t_local : (r + 1) * t_local].contiguous(), logits[r * t_local : (r + 1) * t_local].contiguous())
        torch.cuda.synchronize()
        for r, ep in enumerate(ranks):
            ep.run_experts(shard(w_gu_i, world, r), shard(w_d, world, r))
        torch.cuda.synchronize()
        got = torch.cat([ep.combine() for ep in ranks])
        assert status_ok()
        # the sum over a token's slots is taken per expert rank first (11 significant bits), then over ranks, then
        # rounded to bf16: against the one-GPU layer that is at most a last-place flip of the bf16 result
        assert rel_err(got, single) <= 2.0**-7
        assert float((got != single).float().mean()) <= 0.2


def test_a_rank_that_receives_nothing_and_experts_without_tokens():
    """All tokens prefer the experts of rank 0: rank 1 receives no pair at all and returns nothing."""
    world, t_local, h, inter, e, k = 2, 48, 256, 128, 8, 2
    x, logits, w_gu, w_d = make_problem(world, t_local, h, inter, e, seed=9)
    logits[:, e // 2 :] = -30.0
    logits[:, 0] += 5.0  # and expert 3 probably gets few or none
    w_gu_i = M.interleave_gate_up(w_gu)
    single = M.nvfp4_moe(x, logits, k, w_gu_i, w_d)
    nbytes = D.ExpertParallel.buffer_bytes(world, t_local, h, k, e)
    buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    ranks = [D.ExpertParallel(torch.device(DEV, torch.cuda.current_device()), t_local, h, k, e, _emulate=(world, r, buffers))
             for r in range(world)]
    for r, ep in enumerate(ranks):
        ep.dispatch(x[r * t_local : (r + 1) * t_local].contiguous(), logits[r * t_local : (r + 1) * t_local].contiguous())
    for r, ep in enumerate(ranks):
        ep.run_experts(shard(w_gu_i, world, r), shard(w_d, world, r))
    got = torch.cat([ep.combine() for ep in ranks])
    assert status_ok()
    assert rel_err(got, single) <= 2.0**-7  # every token's pairs sit on one rank: the same sum, re-rounded once


def test_shapes_the_exchange_does_not_take():
    lib = _lib.load()
    assert lib.hb200_ep_buffer_bytes(3, 64, 256, 2, 8) == _lib.HB200_ERR_UNSUPPORTED   # experts % world
    assert lib.hb200_ep_buffer_bytes(2, 64, 200, 2, 8) == _lib.HB200_ERR_UNSUPPORTED   # hidden % 64
    assert lib.hb200_ep_buffer_bytes(9, 64, 256, 2, 18) == _lib.HB200_ERR_UNSUPPORTED  # world > 8
    assert lib.hb200_ep_slots(2, 64, 256, 8, 8) == 2 * 64 * 4  # capacity: min(top_k, experts per rank) pairs per token


def _two_rank_worker(rank: int, world: int, port: int, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        t_local, h, inter, e, k = 256, 512, 384, 16, 4
        x, logits, w_gu, w_d = make_problem(world, t_local, h, inter, e, seed=21, dev=dev)
        w_gu_i = M.interleave_gate_up(w_gu)
        single = M.nvfp4_moe(x, logits, k, w_gu_i, w_d)
        ep = D.ExpertParallel(dev, t_local, h, k, e)
        ok = True
        for _ in range(3):
            y = ep.moe(x[rank * t_local : (rank + 1) * t_local].contiguous(),
                       logits[rank * t_local : (rank + 1) * t_local].contiguous(), shard(w_gu_i, world, rank), shard(w_d, world, rank))
            ok &= rel_err(y, single[rank * t_local : (rank + 1) * t_local]) <= 1e-2
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
