"""Host-side logic of the multi-GPU paths, run as two gloo ranks on the CPU."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helion_b200 import dist as D
from helion_b200 import layouts as L


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dense_expert_fn(w1, w2):
    """CPU stand-in for a rank's experts: silu(x W1g^T) * (x W1u^T) W2^T in fp32, bf16 out."""

    def fn(rows, local_expert):
        out = torch.zeros(rows.shape[0], w2.shape[1], dtype=torch.float32)
        inter = w1.shape[1] // 2
        for e in range(w1.shape[0]):
            idx = (local_expert == e).nonzero(as_tuple=True)[0]
            if idx.numel():
                h = rows[idx].float() @ w1[e].t()
                out[idx] = (torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]) @ w2[e].t()
        return out.to(torch.bfloat16)

    return fn


def _torch_router(logits, top_k):
    """Tensor-code stand-in for the routing kernel (softmax in fp32, then top-k)."""
    return torch.topk(torch.softmax(logits.to(torch.float32), dim=-1), top_k, dim=-1)


def _torch_combine(back, row_of_pair, pair_weight, tokens):
    """Tensor-code stand-in for the combine kernel: routing-weighted fp32 sum of every token's rows."""
    rows = back.float()[row_of_pair.long()] * pair_weight.float()[:, None]
    return rows.reshape(tokens, -1, back.shape[1]).sum(dim=1).to(torch.bfloat16)


def _worker(rank: int, world: int, port: int, result_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        t, h, inter, e, k = 48, 32, 16, 8, 2
        x = torch.randn(t, h, generator=g).to(torch.bfloat16)
        logits = torch.randn(t, e, generator=g)
        w1 = torch.randn(e, 2 * inter, h, generator=g) * 0.2
        w2 = torch.randn(e, h, inter, generator=g) * 0.2
        per_t, per_e = t // world, e // world
        xs, ls = x[rank * per_t : (rank + 1) * per_t], logits[rank * per_t : (rank + 1) * per_t]
        fn = _dense_expert_fn(w1[rank * per_e : (rank + 1) * per_e], w2[rank * per_e : (rank + 1) * per_e])
        y = D.expert_parallel_moe(xs, ls, k, e, fn, router=_torch_router, combine=_torch_combine)
        torch.save(y, os.path.join(result_dir, f"moe_{rank}.pt"))

        # column-parallel gather: rank r contributes columns [r*N/g, (r+1)*N/g)
        full = torch.arange(4 * 256, dtype=torch.float32).reshape(4, 256)
        lo, hi = D.shard_range(256, world, rank)
        got = D.all_gather_columns(full[:, lo:hi].contiguous())
        torch.save(got, os.path.join(result_dir, f"gather_{rank}.pt"))

        plan = D.plan_dispatch(torch.tensor([[0, 7], [3, 4], [1, 1]]), 8)
        torch.save((plan.send_counts, plan.recv_counts, plan.local_expert), os.path.join(result_dir, f"plan_{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_expert_parallel_and_gather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = torch.Generator().manual_seed(0)
    t, h, inter, e, k = 48, 32, 16, 8, 2
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    w1 = torch.randn(e, 2 * inter, h, generator=g) * 0.2
    w2 = torch.randn(e, h, inter, generator=g) * 0.2
    # single-process answer with the same expert function
    probs = torch.softmax(logits.float(), -1)
    wts, experts = torch.topk(probs, k, dim=-1)
    fn = _dense_expert_fn(w1, w2)
    ref = torch.zeros(t, h)
    for s in range(k):
        ref += fn(x, experts[:, s]).float() * wts[:, s : s + 1]
    got = torch.cat([torch.load(tmp_path / f"moe_{r}.pt") for r in range(world)])
    assert torch.allclose(got.float(), ref.to(torch.bfloat16).float(), rtol=2e-2, atol=1e-3)

    full = torch.arange(4 * 256, dtype=torch.float32).reshape(4, 256)
    for r in range(world):
        assert torch.equal(torch.load(tmp_path / f"gather_{r}.pt"), full)
    # every rank sent pairs {0,1,1,3 -> rank 0; 4,7 -> rank 1}
    for r in range(world):
        send, recv, local = torch.load(tmp_path / f"plan_{r}.pt")
        assert send == [4, 2]
        assert recv == ([4, 4] if r == 0 else [2, 2])
        assert local.tolist() == ([0, 1, 1, 3] * 2 if r == 0 else [0, 3] * 2)


def test_shard_helpers():
    assert D.shard_range(1024, 4, 1) == (256, 512)
    with pytest.raises(ValueError, match="multiple of 128"):
        D.shard_range(1024, 16, 0)
    with pytest.raises(ValueError, match="evenly"):
        D.shard_range(1000, 3, 0)
    n, k = 512, 160
    packed = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8)
    logical = (torch.rand(n, k // 16) + 0.5).to(torch.float8_e4m3fn)
    scales = L.swizzle_fp8_scales(logical)
    for r in range(4):
        p, s = D.shard_weight_rows(packed, scales, 4, r)
        assert torch.equal(p, packed[r * 128 : (r + 1) * 128])
        assert torch.equal(
            s.view(torch.uint8), L.swizzle_fp8_scales(logical[r * 128 : (r + 1) * 128]).view(torch.uint8)
        )
