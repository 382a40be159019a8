"""Parity of the NVFP4 GEMV / decode-batch kernels with the CPU oracle (runs on the B200 box)."""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from helion_b200 import _lib
from helion_b200 import layouts as L
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"

# bf16 outputs, fp32 accumulation: |y - ref| <= 1e-2 * max(|ref|, rms(ref)) elementwise.  The floor keeps
# the relative bound meaningful for outputs that cancel to (almost) zero.
REL_TOL = 1e-2


def assert_close_rel(y: torch.Tensor, ref: torch.Tensor, tol: float = REL_TOL) -> float:
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    assert y.shape == ref.shape
    assert torch.isfinite(y).all()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    err = (y - ref).abs() / torch.maximum(ref.abs(), floor)
    worst = float(err.max()) if err.numel() else 0.0
    assert worst <= tol, f"max relative error {worst:.3e} > {tol}"
    return worst


def make_case(n: int, k: int, seed: int, batch: int = 1):
    """Benchmark-style inputs: W ~ N(0, 0.02) quantised to NVFP4 with a global scale, x ~ N(0, 1) bf16."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(batch, k, generator=g).to(torch.bfloat16)
    packed, scales, gs = O.nvfp4_quantize(w)
    return packed, scales, float(gs), x


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_golden_fixtures(golden, tag):
    g = golden("gemv.npz")
    w, x, xp = g.raw(f"{tag}_w"), g.bf16(f"{tag}_x"), g.raw(f"{tag}_xp")
    ws, xs, alpha = g.e4m3(f"{tag}_ws"), g.e4m3(f"{tag}_xs"), g.scalar(f"{tag}_alpha")
    y = hb.nvfp4_gemv_bf16in(w.to(DEV), x.to(DEV), ws.to(DEV), alpha)
    assert y.shape == (w.shape[0],) and y.dtype is torch.bfloat16
    assert_close_rel(y, g.bf16(f"{tag}_y_bf16in"))
    y = hb.nvfp4_gemv_fp4in(w.to(DEV).view(torch.float4_e2m1fn_x2), xp.to(DEV), ws.to(DEV), xs.to(DEV), alpha)
    assert_close_rel(y, g.bf16(f"{tag}_y_fp4in"))
    # tensor-core formulation of the same product
    y = hb.nvfp4_gemv_bf16in_batched(w.to(DEV), x.to(DEV).reshape(1, -1), ws.to(DEV), alpha, use_mma=True)
    assert_close_rel(y.reshape(-1), g.bf16(f"{tag}_y_bf16in"))


@pytest.mark.parametrize(
    "n,k",
    [(8192, 4096), (128, 16384), (96, 28672), (1000, 1040), (33, 16), (256, 256), (4096, 14336)],
)
def test_bf16in_against_oracle(n, k):
    packed, scales, gs, x = make_case(n, k, seed=0)
    ref = O.nvfp4_gemv_bf16in(packed, x.reshape(-1), scales, gs)
    y = hb.nvfp4_gemv_bf16in(packed.to(DEV), x.reshape(-1).to(DEV), scales.to(DEV), gs)
    assert_close_rel(y, ref)
    y2 = hb.nvfp4_gemv_bf16in_batched(packed.to(DEV), x.to(DEV), scales.to(DEV), gs, use_mma=True)
    assert_close_rel(y2.reshape(-1), ref)
    # the dequantise-then-fp32-matmul formulation
    ref2 = O.nvfp4_gemm_bf16in(packed, x, scales, gs).reshape(-1)
    assert_close_rel(y, ref2)


@pytest.mark.parametrize("n,k", [(8192, 4096), (200, 592), (128, 8192)])
def test_fp4in_against_oracle(n, k):
    packed, scales, gs, x = make_case(n, k, seed=1)
    xp, xs, xg = O.nvfp4_quantize(x)
    ref = O.nvfp4_gemv_fp4in(packed, xp.reshape(-1), scales, xs, gs * float(xg))
    y = hb.nvfp4_gemv_fp4in(packed.to(DEV), xp.reshape(-1).to(DEV), scales.to(DEV), xs.to(DEV), gs * float(xg))
    assert_close_rel(y, ref)


@pytest.mark.parametrize("batch", [2, 3, 4, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n,k", [(1024, 2048), (200, 592), (128, 12288)])
def test_decode_batch_against_oracle(batch, n, k):
    packed, scales, gs, x = make_case(n, k, seed=4, batch=batch)
    ref = O.nvfp4_gemm_bf16in(packed, x, scales, gs)
    y = hb.nvfp4_gemv_bf16in_batched(packed.to(DEV), x.to(DEV), scales.to(DEV), gs)
    assert y.shape == (batch, n)
    assert_close_rel(y, ref)


def test_linearity_at_full_size():
    """Size-independent property on a 70B-class matrix: GEMV(x1 + x2) == GEMV(x1) + GEMV(x2) for exactly
    representable inputs (small integers), bit for bit, and scaling alpha by 2 doubles the output."""
    n, k = 57344, 8192
    g = torch.Generator().manual_seed(4)
    w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g).to(DEV)
    s = L.swizzle_fp8_scales(torch.ones(n, k // 16).to(torch.float8_e4m3fn)).to(DEV)
    x1 = torch.randint(-2, 3, (k,), generator=g).to(torch.bfloat16).to(DEV)
    x2 = torch.randint(-2, 3, (k,), generator=g).to(torch.bfloat16).to(DEV)
    alpha = 2.0**-6
    y1 = hb.nvfp4_gemv_bf16in(w, x1, s, alpha, path="simt").float()
    y2 = hb.nvfp4_gemv_bf16in(w, x2, s, alpha, path="simt").float()
    y12 = hb.nvfp4_gemv_bf16in(w, x1 + x2, s, alpha, path="simt").float()
    # all partial sums are small integers times 0.5: exact in fp16/fp32, so only the final bf16 rounding differs
    assert ((y1 + y2) - y12).abs().max() <= 2.0**-7 * y12.abs().max()
    y_half = hb.nvfp4_gemv_bf16in(w, x1, s, alpha / 2, path="simt").float()
    assert torch.equal(y_half * 2, y1)
    yb = hb.nvfp4_gemv_bf16in_batched(w, torch.stack([x1, x2]), s, alpha, path="simt").float()
    assert torch.equal(yb[0], y1) and torch.equal(yb[1], y2)
    # the tensor-core path sees the activations through four NVFP4 terms: the last bf16 place may differ
    yt = hb.nvfp4_gemv_bf16in_batched(w, torch.stack([x1, x2]), s, alpha, path="tc").float()
    assert (yt[0] - y1).abs().max() <= 2.0**-7 * y1.abs().max() and (yt[1] - y2).abs().max() <= 2.0**-7 * y2.abs().max()
    # which is what a single row takes by default on a matrix of this size
    ya = hb.nvfp4_gemv_bf16in(w, x1, s, alpha).float()
    assert (ya - y1).abs().max() <= 2.0**-7 * y1.abs().max()


def test_c_abi_direct_call_respects_output_bounds():
    """Call the C entry point on a canary-padded, poison-filled output buffer."""
    n, k = 300, 1024
    packed, scales, gs, x = make_case(n, k, seed=9)
    w, xs_, sc = packed.to(DEV), x.reshape(-1).to(DEV), scales.to(DEV).view(torch.uint8)
    pad = 64
    buf = torch.full((n + 2 * pad,), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = buf[pad : pad + n]
    _lib.call(
        "hb200_nvfp4_gemv_bf16in", w.data_ptr(), xs_.data_ptr(), sc.data_ptr(), out.data_ptr(), n, k, 1, gs,
        torch.cuda.current_stream().cuda_stream,
    )
    torch.cuda.synchronize()
    assert torch.isnan(buf[:pad]).all() and torch.isnan(buf[pad + n :]).all()
    assert_close_rel(out, O.nvfp4_gemv_bf16in(packed, x.reshape(-1), scales, gs))


def test_cuda_graph_capture_and_replay():
    """The entry points neither allocate nor synchronise, so a call can be captured and replayed on new data."""
    n, k = 512, 2048
    packed, scales, gs, x = make_case(n, k, seed=11)
    w, sc = packed.to(DEV), scales.to(DEV)
    xd = x.reshape(-1).to(DEV)
    hb.nvfp4_gemv_bf16in(w, xd, sc, gs)  # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = hb.nvfp4_gemv_bf16in(w, xd, sc, gs)
    x2 = torch.randn(k, generator=torch.Generator().manual_seed(12)).to(torch.bfloat16)
    xd.copy_(x2.to(DEV))
    y.fill_(13.0)
    graph.replay()
    torch.cuda.synchronize()
    assert_close_rel(y, O.nvfp4_gemv_bf16in(packed, x2, scales, gs))


def test_empty_shapes():
    w = torch.empty(0, 64, dtype=torch.uint8, device=DEV)
    s = torch.empty(0, dtype=torch.float8_e4m3fn, device=DEV)
    x = torch.zeros(128, dtype=torch.bfloat16, device=DEV)
    assert hb.nvfp4_gemv_bf16in(w, x, s).shape == (0,)
