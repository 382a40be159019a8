"""Parity of the tcgen05 block-scaled NVFP4 GEMM with the dequantise-then-fp32-matmul oracle."""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from helion_b200 import _lib
from helion_b200 import layouts as L
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_TOL = 1e-2  # bf16 output, fp32 accumulate: |y - ref| <= 1e-2 * max(|ref|, rms(ref))


def assert_close_rel(y, ref, tol=REL_TOL):
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    assert y.shape == ref.shape
    assert torch.isfinite(y).all()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    worst = float(((y - ref).abs() / torch.maximum(ref.abs(), floor)).max())
    assert worst <= tol, f"max relative error {worst:.3e} > {tol}"
    return worst


def device_status_ok():
    torch.cuda.synchronize()
    return _lib.load().hb200_device_status(1) == 0


def random_operands(m, n, k, seed):
    """Random codes and scales in [0.5, 1.5) as the reference's own checks use (examples/nvfp4_gemm.py:583-596)."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
    sa = O.swizzle_scales((torch.rand(m, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
    sb = O.swizzle_scales((torch.rand(n, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
    return a, b, sa, sb


@pytest.mark.parametrize(
    "m,n,k",
    [(128, 256, 256), (128, 128, 64), (128, 256, 1024), (256, 512, 512), (64, 64, 128), (100, 72, 96),
     (300, 520, 2080), (129, 257, 320), (1, 8, 32), (1024, 1024, 4096)],
)
def test_scaled_matmul_random_codes(m, n, k):
    a, b, sa, sb = random_operands(m, n, k, seed=m + n + k)
    ref = O.nvfp4_scaled_matmul(a, b, sa, sb, torch.float32)
    y = hb.nvfp4_scaled_matmul(a.to(DEV), b.to(DEV).t(), sa.to(DEV), sb.to(DEV), torch.float32)
    assert device_status_ok()
    assert y.shape == (m, n) and y.dtype is torch.float32
    # e2m1 x e4m3 products and fp32 accumulation: only summation order differs
    assert_close_rel(y, ref, 1e-4)
    yb = hb.nvfp4_scaled_matmul(a.to(DEV), b.to(DEV).t(), sa.to(DEV), sb.to(DEV))
    assert_close_rel(yb, ref)
    yh = hb.nvfp4_scaled_matmul(a.to(DEV), b.to(DEV).t(), sa.to(DEV), sb.to(DEV), torch.float16, alpha=2.0**-4)
    assert_close_rel(yh, ref * 2.0**-4)


def test_golden_w4a4_fixture(golden):
    """The reference's W4A4 golden outputs (N-major B) re-laid out K-major."""
    g = golden("gemm.npz")
    for tag in "ab":
        ap, bp = g.raw(f"{tag}_a_packed"), g.raw(f"{tag}_b_packed")
        sa, sb = g.e4m3(f"{tag}_sa"), g.e4m3(f"{tag}_sb")
        b_k_major = L.pack_fp4_last_dim(L.unpack_fp4(bp).t().contiguous())
        y = hb.nvfp4_scaled_matmul(ap.to(DEV), b_k_major.to(DEV).t(), sa.to(DEV), sb.to(DEV), alpha=0.5)
        assert device_status_ok()
        assert_close_rel(y, g.bf16(f"{tag}_y_w4a4"))


def test_quantised_operands_config1_scaled_down():
    """The dense-GEMM benchmark configuration at 1/8 scale: A ~ N(0,1) bf16, B ~ N(0,0.02), both NVFP4-quantised with global scales."""
    m = n = k = 1024
    g = torch.Generator().manual_seed(1)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    b = torch.randn(n, k, generator=g) * 0.02
    ap, sa, ga = O.nvfp4_quantize(a)
    bp, sb, gb = O.nvfp4_quantize(b)
    alpha = float(ga) * float(gb)
    ref = O.nvfp4_scaled_matmul(ap, bp, sa, sb, torch.float32, alpha=alpha)
    y = hb.nvfp4_scaled_matmul(ap.to(DEV), bp.to(DEV).t(), sa.to(DEV), sb.to(DEV), alpha=alpha)
    assert device_status_ok()
    assert_close_rel(y, ref)
    # the quantised product stays close to the unquantised one (sanity, loose)
    full = a.float() @ b.t()
    assert (y.float().cpu() - full).pow(2).mean().sqrt() <= 0.2 * full.pow(2).mean().sqrt()


def test_b_layout_variants_and_errors():
    a, b, sa, sb = random_operands(128, 128, 128, seed=3)
    ref = O.nvfp4_scaled_matmul(a, b, sa, sb, torch.float32)
    ad, bd, sad, sbd = a.to(DEV), b.to(DEV), sa.to(DEV), sb.to(DEV)
    # a row-major [K/2, N] right-hand side is re-laid out like the reference does
    b_rowmajor = bd.t().contiguous()
    y = hb.nvfp4_scaled_matmul(ad.view(torch.float4_e2m1fn_x2), b_rowmajor, sad, sbd, torch.float32)
    assert_close_rel(y, ref, 1e-4)
    with pytest.raises(TypeError, match="unsupported output dtype"):
        hb.nvfp4_scaled_matmul(ad, bd.t(), sad, sbd, torch.float64)
    with pytest.raises(TypeError, match="scale_a must be torch.float8_e4m3fn"):
        hb.nvfp4_scaled_matmul(ad, bd.t(), sad.view(torch.uint8), sbd)
    with pytest.raises(ValueError, match="is incompatible with"):
        hb.nvfp4_scaled_matmul(ad, bd[:, :32].t(), sad, sbd)
    with pytest.raises(ValueError, match="scale_b must contain"):
        hb.nvfp4_scaled_matmul(ad, bd.t(), sad, sbd[:-1])


@pytest.mark.parametrize("chunks", [1, 2, 4])
def test_host_pipelined_matmul_equals_the_resident_path(chunks):
    """Activations in pinned host memory, rows in chunks over three streams: the same bits as quantising and
    multiplying the whole matrix on the device; two calls in a row reuse the buffers."""
    m, n, k = 1024, 512, 1024
    g = torch.Generator().manual_seed(21)
    w = torch.randn(n, k, generator=g) * 0.02
    wp, ws, wg = O.nvfp4_quantize(w)
    wp, ws = wp.to(DEV), ws.to(DEV)
    pipe = None
    for call in range(2):
        a = torch.randn(m, k, generator=g).to(torch.bfloat16)
        ga = (a.float().abs().amax() / (6.0 * 448.0)).reshape(1).to(DEV)
        alpha = float(ga) * float(wg)
        pipe = hb.HostPipelinedMatmul(wp, ws, ga, alpha, m, chunks=chunks)  # scales change with the activations
        host_a, host_out = a.pin_memory(), torch.full((m, n), float("nan"), dtype=torch.bfloat16).pin_memory()
        pipe(host_a, host_out)
        torch.cuda.synchronize()
        codes, scales, _ = hb.nvfp4_quantize(a.to(DEV), ga)
        want = hb.nvfp4_scaled_matmul(codes, wp.t(), scales, ws, alpha=alpha)
        assert torch.equal(host_out.to(DEV), want)
    with pytest.raises(ValueError):
        hb.HostPipelinedMatmul(wp, ws, ga, alpha, m, chunks=8)  # 128-row chunks
    with pytest.raises(ValueError):
        pipe(a, host_out)  # not pinned
