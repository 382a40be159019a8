"""The tensor-core GEMV / decode-batch path (tcgen05 on packed weights, activations as NVFP4 residual terms)
against the CPU oracle and against the SIMT kernels that take the bf16 activations exactly."""

from __future__ import annotations

import ctypes

import pytest
import torch

import helion_b200 as hb
from helion_b200 import _lib
from helion_b200 import ops
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_TOL = 1e-2  # bf16 out, fp32 accumulate: |y - ref| <= 1e-2 * max(|ref|, rms(ref))


def rel_err(y, ref):
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    assert y.shape == ref.shape
    assert torch.isfinite(y).all()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    return (y - ref).abs() / torch.maximum(ref.abs(), floor)


def device_status_ok():
    torch.cuda.synchronize()
    return _lib.load().hb200_device_status(1) == 0


def make_case(n, k, batch, seed, dist="normal"):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(batch, k, generator=g)
    if dist == "outliers":  # a few activations a hundred times larger than the rest
        x = x * torch.where(torch.rand(batch, k, generator=g) < 0.002, 100.0, 1.0)
    elif dist == "tiny":
        x = x * 1e-6
    elif dist == "sparse":
        x = x * (torch.rand(batch, k, generator=g) < 0.05)
    packed, scales, gs = O.nvfp4_quantize(w)
    return packed, scales, float(gs), x.to(torch.bfloat16)


@pytest.mark.parametrize(
    "n,k,batch",
    [(1024, 2048, 1), (4096, 4096, 1), (8192, 8192, 1), (2048, 8192, 4), (1000, 2048, 8), (512, 28672, 16),
     (2048, 4096, 32), (640, 2080, 3), (128, 96, 2), (300, 32, 1), (10240, 8192, 5)],
)
def test_bf16in_tc_against_oracle_and_simt(n, k, batch):
    packed, scales, gs, x = make_case(n, k, batch, seed=n + k + batch)
    ref = O.nvfp4_gemm_bf16in(packed, x, scales, gs)
    y = hb.nvfp4_gemv_bf16in_batched(packed.to(DEV), x.to(DEV), scales.to(DEV), gs, path="tc")
    assert device_status_ok()
    assert y.shape == (batch, n) and y.dtype is torch.bfloat16
    e = rel_err(y, ref)
    assert float(e.max()) <= REL_TOL, f"max relative error {float(e.max()):.3e}"
    # the expansion error itself is far smaller than the bf16 rounding both paths share
    y_simt = hb.nvfp4_gemv_bf16in_batched(packed.to(DEV), x.to(DEV), scales.to(DEV), gs, path="simt")
    d = rel_err(y, y_simt.float())
    assert float(d.max()) <= REL_TOL
    assert float(d.pow(2).mean().sqrt()) <= 2e-3


@pytest.mark.parametrize("dist", ["outliers", "tiny", "sparse"])
def test_bf16in_tc_activation_distributions(dist):
    n, k, batch = 2048, 4096, 4
    packed, scales, gs, x = make_case(n, k, batch, seed=17, dist=dist)
    ref = O.nvfp4_gemm_bf16in(packed, x, scales, gs)
    y = hb.nvfp4_gemv_bf16in_batched(packed.to(DEV), x.to(DEV), scales.to(DEV), gs, path="tc")
    assert device_status_ok()
    assert float(rel_err(y, ref).max()) <= REL_TOL


def test_zero_activation_gives_zero():
    packed, scales, gs, x = make_case(512, 1024, 2, seed=3)
    y = hb.nvfp4_gemv_bf16in_batched(packed.to(DEV), torch.zeros_like(x).to(DEV), scales.to(DEV), gs, path="tc")
    assert device_status_ok()
    assert torch.count_nonzero(y) == 0


@pytest.mark.parametrize("n,k", [(1024, 2048), (8192, 8192), (1000, 4096), (256, 28672), (640, 2080)])
def test_fp4in_tc_against_oracle(n, k):
    g = torch.Generator().manual_seed(n + k)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(1, k, generator=g).to(torch.bfloat16)
    packed, scales, gs = O.nvfp4_quantize(w)
    xp, xs, gx = O.nvfp4_quantize(x.float())
    alpha = float(gs) * float(gx)
    ref = O.nvfp4_gemv_fp4in(packed, xp.reshape(-1), scales, xs, alpha)
    args = (packed.to(DEV), xp.reshape(-1).to(DEV), scales.to(DEV), xs.to(DEV), alpha)
    y = hb.nvfp4_gemv_fp4in(*args, path="tc")
    assert device_status_ok()
    assert y.shape == (n,) and y.dtype is torch.bfloat16
    assert float(rel_err(y, ref.float()).max()) <= REL_TOL
    # same products, fp32 accumulation in another order: at most the last bf16 place apart from the SIMT kernel
    y_simt = hb.nvfp4_gemv_fp4in(*args, path="simt")
    assert float(rel_err(y, y_simt.float()).max()) <= 8e-3


def test_repeat_calls_are_bit_identical_and_leave_counters_at_zero():
    n, k, batch = 8192, 8192, 2  # 64 row tiles over 148 CTAs: every tile is shared between CTAs
    packed, scales, gs, x = make_case(n, k, batch, seed=5)
    w, s, xd = packed.to(DEV), scales.to(DEV), x.to(DEV)
    first = hb.nvfp4_gemv_bf16in_batched(w, xd, s, gs, path="tc")
    for _ in range(5):
        again = hb.nvfp4_gemv_bf16in_batched(w, xd, s, gs, path="tc")
        assert torch.equal(first, again)
    assert device_status_ok()
    ws = ops.tc_workspace(torch.device(DEV, torch.cuda.current_device()), 0)
    assert torch.count_nonzero(ws[: 4 * 4096]) == 0  # the counter region


def test_workspace_too_small_is_rejected():
    n, k = 1024, 2048
    packed, scales, gs, x = make_case(n, k, 1, seed=9)
    w, s, xd = packed.to(DEV), scales.to(DEV).view(torch.uint8), x.to(DEV)
    out = torch.empty(1, n, dtype=torch.bfloat16, device=DEV)
    need = _lib.load().hb200_nvfp4_gemv_tc_workspace_bytes(n, k, 1, 4)
    assert need > 0
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    ptrs = (ctypes.c_void_p * 1)(out.data_ptr())
    lib = _lib.load()
    rc = lib.hb200_nvfp4_gemv_bf16in_tc(w.data_ptr(), xd.data_ptr(), s.data_ptr(), ptrs, 1, n, k, 1, n, 0, 1.0,
                                        ws.data_ptr(), need - 1, None)
    assert rc == _lib.HB200_ERR_WORKSPACE
    rc = lib.hb200_nvfp4_gemv_bf16in_tc(w.data_ptr(), xd.data_ptr(), s.data_ptr(), ptrs, 1, n, 2064, 1, n, 0, 1.0,
                                        ws.data_ptr(), need, None)
    assert rc == _lib.HB200_ERR_UNSUPPORTED  # K % 32 != 0
    assert lib.hb200_nvfp4_gemv_tc_workspace_bytes(n, k, 33, 4) == _lib.HB200_ERR_UNSUPPORTED
    rc = lib.hb200_nvfp4_gemv_bf16in_tc(w.data_ptr(), xd.data_ptr(), s.data_ptr(), ptrs, 1, n, k, 1, n, 0, gs,
                                        ws.data_ptr(), need, None)
    assert rc == 0 and device_status_ok()
    ref = O.nvfp4_gemm_bf16in(packed, x, scales, gs)
    assert float(rel_err(out, ref).max()) <= REL_TOL


def test_dirty_workspace_outside_the_counters_is_harmless():
    """Only the counter region has to be zero: everything else may hold any bytes from earlier shapes."""
    n, k, batch = 1000, 2080, 3  # K ends inside a 64-element scale atom: its padding columns multiply zero codes
    packed, scales, gs, x = make_case(n, k, batch, seed=21)
    w, s, xd = packed.to(DEV), scales.to(DEV).view(torch.uint8), x.to(DEV)
    lib = _lib.load()
    need = lib.hb200_nvfp4_gemv_tc_workspace_bytes(n, k, batch, 4)
    outs = []
    for fill in (0x00, 0xFF, 0x7F):
        ws = torch.full((need,), fill, dtype=torch.uint8, device=DEV)
        ws[: 4 * 4096] = 0
        out = torch.empty(batch, n, dtype=torch.bfloat16, device=DEV)
        ptrs = (ctypes.c_void_p * 1)(out.data_ptr())
        rc = lib.hb200_nvfp4_gemv_bf16in_tc(w.data_ptr(), xd.data_ptr(), s.data_ptr(), ptrs, 1, n, k, batch, n, 0, gs,
                                            ws.data_ptr(), need, None)
        assert rc == 0 and device_status_ok()
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert float(rel_err(outs[0], O.nvfp4_gemm_bf16in(packed, x, scales, gs)).max()) <= REL_TOL
