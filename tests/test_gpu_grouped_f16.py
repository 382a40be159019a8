"""bf16 / fp16 grouped GEMM entry points and the N-major NVFP4 matmul wrappers against the oracle."""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from helion_b200 import _lib
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(y, ref):
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    assert y.shape == ref.shape and torch.isfinite(y).all()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    return float(((y - ref).abs() / torch.maximum(ref.abs(), floor)).max())


def status_ok():
    torch.cuda.synchronize()
    return _lib.load().hb200_device_status(1) == 0


def test_moe_matmul_ogs_golden(golden):
    g = golden("moe.npz")
    a, w, top1 = g.bf16("moe_a"), g.bf16("moe_w"), g.raw("moe_top1")
    args = hb.moe_matmul_ogs_helion_kernel_args_gen(a.to(DEV), w.to(DEV), top1.to(DEV))
    assert torch.equal(args[2].cpu(), g.raw("moe_counts")) and torch.equal(args[3].cpu(), g.raw("moe_offsets"))
    assert torch.equal(args[4].cpu(), g.raw("moe_sorted"))
    c = hb.moe_matmul_ogs(*args)
    assert status_ok()
    assert rel_err(c, g.bf16("moe_c")) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_moe_matmul_ogs_reference_shape(dtype):
    """The shape of test/test_examples.py:1158-1179 (T=1000, K=500, N=200, E=30)."""
    g = torch.Generator().manual_seed(0)
    t, k, n, e = 1000, 500, 200, 30
    a = torch.randn(t, k, generator=g).to(dtype)
    w = torch.randn(e, k, n, generator=g).to(dtype)
    top1 = torch.randint(e, (t,), generator=g)
    c = hb.moe_matmul_ogs(*hb.moe_matmul_ogs_helion_kernel_args_gen(a.to(DEV), w.to(DEV), top1.to(DEV)))
    assert status_ok()
    assert c.dtype is dtype
    assert rel_err(c, O.moe_matmul_ogs(a, w, top1)) <= 1e-2


def test_grouped_gemm_jagged_reference_shape():
    """G=3, M_i = 32*(i+1), K=N=64 (test/test_examples.py:1697-1766) and a ragged case with an empty group."""
    for sizes, k, n in (([32, 64, 96], 64, 64), ([5, 0, 300, 129], 192, 520)):
        g = torch.Generator().manual_seed(1)
        a = torch.randn(sum(sizes), k, generator=g).to(torch.bfloat16)
        b = torch.randn(k, n, generator=g).to(torch.bfloat16)
        offs = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32)
        y = hb.grouped_gemm_jagged(a.to(DEV), b.to(DEV), offs.to(DEV))
        assert status_ok()
        assert rel_err(y, O.grouped_gemm_jagged(a, b, offs)) <= 1e-2
        y2 = hb.grouped_gemm_jagged_persistent(a.to(DEV), b.to(DEV), offs.to(DEV))
        assert torch.equal(y, y2)


def test_grouped_gemm_deepgemm_worklist():
    """make_case of benchmarks/cute/deepgemm_selected_path.py:209-238: aligned groups, zero padding rows."""
    g = torch.Generator().manual_seed(2)
    actual, n, k, align = [100, 1, 128, 0, 300], 384, 256, 128
    aligned = [(m + align - 1) // align * align for m in actual]
    total = sum(aligned)
    a = torch.randn(total, k, generator=g).to(torch.bfloat16)
    b = torch.randn(len(actual), n, k, generator=g).to(torch.bfloat16)
    rows, start = [], 0
    for grp, (m, am) in enumerate(zip(actual, aligned)):
        a[start + m : start + am] = 7.0  # garbage in the padding rows: outputs there must still be zero
        rows.append((grp, start, m, am))
        start += am
    wl = torch.tensor(rows, dtype=torch.int32)
    y = hb.grouped_gemm_deepgemm(a.to(DEV), b.to(DEV), wl.to(DEV))
    assert status_ok()
    ref = O.grouped_gemm_worklist(a, b, wl)
    assert rel_err(y, ref) <= 1e-2
    for grp, s0, m, am in rows:
        assert float(y[s0 + m : s0 + am].float().abs().max()) == 0.0 if am > m else True


def test_n_major_nvfp4_matmuls_golden(golden):
    g = golden("gemm.npz")
    for tag in "ab":
        a, ap, bp = g.bf16(f"{tag}_a"), g.raw(f"{tag}_a_packed"), g.raw(f"{tag}_b_packed")
        sa, sb = g.e4m3(f"{tag}_sa"), g.e4m3(f"{tag}_sb")
        y = hb.nvfp4_w4a4_matmul(ap.to(DEV), bp.to(DEV).view(torch.float4_e2m1fn_x2), sa.to(DEV), sb.to(DEV), 0.5)
        assert status_ok()
        assert rel_err(y, g.bf16(f"{tag}_y_w4a4")) <= 1e-2
        y = hb.nvfp4_w4a16_matmul(a.to(DEV), bp.to(DEV), sb.to(DEV), 0.5)
        assert rel_err(y, g.bf16(f"{tag}_y_w4a16")) <= 1e-2
    with pytest.raises(ValueError, match="K must be divisible by 16"):
        hb.nvfp4_w4a16_matmul(torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV),
                              torch.zeros(4, 8, dtype=torch.uint8, device=DEV), sb.to(DEV))
