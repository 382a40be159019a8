"""Host-side mirror of the reference interface: layouts, validators, error messages, fake tensors."""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from helion_b200 import layouts as L
from oracle import oracle as O


def test_layout_helpers_match_golden(golden):
    g = golden("formats.npz")
    for rows, cols in ((1, 1), (5, 3), (130, 9), (256, 8)):
        r = torch.arange(rows)[:, None]
        c = torch.arange(cols)[None, :]
        assert torch.equal(L.swizzled_scale_offsets(r, c, cols), g.raw(f"swz_off_{rows}x{cols}"))
        assert L.swizzled_scale_numel(rows, cols) == g.scalar(f"swz_numel_{rows}x{cols}")
        logical = torch.arange(rows * cols, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(rows, cols)
        buf = L.swizzle_fp8_scales(logical)
        assert torch.equal(buf, g.raw(f"swz_buf_{rows}x{cols}"))
        assert torch.equal(L.unswizzle_fp8_scales(buf, rows, cols), logical)
    assert L.swizzled_scale_offsets(200, 7, 9) == int(g.raw("swz_off_256x8")[0, 0]) + ((200 // 128) * 3 + 1) * 512 + (200 % 32) * 16 + ((200 % 128) // 32) * 4 + 3
    assert torch.equal(L.quantize_fp4_e2m1(g.raw("quant_in")), g.raw("quant_codes"))
    codes = g.raw("pack_codes")
    assert torch.equal(L.pack_fp4_last_dim(codes), g.raw("pack_last_dim"))
    assert torch.equal(L.pack_fp4(codes.t().contiguous()), g.raw("pack_dim0"))
    assert torch.equal(L.unpack_fp4_last_dim(g.raw("pack_last_dim")), codes)
    assert torch.equal(L.unpack_fp4(g.raw("pack_dim0")), codes.t())
    assert torch.equal(L.dequantize_fp4_codes(torch.arange(16)), O.dequant_e2m1(torch.arange(16)))


def test_swizzle_of_float8_and_1d_input():
    s = (torch.rand(3, 5) + 0.5).to(torch.float8_e4m3fn)
    buf = L.swizzle_fp8_scales(s)
    assert buf.dtype is torch.float8_e4m3fn and buf.numel() == 128 * 8
    assert torch.equal(L.unswizzle_fp8_scales(buf, 3, 5).view(torch.uint8), s.view(torch.uint8))
    one = L.swizzle_fp8_scales(s[0])
    assert torch.equal(one.view(torch.uint8), L.swizzle_fp8_scales(s[:1]).view(torch.uint8))
    with pytest.raises(ValueError, match="expected 1D or 2D scales"):
        L.swizzle_fp8_scales(torch.zeros(1, 1, 1))


def test_host_quantiser_matches_oracle():
    torch.manual_seed(3)
    x = (torch.randn(40, 96) * 0.02).to(torch.bfloat16)
    for per_token in (False, True):
        p, s, g = L.nvfp4_quantize_host(x, per_token=per_token)
        po, so, go = O.nvfp4_quantize(x, per_token=per_token)
        assert torch.equal(p, po) and torch.equal(s.view(torch.uint8), so.view(torch.uint8)) and torch.equal(g, go)
        deq = L.nvfp4_dequantize_host(p, s, g)
        ref = O.dequant_scaled_k_major(po, so) * (go.reshape(-1, 1) if per_token else go)
        assert torch.equal(deq, ref)


def _gemv_inputs(n=64, kb=128):
    w = torch.randint(0, 256, (n, kb), dtype=torch.uint8)
    x = torch.randn(kb * 2, dtype=torch.bfloat16)
    s = L.swizzle_fp8_scales((torch.rand(n, kb // 8) + 0.5).to(torch.float8_e4m3fn))
    return w, x, s


def test_gemv_validators_match_reference_messages():
    """The error contract of test/test_examples.py:2031-2055."""
    w, x, s = _gemv_inputs()
    with pytest.raises(ValueError, match="x_bf16 must contain"):
        hb.nvfp4_gemv_bf16in(w, x[:-2], s)
    with pytest.raises(ValueError, match="x_packed must contain"):
        hb.nvfp4_gemv_fp4in(w, torch.zeros(100, dtype=torch.uint8), s, L.swizzle_fp8_scales(torch.ones(16).to(torch.float8_e4m3fn)))
    with pytest.raises(ValueError, match="weight_packed must be contiguous"):
        hb.nvfp4_gemv_bf16in(w.t(), x, s)
    with pytest.raises(ValueError, match="K bytes must be divisible by 8"):
        hb.nvfp4_gemv_bf16in(w[:, :4].contiguous(), x[:8], s)
    with pytest.raises(ValueError, match=r"weight_scale must contain 2048 SWIZZLE_32_4_4 scale values for logical shape \(64, 16\); got 2047"):
        hb.nvfp4_gemv_bf16in(w, x, s[:-1])
    with pytest.raises(ValueError, match="must be a 2D packed FP4 tensor"):
        hb.nvfp4_gemv_bf16in(w.reshape(-1), x, s)
    with pytest.raises(TypeError, match="expected uint8 or float4_e2m1fn_x2 tensor"):
        hb.nvfp4_gemv_bf16in(w.to(torch.int32), x, s)


def test_no_cpu_fallback():
    w, x, s = _gemv_inputs()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hb.nvfp4_gemv_bf16in(w, x, s)
    q = torch.empty(4, 128, dtype=torch.float8_e4m3fn)
    sc = torch.empty(4, 1, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hb.per_token_group_fp8_quant(torch.randn(4, 128, dtype=torch.bfloat16), q, sc, 128, 1e-10, -448.0, 448.0, False)


def test_fp8_consumers_validate_and_have_no_cpu_fallback():
    a = torch.zeros(4, 64).to(torch.float8_e4m3fn)
    b = torch.zeros(32, 64).to(torch.float8_e4m3fn).t()  # [K, N] with unit stride along K, as the reference wants
    c = torch.empty(4, 32, dtype=torch.bfloat16)
    one = torch.ones(1)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hb.scaled_mm(c, a, b, one, one)
    with pytest.raises(AssertionError):
        hb.scaled_mm(c, a, b.contiguous(), one, one)  # b no longer K-major
    with pytest.raises(AssertionError):
        hb.scaled_mm(c, a, b, torch.ones(3), one)  # scale_a neither [1] nor [M]
    with pytest.raises(AssertionError):
        hb.scaled_mm(c, a, b, one, one, torch.zeros(32))  # bias not in c's dtype
    with pytest.raises(TypeError):
        hb.scaled_mm(c, a.view(torch.uint8), b.view(torch.uint8), one, one)  # neither FP8 nor int8
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hb.scaled_mm(c, a.view(torch.int8), b.view(torch.int8), one, one)  # the int8 form, like the FP8 one, needs the GPU
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hb.silu_mul_fp8(x, one)
    with pytest.raises(AssertionError, match="Scale must be a scalar Tensor"):
        hb.silu_mul_fp8(x, torch.ones(2))
    with pytest.raises(ValueError):
        hb.silu_mul_fp8(torch.zeros(4, 24, dtype=torch.bfloat16), one)


def test_quant_producer_assertions():
    x = torch.randn(4, 256, dtype=torch.bfloat16)
    out = torch.empty(4, 128, dtype=torch.float8_e4m3fn)
    with pytest.raises(AssertionError):
        hb.silu_and_mul_per_block_quant(out, x, torch.empty(4, 1), 32)  # group size not in {64, 128}
    with pytest.raises(AssertionError):
        hb.silu_and_mul_per_block_quant(out, x, torch.empty(4, 2), 128)  # wrong number of groups
    with pytest.raises(AssertionError):
        hb.rms_norm_dynamic_per_token_quant(out, x[:, :128].contiguous(), torch.ones(128), torch.empty(4, 1), 1e-6)  # dtype mismatch
    with pytest.raises(AssertionError):
        hb.per_token_group_fp8_quant(x, torch.empty(4, 256, dtype=torch.float8_e4m3fn), torch.empty(4, 3), 128, 1e-10, -448.0, 448.0, False)


def test_custom_ops_registered_with_fake_impls():
    from torch._subclasses.fake_tensor import FakeTensorMode

    assert hasattr(torch.ops.helion_b200, "nvfp4_gemv_bf16in")
    with FakeTensorMode():
        w = torch.empty(64, 128, dtype=torch.uint8, device="cuda")
        x = torch.empty(2, 256, dtype=torch.bfloat16, device="cuda")
        s = torch.empty(2048, dtype=torch.uint8, device="cuda")
        y = torch.ops.helion_b200.nvfp4_gemv_bf16in(w, x, s, 1.0, "auto")
        assert y.shape == (2, 64) and y.dtype is torch.bfloat16 and y.device.type == "cuda"
        y = torch.ops.helion_b200.nvfp4_gemv_fp4in(w, torch.empty(128, dtype=torch.uint8, device="cuda"), s, s, 1.0, "auto")
        assert y.shape == (64,)
        y8 = torch.ops.helion_b200.silu_mul_fp8(x, torch.empty(1, device="cuda"))
        assert y8.shape == (2, 128) and y8.dtype is torch.float8_e4m3fn
        c, sc, g = torch.ops.helion_b200.nvfp4_quantize(x, None)
        assert c.shape == (2, 128) and sc.numel() == 128 * 16 and g.shape == (2,)


def test_grouped_and_moe_ops_registered_with_fake_impls():
    """Every grouped / MoE entry point is a ``torch.library`` custom op with a fake implementation, as
    test/test_custom_op.py:23-33 does for a kernel: shapes and dtypes trace without a device."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    from helion_b200 import moe as M

    for name in ("moe_matmul_ogs", "grouped_gemm_jagged", "grouped_gemm_deepgemm", "grouped_matmul_f16",
                 "grouped_matmul_f16_out", "nvfp4_moe", "moe_route_top_k", "moe_build_schedule"):
        assert hasattr(torch.ops.helion_b200, name), name
    with FakeTensorMode():
        cuda = dict(device="cuda")
        a = torch.empty(300, 64, dtype=torch.bfloat16, **cuda)
        y = hb.grouped_gemm_jagged(a, torch.empty(64, 96, dtype=torch.bfloat16, **cuda), torch.empty(4, dtype=torch.int32, **cuda))
        assert y.shape == (300, 96) and y.dtype is torch.bfloat16
        y = hb.grouped_gemm_deepgemm(a, torch.empty(3, 96, 64, dtype=torch.bfloat16, **cuda), torch.empty(5, 4, dtype=torch.int32, **cuda))
        assert y.shape == (300, 96)
        y = hb.moe_matmul_ogs(a.half(), torch.empty(4, 64, 96, dtype=torch.float16, **cuda), torch.empty(4, dtype=torch.int32, **cuda),
                              torch.empty(5, dtype=torch.int32, **cuda), torch.empty(300, dtype=torch.int32, **cuda), 300)
        assert y.shape == (300, 96) and y.dtype is torch.float16
        x = torch.empty(64, 256, dtype=torch.bfloat16, **cuda)
        logits = torch.empty(64, 8, **cuda)
        w, e = M.route_top_k(logits, 2)
        assert w.shape == (64, 2) and w.dtype is torch.float32 and e.dtype is torch.int64
        sched = M.build_schedule(e, 8)
        assert sched.tile_info.shape == (sched.max_tiles, 2) and sched.max_tiles == 1 + 8 and sched.row_of_pair.shape == (128,)
        gu = M.GroupedNvfp4Weight(torch.empty(8, 256, 128, dtype=torch.uint8, **cuda),
                                  torch.empty(8, 256 * 16, dtype=torch.float8_e4m3fn, **cuda), torch.empty(8, **cuda))
        dn = M.GroupedNvfp4Weight(torch.empty(8, 256, 64, dtype=torch.uint8, **cuda),
                                  torch.empty(8, 256 * 8, dtype=torch.float8_e4m3fn, **cuda), torch.empty(8, **cuda))
        y = M.nvfp4_moe(x, logits, 2, gu, dn)
        assert y.shape == (64, 256) and y.dtype is torch.bfloat16 and y.device.type == "cuda"
        from helion_b200 import dist as D

        assert hasattr(torch.ops.helion_b200, "dense_matmul_out")
        y = D.dense_matmul(torch.empty(512, 128, dtype=torch.bfloat16, **cuda), torch.empty(384, 128, dtype=torch.bfloat16, **cuda).t())
        assert y.shape == (512, 384) and y.dtype is torch.bfloat16


def test_product_modules_have_no_cpu_path():
    """CPU tensors are refused by the routing and combine entry points (the multi-rank host-logic tests inject
    their own stand-ins instead)."""
    from helion_b200 import dist as D
    from helion_b200 import moe as M

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        M.route_top_k(torch.zeros(4, 8), 2)
    with pytest.raises(ValueError, match="CUDA"):
        D.combine_rows(torch.zeros(8, 16, dtype=torch.bfloat16), torch.arange(8, dtype=torch.int32), torch.ones(8), 4)


def test_interleave_gate_up_moves_whole_128_row_tiles():
    """Host-side weight preparation for the SiLU-mul epilogue: codes and scale tiles move together."""
    from helion_b200 import moe as M

    e, inter, k = 2, 256, 64
    n = 2 * inter
    g = torch.Generator().manual_seed(0)
    packed = torch.randint(0, 256, (e, n, k // 2), dtype=torch.uint8, generator=g)
    logical = [(torch.rand(n, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn) for _ in range(e)]
    scales = torch.stack([L.swizzle_fp8_scales(s).view(torch.uint8) for s in logical]).view(torch.float8_e4m3fn)
    w = M.GroupedNvfp4Weight(packed, scales, torch.ones(e))
    wi = M.interleave_gate_up(w)
    assert wi.gate_up_interleaved and M.interleave_gate_up(wi) is wi
    for i in range(e):
        un = L.unswizzle_fp8_scales(wi.scales[i], n, k // 16).view(torch.uint8)
        for j in range(inter // 128):
            rows_g = slice(256 * j, 256 * j + 128)
            rows_u = slice(256 * j + 128, 256 * j + 256)
            assert torch.equal(wi.packed[i, rows_g], packed[i, 128 * j : 128 * j + 128])
            assert torch.equal(wi.packed[i, rows_u], packed[i, inter + 128 * j : inter + 128 * j + 128])
            assert torch.equal(un[rows_g], logical[i][128 * j : 128 * j + 128].view(torch.uint8))
            assert torch.equal(un[rows_u], logical[i][inter + 128 * j : inter + 128 * j + 128].view(torch.uint8))
    with pytest.raises(ValueError, match="multiple of 256"):
        M.interleave_gate_up(M.GroupedNvfp4Weight(packed[:, :384], scales, torch.ones(e)))
