"""Pins the CPU oracle against fixtures produced by the reference's own functions."""

from __future__ import annotations

import torch

from oracle import oracle as O


def _eq_bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.shape == b.shape and torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def test_e2m1_truth_table(golden):
    g = golden("formats.npz")
    codes = torch.arange(256, dtype=torch.int32)
    assert torch.equal(O.dequant_e2m1(codes & 0xF), g.raw("e2m1_lo"))
    assert torch.equal(O.dequant_e2m1((codes >> 4) & 0xF), g.raw("e2m1_hi"))
    # the byte patterns of test/test_quantized_ops.py:67-88 and :118-124
    for raw in (torch.tensor([0x10, 0x21, 0x32, 0x43, 0x54, 0x65, 0x76, 0x87, 0x98, 0xA9, 0xBA, 0xCB, 0xDC, 0xED, 0xFE, 0xFF]),
                torch.arange(16) * 17):
        vals = O.unpack_k_major(raw.to(torch.uint8).reshape(1, -1)).reshape(-1)
        assert torch.equal(vals[0::2], g.raw("e2m1_lo")[raw])
        assert torch.equal(vals[1::2], g.raw("e2m1_hi")[raw])


def test_swizzle_layout(golden):
    g = golden("formats.npz")
    for rows, cols in ((1, 1), (5, 3), (130, 9), (256, 8)):
        assert torch.equal(O.swizzled_offsets(rows, cols), g.raw(f"swz_off_{rows}x{cols}"))
        assert O.swizzled_numel(rows, cols) == g.scalar(f"swz_numel_{rows}x{cols}")
        logical = torch.arange(rows * cols, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(rows, cols)
        buf = O.swizzle_scales(logical)
        assert torch.equal(buf, g.raw(f"swz_buf_{rows}x{cols}"))
        assert torch.equal(O.unswizzle_scales(buf, rows, cols), logical)


def test_quantize_and_pack_rules(golden):
    g = golden("formats.npz")
    assert torch.equal(O.quantize_fp4_e2m1(g.raw("quant_in")), g.raw("quant_codes"))
    codes = g.raw("pack_codes")
    assert torch.equal(O.pack_k_major(codes), g.raw("pack_last_dim"))
    assert torch.equal(O.unpack_k_major(g.raw("pack_last_dim")), g.raw("unpack_last_dim"))
    assert torch.equal(O.unpack_n_major(g.raw("pack_dim0")), g.raw("unpack_dim0"))
    assert torch.equal(g.raw("e4m3_in").to(torch.float8_e4m3fn).view(torch.uint8), g.raw("e4m3_bytes"))


def test_gemv_references(golden):
    g = golden("gemv.npz")
    for tag in "abc":
        w, x, xp = g.raw(f"{tag}_w"), g.bf16(f"{tag}_x"), g.raw(f"{tag}_xp")
        ws, xs, alpha = g.e4m3(f"{tag}_ws"), g.e4m3(f"{tag}_xs"), g.scalar(f"{tag}_alpha")
        assert _eq_bits(O.nvfp4_gemv_bf16in(w, x, ws, alpha), g.bf16(f"{tag}_y_bf16in"))
        assert _eq_bits(O.nvfp4_gemv_fp4in(w, xp, ws, xs, alpha), g.bf16(f"{tag}_y_fp4in"))
        # the batched formulation (dequantise -> matmul) agrees with the GEMV reference to bf16 rounding
        yb = O.nvfp4_gemm_bf16in(w, x.reshape(1, -1), ws, alpha).reshape(-1).float()
        ya = g.bf16(f"{tag}_y_bf16in").float()
        assert (yb - ya).abs().max() <= 2e-2 * ya.abs().max()


def test_gemm_references(golden):
    g = golden("gemm.npz")
    for tag in "ab":
        a, ap, bp = g.bf16(f"{tag}_a"), g.raw(f"{tag}_a_packed"), g.raw(f"{tag}_b_packed")
        sa, sb = g.e4m3(f"{tag}_sa"), g.e4m3(f"{tag}_sb")
        assert _eq_bits(O.nvfp4_w4a16_matmul(a, bp, sb, 0.5), g.bf16(f"{tag}_y_w4a16"))
        assert _eq_bits(O.nvfp4_w4a4_matmul(ap, bp, sa, sb, 0.5), g.bf16(f"{tag}_y_w4a4"))
        # K-major restatement used for the block-scaled GEMM: same numbers up to fp32 summation order
        k2, n = bp.shape
        codes = torch.stack((bp & 0xF, bp >> 4), dim=1).reshape(k2 * 2, n)
        b_k_major = O.pack_k_major(codes.t().contiguous())
        y = O.nvfp4_scaled_matmul(ap, b_k_major, sa, sb, alpha=0.5).float()
        ref = g.bf16(f"{tag}_y_w4a4").float()
        assert (y - ref).abs().max() <= 1e-2 * ref.abs().max()


def test_quant_producer_references(golden):
    g = golden("quant_producers.npz")
    x = g.bf16("silu_x")
    for gs in (64, 128):
        q, s = O.silu_and_mul_per_block_quant(x, gs)
        assert _eq_bits(q, g.e4m3(f"silu_q_{gs}")) and _eq_bits(s, g.raw(f"silu_s_{gs}"))
    q, s = O.silu_and_mul_per_block_quant(x, 128, g.raw("silu_ub"))
    assert _eq_bits(q, g.e4m3("silu_q_ub")) and _eq_bits(s, g.raw("silu_s_ub"))

    xr, wr = g.bf16("rms_x"), g.bf16("rms_w")
    q, s, _ = O.rms_norm_dynamic_per_token_quant(xr, wr, 1e-6)
    assert _eq_bits(q, g.e4m3("rms_q")) and _eq_bits(s, g.raw("rms_s"))
    q, s, res = O.rms_norm_dynamic_per_token_quant(xr, wr, 1e-6, torch.tensor(2.0), g.bf16("rms_res_in"))
    assert _eq_bits(q, g.e4m3("rms_q_res")) and _eq_bits(s, g.raw("rms_s_res"))
    assert _eq_bits(res, g.bf16("rms_res_out"))

    xg = g.bf16("grp_x")
    for ue in (0, 1):
        q, s = O.per_token_group_fp8_quant(xg, 128, 1e-10, -448.0, 448.0, bool(ue))
        assert _eq_bits(q, g.e4m3(f"grp_q_{ue}")) and _eq_bits(s, g.raw(f"grp_s_{ue}"))


def test_sibling_quant_producer_references(golden):
    g = golden("quant_siblings.npz")
    x = g.bf16("dyn_x")
    q, s = O.dynamic_per_token_scaled_fp8_quant(x)
    assert _eq_bits(q, g.e4m3("dyn_q")) and _eq_bits(s, g.raw("dyn_s"))
    q, s = O.dynamic_per_token_scaled_fp8_quant(x, torch.tensor(0.01))
    assert _eq_bits(q, g.e4m3("dyn_q_ub")) and _eq_bits(s, g.raw("dyn_s_ub"))
    xr, wr, res = g.bf16("rpb_x"), g.bf16("rpb_w"), g.bf16("rpb_res")
    for gs in (64, 128):
        q, s, _ = O.rms_norm_per_block_quant(xr, wr, 1e-6, gs)
        assert _eq_bits(q, g.e4m3(f"rpb_q_{gs}")) and _eq_bits(s, g.raw(f"rpb_s_{gs}"))
        q, s, new_res = O.rms_norm_per_block_quant(xr, wr, 1e-6, gs, None, res)
        assert _eq_bits(q, g.e4m3(f"rpb_q_{gs}_res")) and _eq_bits(s, g.raw(f"rpb_s_{gs}_res"))
        assert _eq_bits(new_res, g.bf16(f"rpb_newres_{gs}"))


def test_scaled_mm_reference_kernel(golden):
    """The oracle against outputs of the reference's scaled_mm kernel itself (run by its CPU interpreter)."""
    g = golden("scaled_mm.npz")
    ulp = {"bf16": 2.0**-8, "f16": 2.0**-11, "f32": 2.0**-20}
    for tag in "abc":
        a, b = g.e4m3(f"smm_{tag}_a"), g.e4m3(f"smm_{tag}_b_nk").t()
        for stag in ("tensor", "rows", "mixed"):
            sa, sb = g.raw(f"smm_{tag}_{stag}_sa"), g.raw(f"smm_{tag}_{stag}_sb")
            for dtag in ("bf16", "f16", "f32"):
                bias = g.typed(f"smm_{tag}_{stag}_{dtag}_bias", dtag)
                for btag, bb in (("bias", bias), ("nobias", None)):
                    ref = g.typed(f"smm_{tag}_{stag}_{dtag}_{btag}_c", dtag)
                    got = O.scaled_mm(a, b, sa, sb, bb, ref.dtype)
                    assert got.dtype == ref.dtype and got.shape == ref.shape
                    # the kernel sums fp32 in tile order, the oracle rounds an exact sum once: outputs may sit
                    # on either side of a rounding boundary, by one place of the larger of result and bias
                    mag = ref.float().abs() if bb is None else torch.maximum(ref.float().abs(), bb.float().abs()[None, :])
                    assert bool(((got.float() - ref.float()).abs() <= ulp[dtag] * mag + 1e-30).all())
                    if dtag != "f32":
                        assert float((got == ref).float().mean()) >= 0.97


def test_silu_mul_fp8_reference_kernel(golden):
    """The oracle against outputs of the reference's silu_mul_fp8 kernel (run by its CPU interpreter).

    Where the scaled value leaves the e4m3 range the interpreter's torch cast gives NaN; the compiled kernel's
    conversion saturates, and so do the oracle and the CUDA kernel: those positions must hold +-448."""
    g = golden("silu_mul_fp8.npz")
    for tag, dt in (("a", torch.bfloat16), ("b", torch.bfloat16), ("c", torch.float16)):
        x = g.raw(f"smf_{tag}_x").view(dt)
        scale = g.raw(f"smf_{tag}_scale")
        ref = g.e4m3(f"smf_{tag}_kernel")
        assert _eq_bits(ref, g.e4m3(f"smf_{tag}_torch"))  # the module's torch reference agrees with its kernel
        got = O.silu_mul_fp8(x, scale)
        overflow = torch.isnan(ref.float())
        assert torch.equal(got.view(torch.uint8)[~overflow], ref.view(torch.uint8)[~overflow])
        assert bool((got.float()[overflow].abs() == 448.0).all())
    assert bool(torch.isnan(g.e4m3("smf_b_kernel").float()).any())  # the fixture does exercise the overflow case


def test_quant_producer_reference_kernels(golden):
    """The oracle against outputs of the reference's quant KERNELS (run by the reference's CPU interpreter), in
    addition to the modules' torch references above."""
    g = golden("reference_kernels.npz")
    x = g.bf16("k_silu_x")
    for gs in (64, 128):
        q, s = O.silu_and_mul_per_block_quant(x, gs)
        assert _eq_bits(q, g.e4m3(f"k_silu_q_{gs}")) and _eq_bits(s, g.raw(f"k_silu_s_{gs}"))
    xr, wr, res = g.bf16("k_rms_x"), g.bf16("k_rms_w"), g.bf16("k_rms_res")
    q, s, _ = O.rms_norm_dynamic_per_token_quant(xr, wr, 1e-6)
    assert _eq_bits(q, g.e4m3("k_rms_q")) and _eq_bits(s, g.raw("k_rms_s"))
    q, s, new_res = O.rms_norm_dynamic_per_token_quant(xr, wr, 1e-6, None, res)
    assert _eq_bits(q, g.e4m3("k_rms_q_res")) and _eq_bits(s, g.raw("k_rms_s_res"))
    assert _eq_bits(new_res, g.bf16("k_rms_newres"))
    q, s = O.dynamic_per_token_scaled_fp8_quant(xr)
    assert _eq_bits(q, g.e4m3("k_dyn_q")) and _eq_bits(s, g.raw("k_dyn_s"))
    # per_token_group_fp8_quant: the kernel takes the group maximum and divides in the input type, its module's
    # fp32 reference (which the oracle and the CUDA kernel follow) does not: scales agree to bf16 precision only
    q, s = O.per_token_group_fp8_quant(xr, 128, 1e-10, -448.0, 448.0, False)
    ks, kq = g.raw("k_grp_s"), g.e4m3("k_grp_q")
    assert float(((s - ks).abs() / s).max()) <= 2.0**-7
    assert float((q.view(torch.uint8) == kq.view(torch.uint8)).float().mean()) >= 0.9
    assert float((q.float() - kq.float()).abs().max()) <= 32.0  # one e4m3 step at the top of the range


def test_moe_references(golden):
    g = golden("moe.npz")
    a, w, top1 = g.bf16("moe_a"), g.bf16("moe_w"), g.raw("moe_top1")
    c = O.moe_matmul_ogs(a, w, top1)
    ref = g.bf16("moe_c")
    routed = torch.isin(top1, torch.unique(top1))
    # bf16 @ bf16 on CPU may accumulate in a different order than fp32-upcast matmul: compare to bf16 rounding
    assert (c[routed].float() - ref[routed].float()).abs().max() <= 2e-2 * ref[routed].float().abs().max()
    order, counts, offsets = O.moe_sort(top1.reshape(-1, 1), w.shape[0])
    assert torch.equal(order, g.raw("moe_sorted"))
    assert torch.equal(counts, g.raw("moe_counts")) and torch.equal(offsets, g.raw("moe_offsets"))
    assert int(counts.max()) == g.scalar("moe_max_t")


def test_nvfp4_quantiser_composition():
    """The quantiser has no reference function; check its defining properties."""
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.02
    packed, scales, g = O.nvfp4_quantize(w)
    assert float(g) == float(w.abs().amax() / (6 * 448))
    deq = O.dequant_scaled_k_major(packed, scales) * g
    # every block reproduces its largest element to e4m3 precision, others within half a code step
    blk = w.reshape(64, 16, 16)
    err = (deq.reshape(64, 16, 16) - blk).abs().amax(-1)
    assert (err <= blk.abs().amax(-1) * 0.27).all()
    # zero rows stay zero and do not produce NaNs
    z = torch.zeros(2, 32)
    p, s, gz = O.nvfp4_quantize(z, per_token=True)
    assert p.sum() == 0 and s.view(torch.uint8).sum() == 0 and (gz == 0).all()
