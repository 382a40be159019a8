"""Regenerates ``tests/golden/*.npz`` by running the REFERENCE's own functions on seeded CPU inputs.

Run from the repository root in a container that has the reference checkout:

    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py <reference checkout>

The fixtures hold inputs and the reference's outputs as raw integer views (bf16 as
uint16, float8_e4m3fn and packed fp4 as uint8), so loading them needs numpy only.
Nothing at test time reads the reference checkout; this script is the only link.
"""

from __future__ import annotations

import importlib.util
import os
from pathlib import Path
import sys

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.uint16)
    elif t.dtype in (torch.float8_e4m3fn, torch.float4_e2m1fn_x2):
        t = t.view(torch.uint8)
    return t.numpy().copy()  # a copy: callers reuse their output buffers


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    gemv = _load(ref / "examples" / "nvfp4_gemv.py", "ref_nvfp4_gemv")
    gemm = _load(ref / "examples" / "nvfp4_gemm.py", "ref_nvfp4_gemm")
    moe = _load(ref / "examples" / "moe_matmul_ogs.py", "ref_moe")
    pk = ref / "pretuned_kernels"
    silu = _load(pk / "silu_and_mul_per_block_quant" / "silu_and_mul_per_block_quant.py", "ref_silu")
    rms = _load(pk / "rms_norm_dynamic_per_token_quant" / "rms_norm_dynamic_per_token_quant.py", "ref_rms")
    grp = _load(pk / "per_token_group_fp8_quant" / "per_token_group_fp8_quant.py", "ref_grp")

    # ---- formats: e2m1 truth table, swizzle offsets, quantiser rule ------------------------------
    all_bytes = torch.arange(256, dtype=torch.int32)
    fmt = {
        "e2m1_lo": _np(gemv._dequant_e2m1(all_bytes & 0xF)),
        "e2m1_hi": _np(gemv._dequant_e2m1((all_bytes >> 4) & 0xF)),
    }
    for rows, cols in ((1, 1), (5, 3), (130, 9), (256, 8)):
        r = torch.arange(rows, dtype=torch.int64)[:, None]
        c = torch.arange(cols, dtype=torch.int64)[None, :]
        fmt[f"swz_off_{rows}x{cols}"] = _np(gemv.swizzled_scale_offsets(r, c, cols))
        fmt[f"swz_numel_{rows}x{cols}"] = np.int64(gemv.swizzled_scale_numel(rows, cols))
        logical = torch.arange(rows * cols, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(rows, cols)
        fmt[f"swz_buf_{rows}x{cols}"] = _np(gemv.swizzle_fp8_scales(logical))
    ties = torch.tensor(
        [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.0, -0.1, -0.25, -0.75, 0.0, 0.1, -6.5, 2.4999, 2.5001],
        dtype=torch.float32,
    )
    torch.manual_seed(10)
    qin = torch.cat([ties, torch.randn(4096) * 3.0])
    fmt["quant_in"] = _np(qin)
    fmt["quant_codes"] = _np(gemm.quantize_fp4_e2m1(qin))
    codes = torch.randint(0, 16, (6, 32), dtype=torch.uint8)
    fmt["pack_codes"] = _np(codes)
    fmt["pack_last_dim"] = _np(gemm.pack_fp4_last_dim(codes))
    fmt["pack_dim0"] = _np(gemm.pack_fp4(codes.t().contiguous()))
    fmt["unpack_last_dim"] = _np(gemm.unpack_and_dequantize_fp4(gemm.pack_fp4_last_dim(codes), last_dim=True))
    fmt["unpack_dim0"] = _np(gemm.unpack_and_dequantize_fp4(gemm.pack_fp4(codes.t().contiguous())))
    # torch's fp32 -> e4m3 cast on boundary cases (what every reference function relies on)
    e4 = torch.tensor([2.0**-9, 2.0**-10, 1.5 * 2.0**-10, -0.0, 17.0, 19.0, 21.0, 448.0, 460.0, 464.0, 0.3, -447.9])
    fmt["e4m3_in"] = _np(e4)
    fmt["e4m3_bytes"] = _np(e4.to(torch.float8_e4m3fn))
    np.savez_compressed(HERE / "formats.npz", **fmt)

    # ---- GEMV (shapes of test/test_examples.py:2001-2055 plus ragged ones) -----------------------
    out = {}
    for tag, (n, kb, seed) in {"a": (64, 128, 0), "b": (200, 296, 1), "c": (130, 8, 2)}.items():
        torch.manual_seed(seed)
        w = torch.randint(0, 256, (n, kb), dtype=torch.uint8)
        x = torch.randn(kb * 2, dtype=torch.bfloat16)
        xp = torch.randint(0, 256, (kb,), dtype=torch.uint8)
        ws = gemv.make_fp8_scales((n, kb // 8), torch.device("cpu"))
        xs = gemv.make_fp8_scales((kb // 8,), torch.device("cpu"))
        alpha = 0.37
        out[f"{tag}_w"], out[f"{tag}_x"], out[f"{tag}_xp"] = _np(w), _np(x), _np(xp)
        out[f"{tag}_ws"], out[f"{tag}_xs"] = _np(ws), _np(xs)
        out[f"{tag}_alpha"] = np.float64(alpha)
        out[f"{tag}_y_bf16in"] = _np(gemv.reference_nvfp4_gemv_bf16in(w, x, ws, alpha))
        out[f"{tag}_y_fp4in"] = _np(gemv.reference_nvfp4_gemv_fp4in(w, xp, ws, xs, alpha))
    np.savez_compressed(HERE / "gemv.npz", **out)

    # ---- GEMM references (N-major B, shapes of test/test_examples.py:1940-1998) ------------------
    out = {}
    for tag, (m, k, n, seed) in {"a": (64, 128, 64, 3), "b": (48, 256, 136, 4)}.items():
        torch.manual_seed(seed)
        a = torch.randn(m, k, dtype=torch.bfloat16)
        wf = torch.randn(k, n, dtype=torch.bfloat16)
        b_packed = gemm.pack_fp4(gemm.quantize_fp4_e2m1(wf))
        a_packed = gemm.pack_fp4_last_dim(gemm.quantize_fp4_e2m1(a))
        sa = gemm.make_fp8_scales((m, k // 16), torch.device("cpu"))
        sb = gemm.make_fp8_scales((n, k // 16), torch.device("cpu"))
        out[f"{tag}_a"], out[f"{tag}_a_packed"], out[f"{tag}_b_packed"] = _np(a), _np(a_packed), _np(b_packed)
        out[f"{tag}_sa"], out[f"{tag}_sb"] = _np(sa), _np(sb)
        out[f"{tag}_y_w4a16"] = _np(gemm.reference_nvfp4_w4a16_matmul(a, b_packed, sb, 0.5))
        out[f"{tag}_y_w4a4"] = _np(gemm.reference_nvfp4_w4a4_matmul(a_packed, b_packed, sa, sb, 0.5))
    np.savez_compressed(HERE / "gemm.npz", **out)

    # ---- quant producers ---------------------------------------------------------------------------
    out = {}
    torch.manual_seed(5)
    x = torch.randn(24, 2 * 512, dtype=torch.bfloat16)
    for gs in (64, 128):
        q = torch.empty(24, 512, dtype=torch.float8_e4m3fn)
        s = torch.empty(24, 512 // gs, dtype=torch.float32)
        silu._silu_and_mul_per_block_quant_torch(q, x, s, gs)
        out[f"silu_q_{gs}"], out[f"silu_s_{gs}"] = _np(q), _np(s)
    ub = torch.tensor(0.75, dtype=torch.float32)
    q = torch.empty(24, 512, dtype=torch.float8_e4m3fn)
    s = torch.empty(24, 4, dtype=torch.float32)
    silu._silu_and_mul_per_block_quant_torch(q, x, s, 128, ub)
    out["silu_x"], out["silu_ub"], out["silu_q_ub"], out["silu_s_ub"] = _np(x), _np(ub), _np(q), _np(s)

    torch.manual_seed(6)
    xr = torch.randn(24, 1024, dtype=torch.bfloat16)
    wr = (torch.rand(1024) + 0.5).to(torch.bfloat16)
    res = torch.randn(24, 1024, dtype=torch.bfloat16)
    q = torch.empty(24, 1024, dtype=torch.float8_e4m3fn)
    s = torch.empty(24, 1, dtype=torch.float32)
    rms._rms_norm_dynamic_per_token_quant_torch(q, xr, wr, s, 1e-6)
    out["rms_x"], out["rms_w"], out["rms_q"], out["rms_s"] = _np(xr), _np(wr), _np(q), _np(s)
    res2 = res.clone()
    rms._rms_norm_dynamic_per_token_quant_torch(q, xr, wr, s, 1e-6, torch.tensor(2.0), res2)
    out["rms_res_in"], out["rms_res_out"], out["rms_q_res"], out["rms_s_res"] = _np(res), _np(res2), _np(q), _np(s)

    torch.manual_seed(7)
    xg = torch.randn(24, 512, dtype=torch.bfloat16)
    xg[3, 128:256] = 0  # an all-zero group exercises the eps clamp
    for ue in (False, True):
        q = torch.empty(24, 512, dtype=torch.float8_e4m3fn)
        s = torch.empty(24, 4, dtype=torch.float32)
        grp._per_token_group_fp8_quant_torch(xg, q, s, 128, 1e-10, -448.0, 448.0, ue)
        out[f"grp_q_{int(ue)}"], out[f"grp_s_{int(ue)}"] = _np(q), _np(s)
    out["grp_x"] = _np(xg)
    np.savez_compressed(HERE / "quant_producers.npz", **out)

    # ---- sibling quant producers ------------------------------------------------------------------
    dyn = _load(pk / "dynamic_per_token_scaled_fp8_quant" / "dynamic_per_token_scaled_fp8_quant.py", "ref_dyn")
    rpb = _load(pk / "rms_norm_per_block_quant" / "rms_norm_per_block_quant.py", "ref_rpb")
    out = {}
    torch.manual_seed(21)
    xd = (torch.randn(24, 384) * torch.logspace(-3, 2, 24)[:, None]).to(torch.bfloat16)
    xd[5] = 0  # an all-zero row: the scale floor
    for tag, ub in (("", None), ("_ub", torch.tensor(0.01))):
        q = torch.zeros(24, 384, dtype=torch.float8_e4m3fn)
        sc = torch.zeros(24, 1)
        dyn._dynamic_per_token_scaled_fp8_quant_torch(q, xd, sc, ub)
        out[f"dyn_q{tag}"], out[f"dyn_s{tag}"] = _np(q), _np(sc)
    out["dyn_x"] = _np(xd)
    xr = torch.randn(20, 512).to(torch.bfloat16)
    wr = (torch.rand(512) + 0.5).to(torch.bfloat16)
    res = torch.randn(20, 512).to(torch.bfloat16)
    out["rpb_x"], out["rpb_w"], out["rpb_res"] = _np(xr), _np(wr), _np(res)
    for gs in (64, 128):
        for tag, r in (("", None), ("_res", res.clone())):
            q = torch.zeros(20, 512, dtype=torch.float8_e4m3fn)
            sc = torch.zeros(20, 512 // gs)
            rpb._rms_norm_per_block_quant_torch(q, xr, wr, sc, 1e-6, None, r, gs, False)
            out[f"rpb_q_{gs}{tag}"], out[f"rpb_s_{gs}{tag}"] = _np(q), _np(sc)
            if r is not None:
                out[f"rpb_newres_{gs}"] = _np(r)
    np.savez_compressed(HERE / "quant_siblings.npz", **out)

    # ---- row-wise scaled FP8 GEMM: the reference KERNEL itself, run by its interpreter on the CPU ----
    smm = _load(pk / "scaled_mm" / "scaled_mm.py", "ref_scaled_mm")
    out = {}
    torch.manual_seed(33)
    for tag, (m, k, n) in (("a", (16, 256, 128)), ("b", (20, 208, 72)), ("c", (3, 64, 40))):
        scale = 1.0 / k**0.5
        a = (scale * (0.5 + torch.rand(m, k))).to(torch.float8_e4m3fn)
        b = (scale * (torch.rand(n, k) - 0.5)).to(torch.float8_e4m3fn).t()
        out[f"smm_{tag}_a"], out[f"smm_{tag}_b_nk"] = _np(a), _np(b.t())
        for stag, (sa, sb) in (
            ("tensor", (torch.rand(1, 1) + 0.5, torch.rand(1, 1) + 0.5)),
            ("rows", (torch.rand(m, 1) + 0.5, torch.rand(n, 1) + 0.5)),
            ("mixed", (torch.rand(1) + 0.5, torch.rand(n) + 0.5)),
        ):
            out[f"smm_{tag}_{stag}_sa"], out[f"smm_{tag}_{stag}_sb"] = _np(sa), _np(sb)
            for dtag, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
                bias = (torch.rand(n) - 0.5).to(dt)
                out[f"smm_{tag}_{stag}_{dtag}_bias"] = _np(bias)
                for btag, bb in (("bias", bias), ("nobias", None)):
                    c = torch.zeros(m, n, dtype=dt)
                    smm.scaled_mm(c, a, b, sa, sb, bb)
                    out[f"smm_{tag}_{stag}_{dtag}_{btag}_c"] = _np(c)
    np.savez_compressed(HERE / "scaled_mm.npz", **out)

    # ---- silu_mul_fp8: the reference kernel in the CPU interpreter, and the module's torch reference ----------
    smf = _load(pk / "silu_mul_fp8" / "silu_mul_fp8.py", "ref_silu_mul_fp8")
    out = {}
    torch.manual_seed(44)
    for tag, (t, d, dt, sc) in (("a", (8, 256, torch.bfloat16, 1.0)), ("b", (5, 64, torch.bfloat16, 0.037)),
                                ("c", (3, 128, torch.float16, 2.5))):
        x = (torch.randn(t, 2 * d) * 3).to(dt)
        scale = torch.tensor([sc], dtype=torch.float32)
        out[f"smf_{tag}_x"], out[f"smf_{tag}_scale"] = _np(x), _np(scale)
        out[f"smf_{tag}_kernel"] = _np(smf.silu_mul_fp8(x, scale))
        out[f"smf_{tag}_torch"] = _np(smf._silu_mul_fp8_torch(x, scale))
    np.savez_compressed(HERE / "silu_mul_fp8.npz", **out)

    # ---- the quant producers' KERNELS themselves (CPU interpreter), beside their torch references above --------
    # rms_norm_per_block_quant's kernel does not run in the interpreter (a shape error inside its reference-mode
    # broadcasting); the NVFP4 GEMV / GEMM kernels use loads or a backend the interpreter does not have.
    out = {}
    torch.manual_seed(55)
    x = torch.randn(12, 2 * 256, dtype=torch.bfloat16)
    out["k_silu_x"] = _np(x)
    for gs in (64, 128):
        q = torch.zeros(12, 256, dtype=torch.float8_e4m3fn)
        sc = torch.zeros(12, 256 // gs)
        silu.silu_and_mul_per_block_quant(q, x, sc, gs)
        out[f"k_silu_q_{gs}"], out[f"k_silu_s_{gs}"] = _np(q), _np(sc)
    xr = (torch.randn(12, 384) * torch.logspace(-2, 1, 12)[:, None]).to(torch.bfloat16)
    wr = (torch.rand(384) + 0.5).to(torch.bfloat16)
    res = torch.randn(12, 384).to(torch.bfloat16)
    out["k_rms_x"], out["k_rms_w"], out["k_rms_res"] = _np(xr), _np(wr), _np(res)
    for tag, r in (("", None), ("_res", res.clone())):
        q = torch.zeros(12, 384, dtype=torch.float8_e4m3fn)
        sc = torch.zeros(12, 1)
        rms.rms_norm_dynamic_per_token_quant(q, xr, wr, sc, 1e-6, None, r)
        out[f"k_rms_q{tag}"], out[f"k_rms_s{tag}"] = _np(q), _np(sc)
        if r is not None:
            out["k_rms_newres"] = _np(r)
    q = torch.zeros(12, 384, dtype=torch.float8_e4m3fn)
    sc = torch.zeros(12, 1)
    dyn.dynamic_per_token_scaled_fp8_quant(q, xr, sc, None)
    out["k_dyn_q"], out["k_dyn_s"] = _np(q), _np(sc)
    q = torch.zeros(12, 384, dtype=torch.float8_e4m3fn)
    sc = torch.zeros(12, 3)
    grp.per_token_group_fp8_quant(xr, q, sc, 128, 1e-10, -448.0, 448.0, False)
    out["k_grp_q"], out["k_grp_s"] = _np(q), _np(sc)
    np.savez_compressed(HERE / "reference_kernels.npz", **out)

    # ---- MoE / grouped GEMM references ------------------------------------------------------------
    out = {}
    torch.manual_seed(8)
    a = torch.randn(100, 48, dtype=torch.bfloat16)
    w = torch.randn(7, 48, 40, dtype=torch.bfloat16)
    top1 = torch.randint(7, (100,))
    top1[top1 == 4] = 5  # leave one expert empty
    out["moe_a"], out["moe_w"], out["moe_top1"] = _np(a), _np(w), _np(top1)
    c = moe.moe_matmul_ogs_reference(a, w, top1)
    out["moe_c"] = _np(c)
    args = moe.moe_matmul_ogs_helion_kernel_args_gen(a, w, top1)
    out["moe_counts"], out["moe_offsets"], out["moe_sorted"] = _np(args[2]), _np(args[3]), _np(args[4])
    out["moe_max_t"] = np.int64(args[5])
    np.savez_compressed(HERE / "moe.npz", **out)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    os.environ.setdefault("HELION_INTERPRET", "1")  # kernels called below run in the reference's CPU interpreter
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
