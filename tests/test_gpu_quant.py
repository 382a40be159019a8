"""Bit-level parity of the fused quantisation producers and the NVFP4 quantiser with the oracle."""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn


def bits(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8) if t.element_size() == 1 else t.view(torch.int32)


def count_diff(a: torch.Tensor, b: torch.Tensor) -> int:
    return int((bits(a) != bits(b)).sum())


# ------------------------------------------------------------------ per_token_group_fp8_quant
def run_group(x, gs, ue8m0, eps=1e-10):
    t, h = x.shape
    q = torch.full((t, h), float("nan"), device=DEV).to(FP8)
    s = torch.full((t, h // gs), float("nan"), device=DEV)
    hb.per_token_group_fp8_quant(x.to(DEV), q, s, gs, eps, -448.0, 448.0, ue8m0)
    return q, s


def test_group_quant_golden(golden):
    g = golden("quant_producers.npz")
    x = g.bf16("grp_x")
    for ue in (0, 1):
        q, s = run_group(x, 128, bool(ue))
        assert count_diff(q, g.e4m3(f"grp_q_{ue}")) == 0
        assert count_diff(s, g.raw(f"grp_s_{ue}")) == 0


@pytest.mark.parametrize("t,h,gs", [(1, 2048, 128), (64, 4096, 128), (257, 5120, 128), (33, 1024, 64), (1024, 7168, 128)])
@pytest.mark.parametrize("ue", [False, True])
def test_group_quant_bit_exact(t, h, gs, ue):
    x = (torch.randn(t, h, generator=torch.Generator().manual_seed(2)) * 3).to(torch.bfloat16)
    q, s = run_group(x, gs, ue)
    qo, so = O.per_token_group_fp8_quant(x, gs, 1e-10, -448.0, 448.0, ue)
    assert count_diff(s, so) == 0 and count_diff(q, qo) == 0


def test_group_quant_other_dtypes():
    for dt in (torch.float16, torch.float32):
        x = torch.randn(16, 512, generator=torch.Generator().manual_seed(3)).to(dt)
        q, s = run_group(x, 128, False)
        qo, so = O.per_token_group_fp8_quant(x, 128, 1e-10, -448.0, 448.0, False)
        assert count_diff(s, so) == 0 and count_diff(q, qo) == 0


# ---------------------------------------------------------------- silu_and_mul_per_block_quant
def run_silu(x, gs, ub=None, int8=False):
    t, two_i = x.shape
    q = torch.zeros((t, two_i // 2), device=DEV, dtype=torch.int8 if int8 else FP8)
    s = torch.full((t, two_i // 2 // gs), float("nan"), device=DEV)
    hb.silu_and_mul_per_block_quant(q, x.to(DEV), s, gs, None if ub is None else ub.to(DEV))
    return q, s


def check_silu(x, gs, ub=None):
    """Bit-exact against the oracle evaluated by torch on the same device (the reference's own check runs
    its torch function on the GPU).  The CPU evaluation uses a different exp(): there a scale may move by a
    few units in the last place, and codes may differ only inside groups whose scale moved."""
    q, s = run_silu(x, gs, ub)
    qd, sd = O.silu_and_mul_per_block_quant(x.to(DEV), gs, None if ub is None else ub.to(DEV))
    assert count_diff(s, sd) == 0, f"{count_diff(s, sd)} scales differ from the on-device oracle"
    assert count_diff(q, qd) == 0, f"{count_diff(q, qd)} codes differ from the on-device oracle"
    qc, sc = O.silu_and_mul_per_block_quant(x, gs, ub)
    ds = (bits(s).to(torch.int64) - bits(sc).to(torch.int64)).abs()
    assert int(ds.max()) <= 4, "a scale differs from the CPU oracle by more than four ulp"
    bad_groups = ds.reshape(-1) != 0
    qdiff = (bits(q) != bits(qc)).reshape(-1, gs).any(dim=1)
    # a last-place difference in exp() can also flip a single code that sits on a rounding boundary
    stray = int((bits(q) != bits(qc)).reshape(-1, gs)[~bad_groups].sum())
    assert stray <= max(2, q.numel() // 200000), f"{stray} codes differ from the CPU oracle in groups whose scale matches"
    return int(bad_groups.sum()), int(qdiff.sum())


def test_silu_golden(golden):
    g = golden("quant_producers.npz")
    x = g.bf16("silu_x")
    for gs in (64, 128):
        check_silu(x, gs)
    check_silu(x, 128, g.raw("silu_ub"))


@pytest.mark.parametrize("t,i,gs", [(1, 6144, 128), (8, 12288, 128), (65, 1024, 64), (256, 18432, 128)])
def test_silu_bit_exact(t, i, gs):
    x = torch.randn(t, 2 * i, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    check_silu(x, gs)


def test_silu_strided_input_and_int8():
    x = torch.randn(16, 2 * 256 + 64, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    xv = x.to(DEV)[:, : 2 * 256]  # row stride 576
    q = torch.zeros(16, 256, device=DEV, dtype=FP8)
    s = torch.zeros(16, 2, device=DEV)
    hb.silu_and_mul_per_block_quant(q, xv, s, 128)
    qd, sd = O.silu_and_mul_per_block_quant(xv.contiguous(), 128)
    assert count_diff(q, qd) == 0 and count_diff(s, sd) == 0
    # int8 output: y * (1 / s), rounded half to even, clamped to [-128, 127]; s = max(amax / 127, 2^-23)
    q8, s8 = run_silu(x[:, :512].contiguous(), 128, int8=True)
    xd = x[:, :512].to(DEV).float()
    y = (xd[:, :256] * torch.sigmoid(xd[:, :256]) * xd[:, 256:]).reshape(16, 2, 128)
    sref = (y.abs().amax(-1) * (1.0 / 127.0)).clamp(min=1.1920928955078125e-07)
    qref = (y * (1.0 / sref[:, :, None])).round().clamp(-128, 127).to(torch.int8).reshape(16, 256)
    assert count_diff(s8, sref) == 0 and count_diff(q8, qref) == 0


# ------------------------------------------------------------ rms_norm_dynamic_per_token_quant
def run_rms(x, w, eps, ub=None, res=None):
    t, h = x.shape
    q = torch.zeros((t, h), device=DEV, dtype=FP8)
    s = torch.full((t, 1), float("nan"), device=DEV)
    res_d = None if res is None else res.to(DEV).clone()
    hb.rms_norm_dynamic_per_token_quant(q, x.to(DEV), w.to(DEV), s, eps, None if ub is None else ub.to(DEV), res_d)
    return q, s, res_d


def check_rms(x, w, eps, ub=None, res=None):
    """Rows must equal the oracle bit for bit, or equal the oracle with that row's fp32 rms moved by at most
    two units in the last place (the sum of squares is order dependent; nothing else in the chain is)."""
    q, s, res_d = run_rms(x, w, eps, ub, res)
    qo, so, reso = O.rms_norm_dynamic_per_token_quant(x, w, eps, ub, res)
    if res is not None:
        assert count_diff(res_d, reso) == 0
    row_bad = (bits(q) != bits(qo)).any(dim=1) | (bits(s) != bits(so)).reshape(-1)
    unexplained = row_bad.clone()
    for nudge in (-1, 1, -2, 2):
        if not unexplained.any():
            break
        qn, sn, _ = O.rms_norm_dynamic_per_token_quant(
            x, w, eps, ub, res, rms_ulp_nudge=torch.full((x.shape[0],), nudge, dtype=torch.int32)
        )
        ok = ~((bits(q) != bits(qn)).any(dim=1) | (bits(s) != bits(sn)).reshape(-1))
        unexplained &= ~ok
    assert not unexplained.any(), f"{int(unexplained.sum())} rows differ beyond a 2-ulp change of rms"
    return int(row_bad.sum()), int((bits(q) != bits(qo)).sum())


def test_rms_golden(golden):
    g = golden("quant_producers.npz")
    x, w = g.bf16("rms_x"), g.bf16("rms_w")
    check_rms(x, w, 1e-6)
    check_rms(x, w, 1e-6, torch.tensor(2.0), g.bf16("rms_res_in"))


@pytest.mark.parametrize("t,h", [(1, 2048), (17, 4096), (64, 5120), (128, 7168), (4, 16384), (3, 136)])
def test_rms_against_oracle(t, h):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    w = (torch.rand(h, generator=g) + 0.5).to(torch.bfloat16)
    rows, codes = check_rms(x, w, 1e-6)
    assert codes <= max(4, t * h // 100000), f"{codes} codes in {rows} rows differ from the CPU oracle"


def test_rms_fp16_input():
    g = torch.Generator().manual_seed(8)
    x = torch.randn(8, 1024, generator=g).to(torch.float16)
    w = (torch.rand(1024, generator=g) + 0.5).to(torch.float16)
    check_rms(x, w, 1e-6)


# --------------------------------------------------------------------------- NVFP4 quantiser
@pytest.mark.parametrize("rows,k", [(1, 4096), (130, 80), (256, 1536), (77, 4096), (8, 28672)])
@pytest.mark.parametrize("per_token", [False, True])
def test_nvfp4_quantiser_bit_exact(rows, k, per_token):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, k, generator=g).to(torch.bfloat16)
    if rows > 2:
        x[1] = 0  # an all-zero row
        x[2, :16] = 0  # an all-zero block
    if per_token:
        codes, scales, gs = hb.nvfp4_quantize(x.to(DEV))
        co, so, go = O.nvfp4_quantize(x, per_token=True)
    else:
        gt = O.nvfp4_quantize(x)[2]
        codes, scales, gs = hb.nvfp4_quantize(x.to(DEV), gt.to(DEV))
        co, so, go = O.nvfp4_quantize(x, gt)
    assert count_diff(gs.reshape(-1), go.reshape(-1)) == 0
    assert count_diff(scales, so) == 0
    assert count_diff(codes, co) == 0


def test_nvfp4_quantiser_tie_cases():
    """Values exactly on a rounding boundary go to the smaller magnitude (not to even)."""
    vals = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -2.5, -5.0, -6.0, 0.0, -0.0, 3.0])
    x = vals.to(torch.bfloat16).reshape(1, 16)
    g = torch.tensor(1.0 / 448.0 / 6.0 * 6.0)  # block scale (6/6)/g = 448 -> decoded scale * g = 1
    g = torch.tensor(1.0 / 448.0)
    codes, scales, _ = hb.nvfp4_quantize(x.to(DEV), g.to(DEV))
    co, so, _ = O.nvfp4_quantize(x, g)
    assert count_diff(codes, co) == 0 and count_diff(scales, so) == 0
