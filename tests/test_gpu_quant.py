"""Bit-level parity of the fused quantisation producers and the NVFP4 quantiser with the oracle."""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from oracle import checks as C
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


def test_group_quant_with_tiny_eps_and_tiny_groups_or_other_limits():
    """Scales below 2^-60 (tiny eps, tiny values: the kernel moves such a group up by 2^64 before its short
    division) and limits other than the format's own (the kernel then clamps explicitly)."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(32, 1024, generator=g)
    x[:16] *= 1e-30
    x[16:24] *= 1e-36
    x[8, :128] = 0.0
    x[8, 5] = 1e-38
    for dt in (torch.bfloat16, torch.float32):
        xs = x.to(dt)
        q, s = run_group(xs, 128, False, eps=1e-44)
        qo, so = O.per_token_group_fp8_quant(xs, 128, 1e-44, -448.0, 448.0, False)
        assert count_diff(s, so) == 0 and count_diff(q, qo) == 0
    xs = (x[24:] * 3).to(torch.bfloat16)
    q = torch.zeros(8, 1024, device=DEV).to(FP8)
    s = torch.zeros(8, 8, device=DEV)
    hb.per_token_group_fp8_quant(xs.to(DEV), q, s, 128, 1e-10, -200.0, 240.0, False)
    qo, so = O.per_token_group_fp8_quant(xs, 128, 1e-10, -200.0, 240.0, False)
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


@pytest.mark.parametrize("dt", [torch.float16, torch.float32])
def test_silu_other_input_types(dt):
    """The reference converts any float input to fp32 first (silu_and_mul_per_block_quant.py:99-107)."""
    x = torch.randn(33, 2 * 1024, generator=torch.Generator().manual_seed(6)).to(dt)
    check_silu(x, 128)
    check_silu(x, 64, torch.tensor(0.75))


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
    rep = C.rms_quant_report(x, w, eps, q, s, ub, res)
    assert rep["rows_not_explained_by_2ulp_of_rms"] == 0, rep
    return rep["rows_differing"], rep["codes_differing"]


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


def test_nvfp4_quantiser_code_rule_on_every_bf16_value_up_to_six():
    """Every bf16 value in [-6, 6] (both zeros, denormals, every tie and its neighbours), fifteen per block beside
    a 6.0 that pins the block's decoded scale to one: the codes are the oracle's.  Blocks that hold a tie or -0.0
    take the kernel's slow path group by group, all others the hardware conversion."""
    bits = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16)
    every = bits.view(torch.bfloat16)
    vals = every[torch.isfinite(every.float()) & (every.float().abs() <= 6.0)]
    pad = (-vals.numel()) % (15 * 8)  # whole rows of eight blocks; the filler repeats the first values
    vals = torch.cat([vals, vals[:pad]])
    x = torch.cat([vals.reshape(-1, 15), torch.full((vals.numel() // 15, 1), 6.0, dtype=torch.bfloat16)], dim=1)
    x = x.reshape(-1, 8 * 16).contiguous()  # eight blocks per row
    g = torch.tensor(1.0 / 448.0)
    codes, scales, _ = hb.nvfp4_quantize(x.to(DEV), g.to(DEV))
    co, so, _ = O.nvfp4_quantize(x, g)
    assert count_diff(scales, so) == 0
    assert count_diff(codes, co) == 0


# ------------------------------------------------------------------ sibling producers
def run_dyn(x, ub=None):
    t, h = x.shape
    q = torch.zeros((t, h), device=DEV, dtype=FP8)
    s = torch.full((t, 1), float("nan"), device=DEV)
    hb.dynamic_per_token_scaled_fp8_quant(q, x.to(DEV), s, None if ub is None else ub.to(DEV))
    return q, s


def test_dynamic_per_token_golden(golden):
    g = golden("quant_siblings.npz")
    x = g.bf16("dyn_x")
    q, s = run_dyn(x)
    assert count_diff(q, g.e4m3("dyn_q")) == 0 and count_diff(s, g.raw("dyn_s")) == 0
    q, s = run_dyn(x, torch.tensor(0.01))
    assert count_diff(q, g.e4m3("dyn_q_ub")) == 0 and count_diff(s, g.raw("dyn_s_ub")) == 0


@pytest.mark.parametrize("t,h", [(1, 8), (7, 520), (64, 7168), (33, 4096), (5, 32768), (300, 1024)])
def test_dynamic_per_token_bit_exact(t, h):
    g = torch.Generator().manual_seed(t + h)
    x = (torch.randn(t, h, generator=g) * torch.logspace(-2, 2, t)[:, None]).to(torch.bfloat16)
    q, s = run_dyn(x)
    qo, so = O.dynamic_per_token_scaled_fp8_quant(x)
    assert count_diff(q, qo) == 0 and count_diff(s, so) == 0
    q, s = run_dyn(x.to(torch.float16))
    qo, so = O.dynamic_per_token_scaled_fp8_quant(x.to(torch.float16))
    assert count_diff(q, qo) == 0 and count_diff(s, so) == 0


def run_rms_block(x, w, eps, gs, ub=None, res=None, transposed=False, int8=False):
    t, h = x.shape
    q = torch.zeros((t, h), device=DEV, dtype=torch.int8 if int8 else FP8)
    if transposed:
        s = torch.full((h // gs, t), float("nan"), device=DEV).t()
    else:
        s = torch.full((t, h // gs), float("nan"), device=DEV)
    res_d = None if res is None else res.to(DEV).clone()
    hb.rms_norm_per_block_quant(q, x.to(DEV), w.to(DEV), s, eps, None if ub is None else ub.to(DEV), res_d, gs, transposed)
    return q, s, res_d


def test_rms_per_block_golden(golden):
    g = golden("quant_siblings.npz")
    x, w, res = g.bf16("rpb_x"), g.bf16("rpb_w"), g.bf16("rpb_res")
    for gs in (64, 128):
        q, s, _ = run_rms_block(x, w, 1e-6, gs)
        assert count_diff(q, g.e4m3(f"rpb_q_{gs}")) <= 2 and count_diff(s, g.raw(f"rpb_s_{gs}")) <= 1
        q, s, r = run_rms_block(x, w, 1e-6, gs, None, res, transposed=True)
        assert count_diff(q, g.e4m3(f"rpb_q_{gs}_res")) <= 2 and count_diff(s.contiguous(), g.raw(f"rpb_s_{gs}_res")) <= 1
        assert count_diff(r, g.bf16(f"rpb_newres_{gs}")) == 0


@pytest.mark.parametrize("t,h,gs", [(3, 64, 64), (17, 1024, 128), (64, 7168, 128), (9, 4096, 64), (4, 32768, 128)])
def test_rms_per_block_against_oracle(t, h, gs):
    """Rows equal the oracle bit for bit, or the oracle with that row's fp32 rms moved by <= 2 ulp."""
    g = torch.Generator().manual_seed(h + gs)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    w = (torch.rand(h, generator=g) + 0.5).to(torch.bfloat16)
    q, s, _ = run_rms_block(x, w, 1e-6, gs)
    qo, so, _ = O.rms_norm_per_block_quant(x, w, 1e-6, gs)
    bad = (bits(q) != bits(qo)).any(dim=1) | (bits(s) != bits(so)).any(dim=1)
    for nudge in (-1, 1, -2, 2):
        if not bad.any():
            break
        qn, sn, _ = O.rms_norm_per_block_quant(x, w, 1e-6, gs, None, None, torch.full((t,), nudge, dtype=torch.int32))
        bad &= (bits(q) != bits(qn)).any(dim=1) | (bits(s) != bits(sn)).any(dim=1)
    assert not bad.any(), f"{int(bad.sum())} rows differ beyond a 2-ulp change of rms"
    # int8 output (the Helion kernel's rule, rms_norm_per_block_quant.py:84-90,125-128): scale = amax * (1/127)
    # floored at fp32 eps, codes = round(x_norm * (1 / scale)).  A row whose rms moved by an ulp may differ.
    qi, si, _ = run_rms_block(x, w, 1e-6, gs, int8=True)
    xf = x.float()
    rms = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + 1e-6)
    normed = ((xf * rms).to(torch.bfloat16) * w[None, :]).float().reshape(t, h // gs, gs)
    se = (normed.abs().amax(dim=-1) * (1.0 / 127)).clamp(min=1.1920928955078125e-07)
    qe = (normed * (1.0 / se[:, :, None])).round().clamp(-128, 127).to(torch.int8).reshape(t, h)
    assert qi.dtype is torch.int8
    assert float((qi.cpu() != qe).float().mean()) <= 2e-3
    assert torch.allclose(si.cpu(), se, rtol=1e-5, atol=0)


def _silu_mul_fp8_on_device(x, scale):
    """The reference function evaluated by torch on the GPU, with the saturating conversion of the compiled kernel."""
    d = x.shape[-1] // 2
    r = (torch.nn.functional.silu(x[..., :d]) * x[..., d:]).to(torch.float32)
    return (r * (1.0 / scale.reshape(()))).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def test_silu_mul_fp8_golden(golden):
    g = golden("silu_mul_fp8.npz")
    for tag, dt in (("a", torch.bfloat16), ("b", torch.bfloat16), ("c", torch.float16)):
        x = g.raw(f"smf_{tag}_x").view(dt).to(DEV)
        scale = g.raw(f"smf_{tag}_scale").to(DEV)
        ref = g.e4m3(f"smf_{tag}_kernel")
        got = hb.silu_mul_fp8(x, scale).cpu()
        overflow = torch.isnan(ref.float())
        same = got.view(torch.uint8)[~overflow] == ref.view(torch.uint8)[~overflow]
        # exp() on the device may differ from the CPU's in the last place: at most a code or two may move
        assert float(same.float().mean()) >= 0.995
        assert bool((got.float()[overflow].abs() == 448.0).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens,d", [(1, 2048), (8, 2880), (33, 4096), (256, 14336), (3, 8), (0, 64)])
def test_silu_mul_fp8_matches_torch_on_device(tokens, d, dtype):
    g = torch.Generator(device=DEV).manual_seed(tokens + d)
    x = (torch.randn(tokens, 2 * d, device=DEV, generator=g) * 2).to(dtype)
    for sc in (1.0, 0.05, 3.0):
        scale = torch.tensor([sc], device=DEV)
        got = hb.silu_mul_fp8(x, scale)
        assert got.shape == (tokens, d) and got.dtype is torch.float8_e4m3fn
        want = _silu_mul_fp8_on_device(x, scale)
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    torch.cuda.synchronize()


def test_silu_mul_fp8_shapes_and_errors():
    x = torch.randn(2, 3, 64, device=DEV).to(torch.bfloat16)
    scale = torch.tensor(0.5, device=DEV)
    y = hb.silu_mul_fp8(x, scale)
    assert y.shape == (2, 3, 32)
    assert torch.equal(y.view(torch.uint8).reshape(6, 32), _silu_mul_fp8_on_device(x.reshape(6, 64), scale).view(torch.uint8))
    wide = torch.randn(4, 160, device=DEV).to(torch.bfloat16)
    assert torch.equal(hb.silu_mul_fp8(wide[:, :128], scale).view(torch.uint8),
                       _silu_mul_fp8_on_device(wide[:, :128], scale).view(torch.uint8))
    with pytest.raises(AssertionError):
        hb.silu_mul_fp8(x, torch.ones(2, device=DEV))
    with pytest.raises(ValueError):
        hb.silu_mul_fp8(torch.zeros(2, 24, device=DEV, dtype=torch.bfloat16), scale)
    with pytest.raises(TypeError):
        hb.silu_mul_fp8(torch.zeros(2, 32, device=DEV), scale)


def test_against_outputs_of_the_reference_kernels(golden):
    """CUDA kernels against what the reference's own kernels wrote (reference CPU interpreter, tests/golden), with
    exact mismatch counts.  SiLU-mul: the CPU's exp() differs from the GPU's in the last place, so block scales may
    move by a few ulp and single codes with them; what explains a mismatch is that the kernel equals, bit for bit,
    the reference function evaluated by torch on this GPU (the reference's own correctness protocol,
    pretuned_kernels/silu_and_mul_per_block_quant/silu_and_mul_per_block_quant.py:197-216).  RMSNorm: a row differs
    only where its fp32 rms moved by at most two ulp (summation order)."""
    g = golden("reference_kernels.npz")
    x = g.bf16("k_silu_x").to(DEV)
    for gs in (64, 128):
        q = torch.empty(12, 256, dtype=torch.float8_e4m3fn, device=DEV)
        s = torch.empty(12, 256 // gs, device=DEV)
        hb.silu_and_mul_per_block_quant(q, x, s, gs)
        qd, sd = O.silu_and_mul_per_block_quant(x, gs)  # the same function, evaluated on the device
        assert count_diff(q, qd) == 0 and count_diff(s, sd) == 0
        codes_off = int((q.cpu().view(torch.uint8) != g.raw(f"k_silu_q_{gs}")).sum())
        scales_off = int((bits(s) != bits(g.raw(f"k_silu_s_{gs}"))).sum())
        print(f"silu gs={gs}: {codes_off} of {q.numel()} codes and {scales_off} of {s.numel()} scales differ from the CPU run")
        torch.testing.assert_close(s.cpu(), g.raw(f"k_silu_s_{gs}"), rtol=1e-6, atol=0)
        assert codes_off <= 16  # of 3072
    xr = g.bf16("k_rms_x").to(DEV)
    q = torch.empty(12, 384, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.empty(12, 1, device=DEV)
    hb.dynamic_per_token_scaled_fp8_quant(q, xr, s)
    assert torch.equal(q.cpu().view(torch.uint8), g.raw("k_dyn_q")) and torch.equal(s.cpu(), g.raw("k_dyn_s"))
    w = g.bf16("k_rms_w").to(DEV)
    hb.rms_norm_dynamic_per_token_quant(q, xr, w, s, 1e-6)
    # the oracle reproduces the reference kernel's output bit for bit, so the row-wise explanation applies to it
    qo, so, _ = O.rms_norm_dynamic_per_token_quant(xr.cpu(), w.cpu(), 1e-6)
    assert torch.equal(qo.view(torch.uint8), g.raw("k_rms_q")) and torch.equal(so, g.raw("k_rms_s"))
    rep = C.rms_quant_report(xr, w, 1e-6, q, s)
    print("rms against the reference kernel's output:", rep)
    assert rep["rows_not_explained_by_2ulp_of_rms"] == 0


# ------------------------------------------------------------------ fused NVFP4 producers
def _unswizzle_bytes(s, rows, cols):
    return O.unswizzle_scales(s.cpu(), rows, cols).view(torch.uint8)


@pytest.mark.parametrize("t,h", [(3, 256), (130, 2048), (64, 4096), (17, 7168), (4, 16384)])
def test_rms_norm_nvfp4_quant_against_the_oracle(t, h):
    """RMSNorm -> per-token NVFP4 in one kernel against the oracle's two steps (the normalisation of
    rms_norm_dynamic_per_token_quant, then the NVFP4 quantiser).  A row must match bit for bit, or match with its
    fp32 rms moved by at most two units in the last place (summation order)."""
    g = torch.Generator().manual_seed(t + h)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    w = (torch.rand(h, generator=g) + 0.5).to(torch.bfloat16)
    codes, scales, gs = hb.rms_norm_nvfp4_quant(x.to(DEV), w.to(DEV), 1e-6)
    torch.cuda.synchronize()
    codes, sc, gs = codes.cpu(), _unswizzle_bytes(scales, t, h // 16), gs.cpu()
    left = torch.ones(t, dtype=torch.bool)
    for nudge in (0, -1, 1, -2, 2):
        rms = O.rms_norm_row_rms(x, 1e-6)
        rms = (rms.view(torch.int32) + nudge).view(torch.float32)
        normed = (x.float() * rms).to(torch.bfloat16) * w[None, :]
        oc, osc, og = O.nvfp4_quantize(normed, per_token=True)
        ok = (codes == oc).all(dim=1) & (sc == _unswizzle_bytes(osc, t, h // 16)).all(dim=1) & (gs == og)
        left &= ~ok
        if not left.any():
            break
    assert not left.any(), f"{int(left.sum())} of {t} rows differ beyond a 2-ulp change of rms"


@pytest.mark.parametrize("t,d", [(5, 256), (200, 1536), (33, 4096)])
def test_silu_and_mul_nvfp4_quant_against_the_oracle(t, d):
    """SiLU-mul -> per-token NVFP4 in one kernel: y is pinned bit for bit to the reference function evaluated by
    torch on this device (exp() differs from the CPU's in the last place), the quantiser to the oracle's."""
    g = torch.Generator().manual_seed(t + d)
    x = torch.randn(t, 2 * d, generator=g).to(torch.bfloat16).to(DEV)
    codes, scales, gs = hb.silu_and_mul_nvfp4_quant(x)
    xf = x.float()
    y = (xf[:, :d] / (1.0 + torch.exp(-xf[:, :d])) * xf[:, d:]).to(torch.bfloat16)  # on the device
    oc, osc, og = O.nvfp4_quantize(y.cpu(), per_token=True)
    assert torch.equal(codes.cpu(), oc) and torch.equal(gs.cpu(), og)
    assert torch.equal(_unswizzle_bytes(scales, t, d // 16), _unswizzle_bytes(osc, t, d // 16))
    # and it is what the separate quantiser makes of the same y
    c2, s2, g2 = hb.nvfp4_quantize(y)
    assert torch.equal(codes, c2) and torch.equal(gs, g2) and torch.equal(scales.view(torch.uint8), s2.view(torch.uint8))


def test_fused_nvfp4_producers_feed_the_gemv():
    """The producers' outputs are the activation operand of the NVFP4 GEMV: RMSNorm -> NVFP4 -> W4A4 GEMV equals
    the oracle GEMV on the oracle-quantised normalised row."""
    g = torch.Generator().manual_seed(7)
    n, k = 512, 2048
    x = torch.randn(1, k, generator=g).to(torch.bfloat16)
    w_norm = (torch.rand(k, generator=g) + 0.5).to(torch.bfloat16)
    wp, ws, wg = O.nvfp4_quantize(torch.randn(n, k, generator=g) * 0.02)
    codes, scales, gs = hb.rms_norm_nvfp4_quant(x.to(DEV), w_norm.to(DEV), 1e-6)
    alpha = float(wg) * float(gs[0])
    y = hb.nvfp4_gemv_fp4in(wp.to(DEV), codes.reshape(-1), ws.to(DEV), scales, alpha)
    ref = O.nvfp4_gemv_fp4in(wp, codes.reshape(-1).cpu(), ws, scales.cpu(), alpha)
    yc, rc = y.float().cpu(), ref.float()
    floor = rc.pow(2).mean().sqrt()
    assert float(((yc - rc).abs() / torch.maximum(rc.abs(), floor)).max()) <= 1e-2


def test_silu_scales_may_be_a_transposed_view():
    """The reference writes scales by index, so a transposed (column-major) scale tensor works there."""
    x = torch.randn(24, 2 * 512, generator=torch.Generator().manual_seed(13)).to(torch.bfloat16).to(DEV)
    q = torch.empty(24, 512, dtype=FP8, device=DEV)
    s_t = torch.empty(4, 24, device=DEV).t()  # [24, 4] with strides (1, 24)
    assert not s_t.is_contiguous()
    hb.silu_and_mul_per_block_quant(q, x, s_t, 128, None, True)
    qd, sd = O.silu_and_mul_per_block_quant(x, 128)
    assert count_diff(q, qd) == 0 and torch.equal(s_t, sd)



def test_short_reciprocal_and_division_are_exact_on_their_whole_range():
    """The producers replace the general reciprocal / division by a two-FMA Newton step and a one-step exact
    quotient where the divisor is known to lie in [2^-100, 2^125]: every fp32 divisor of that range gives the IEEE
    reciprocal, and four numerators per divisor (7.6e9 pairs) the IEEE quotient."""
    from helion_b200 import _lib

    bad = torch.full((3,), -1, dtype=torch.int64, device=DEV)
    _lib.call("hb200_selftest_exact_reciprocal", bad.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert bad.tolist() == [0, 0, 0], f"reciprocals / one-step / two-step quotients that differ: {bad.tolist()}"


def test_silu_producers_on_extreme_gate_values():
    """Gate values beyond +-86 (where 1 + exp(-a) leaves the short reciprocal's range), denormal-sized values and
    zeros of both signs take the general path or the exact corner of the short one, and still equal torch on the
    device bit for bit.  (The up values beside them are small so that no product overflows into a NaN, whose fp8
    sign bit is nobody's contract.)"""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(8, 2 * 256, generator=g).to(torch.bfloat16)
    special = torch.tensor([-86.0, -87.0, -88.5, -100.0, -3e38, 86.0, 90.0, 3e38, 0.0, -0.0, 1e-30, -1e-30, 1e-38, -1e-38,
                            -85.5, 85.5], dtype=torch.bfloat16)
    for r in range(8):
        x[r, r * 16 : r * 16 + 16] = special  # one group with specials per row, the other groups plain
        x[r, 256 + r * 16 : 256 + r * 16 + 16] = 0.001
    check_silu(x, 128)
    check_silu(x, 64)
    scale = torch.tensor([0.5], device=DEV)
    x[0, 3] = float("inf")  # silu(inf) = inf: saturates to 448
    got = hb.silu_mul_fp8(x.to(DEV), scale)
    assert torch.equal(got.view(torch.uint8), _silu_mul_fp8_on_device(x.to(DEV), scale).view(torch.uint8))
