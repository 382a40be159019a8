"""scaled_mm (row-wise scaled FP8 GEMM) against the reference kernel's golden outputs and the oracle."""

from __future__ import annotations

import math

import pytest
import torch

import helion_b200 as hb
from helion_b200 import _lib
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn
ULP = {torch.bfloat16: 2.0**-8, torch.float16: 2.0**-11, torch.float32: 2.0**-20}


def device_status_ok():
    torch.cuda.synchronize()
    return _lib.load().hb200_device_status(1) == 0


ACC_SLACK = 2.0**-13  # of sum |a||b|: what the tensor core's fp32 accumulation of FP8 products may lose


def close_to_oracle(got, ref, bias, slack):
    """Within one place of the output type at the larger of result and bias, plus the accumulation slack."""
    assert got.dtype == ref.dtype and got.shape == ref.shape
    ulp = ULP[ref.dtype]
    got, ref = got.float().cpu(), ref.float().cpu()
    assert torch.isfinite(got).all()
    mag = ref.abs() if bias is None else torch.maximum(ref.abs(), bias.float().cpu().abs()[None, :])
    return bool(((got - ref).abs() <= 1.01 * ulp * mag + slack + 1e-30).all())


def check(got, a, b, sa, sb, bias):
    a, b, sa, sb = a.cpu(), b.cpu(), sa.cpu(), sb.cpu()
    ref = O.scaled_mm(a, b, sa, sb, None if bias is None else bias.cpu(), got.dtype)
    sums = O.scaled_mm(a.float().abs().to(a.dtype), b.float().abs().to(b.dtype), sa, sb, None, torch.float32)
    assert close_to_oracle(got, ref, bias, ACC_SLACK * sums)


def random_case(m, k, n, seed, fp8=FP8, signed=True):
    g = torch.Generator().manual_seed(seed)
    scale = 1.0 / math.sqrt(k)
    shift = 0.5 if signed else -0.5
    a = (scale * (torch.rand(m, k, generator=g) - shift + 0.0)).to(fp8)
    b = (scale * (torch.rand(n, k, generator=g) - shift)).to(fp8).t()
    return a.to(DEV), b.to(DEV), g


def test_golden_outputs_of_the_reference_kernel(golden):
    g = golden("scaled_mm.npz")
    for tag in "abc":
        a, b = g.e4m3(f"smm_{tag}_a").to(DEV), g.e4m3(f"smm_{tag}_b_nk").to(DEV).t()
        for stag in ("tensor", "rows", "mixed"):
            sa, sb = g.raw(f"smm_{tag}_{stag}_sa").to(DEV), g.raw(f"smm_{tag}_{stag}_sb").to(DEV)
            for dtag in ("bf16", "f16", "f32"):
                bias = g.typed(f"smm_{tag}_{stag}_{dtag}_bias", dtag).to(DEV)
                for btag, bb in (("bias", bias), ("nobias", None)):
                    ref = g.typed(f"smm_{tag}_{stag}_{dtag}_{btag}_c", dtag)
                    c = torch.full(ref.shape, float("nan"), dtype=ref.dtype, device=DEV)
                    hb.scaled_mm(c, a, b, sa, sb, bb)
                    assert close_to_oracle(c, ref, bb, 2.0**-18 * ref.float().abs().max()), (tag, stag, dtag, btag)
    assert device_status_ok()


@pytest.mark.parametrize("m,k,n", [(16, 4096, 4096), (64, 2048, 2048)])
def test_the_reference_tests_own_cases(m, k, n):
    """test/test_pretuned_kernels.py:400-422: positive operands, per-tensor scales, bias, atol = rtol = 1e-1."""
    a, b, g = random_case(m, k, n, seed=m, signed=False)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    sa = (torch.rand(1, 1, generator=g) + 0.5).to(DEV)
    sb = (torch.rand(1, 1, generator=g) + 0.5).to(DEV)
    bias = (torch.rand(n, generator=g) - 0.5).to(torch.bfloat16).to(DEV)
    hb.scaled_mm(c, a, b, sa, sb, bias)
    assert device_status_ok()
    ref = ((a.float() @ b.float()) * sa * sb).to(torch.bfloat16) + bias
    torch.testing.assert_close(c, ref, atol=1e-1, rtol=1e-1)
    check(c, a, b, sa, sb, bias)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,k,n", [
    (1, 512, 256), (16, 2048, 2048), (17, 1040, 200), (64, 6144, 2048), (100, 208, 1000), (256, 1024, 512),
    (300, 512, 384), (1000, 256, 640), (48, 64, 130), (33, 16, 128),
])
def test_shapes_scales_and_output_types(m, k, n, out_dtype):
    a, b, g = random_case(m, k, n, seed=m + k + n)
    sa = (torch.rand(m, 1, generator=g) + 0.5).to(DEV)
    sb = (torch.rand(n, generator=g) + 0.5).to(DEV)
    bias = (torch.rand(n, generator=g) - 0.5).to(out_dtype).to(DEV)
    c = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    hb.scaled_mm(c, a, b, sa, sb, bias)
    assert device_status_ok()
    check(c, a, b, sa, sb, bias)
    c2 = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    hb.scaled_mm(c2, a, b, sa[:1], sb[:1], None)  # per-tensor scales, no bias
    assert device_status_ok()
    check(c2, a, b, sa[:1], sb[:1], None)


@pytest.mark.parametrize("m,k,n,shared_workspace", [
    (16, 8192, 1024, False),  # 8 weight tiles: one thread-block cluster per tile, K split across its CTAs
    (64, 4096, 4096, False),
    (16, 8192, 8192, False),  # 64 tiles, two CTAs each
    (64, 2048, 12288, False), # 96 tiles: nearly one per SM, whole tiles
    (16, 4096, 24576, True),  # 192 tiles: stream-K ranges, shared tiles summed through the workspace
    (64, 5120, 10240, True),
])
def test_split_k_is_deterministic(m, k, n, shared_workspace):
    lib = _lib.load()
    assert (lib.hb200_fp8_scaled_mm_workspace_bytes(m, n, k) > 16384) == shared_workspace
    a, b, g = random_case(m, k, n, seed=5)
    sa = (torch.rand(m, 1, generator=g) + 0.5).to(DEV)
    sb = (torch.rand(n, 1, generator=g) + 0.5).to(DEV)
    bias = (torch.rand(n, generator=g) - 0.5).to(torch.bfloat16).to(DEV)
    outs = []
    for _ in range(4):
        c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        hb.scaled_mm(c, a, b, sa, sb, bias)
        outs.append(c)
    assert device_status_ok()
    check(outs[0], a, b, sa, sb, bias)
    for c in outs[1:]:
        assert torch.equal(c, outs[0])  # which also shows the arrival counters were left clear


def test_e5m2_operands_strided_inputs_and_padded_output():
    m, k, n = 24, 512, 320
    a, b, g = random_case(m, k, n, seed=9, fp8=torch.float8_e5m2)
    sa, sb = torch.full((1,), 0.75, device=DEV), torch.full((1,), 1.5, device=DEV)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    hb.scaled_mm(c, a, b, sa, sb, None)
    check(c, a, b, sa, sb, None)
    # rows of a and of the stored weight with a pitch above K, output rows with a pitch above N
    a8, b8, _ = random_case(m, k, n, seed=10)
    a_wide = torch.zeros(m, k + 64, dtype=FP8, device=DEV)
    a_wide[:, :k] = a8
    w_wide = torch.zeros(n, k + 32, dtype=FP8, device=DEV)
    w_wide[:, :k] = b8.t()
    c_wide = torch.full((m, n + 8), float("nan"), dtype=torch.bfloat16, device=DEV)
    hb.scaled_mm(c_wide[:, :n], a_wide[:, :k], w_wide[:, :k].t(), sa, sb, None)
    assert device_status_ok()
    check(c_wide[:, :n], a8, b8, sa, sb, None)
    assert torch.isnan(c_wide[:, n:]).all()


def test_the_reference_assertions_and_the_abi_errors():
    a, b, _ = random_case(16, 256, 128, seed=1)
    c = torch.empty(16, 128, dtype=torch.bfloat16, device=DEV)
    one = torch.ones(1, device=DEV)
    with pytest.raises(AssertionError):
        hb.scaled_mm(c, a, b.t().contiguous().t().contiguous(), one, one)  # b must be K-major
    with pytest.raises(AssertionError):
        hb.scaled_mm(c, a, b, torch.ones(3, device=DEV), one)
    with pytest.raises(AssertionError):
        hb.scaled_mm(c, a, b, one, one, torch.zeros(128, dtype=torch.float16, device=DEV))
    with pytest.raises(TypeError):
        hb.scaled_mm(c, a.view(torch.uint8), b.view(torch.uint8), one, one)
    lib = _lib.load()
    m, k, n = 16, 4096, 24576
    a, b, _ = random_case(m, k, n, seed=2)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    args = (a.data_ptr(), b.t().data_ptr(), c.data_ptr(), one.data_ptr(), one.data_ptr(), None, m, n, k, k, k, n,
            0, 0, 0, 0)
    assert lib.hb200_fp8_scaled_mm(*args, None, 0, None) == _lib.HB200_ERR_WORKSPACE
    small = torch.zeros(32768, dtype=torch.uint8, device=DEV)
    assert lib.hb200_fp8_scaled_mm(*args, small.data_ptr(), small.numel(), None) == _lib.HB200_ERR_WORKSPACE
    bad = (a.data_ptr() + 8, *args[1:])
    assert lib.hb200_fp8_scaled_mm(*bad, None, 0, None) == _lib.HB200_ERR_UNSUPPORTED
    torch.cuda.synchronize()
    assert torch.isnan(c).all()  # nothing ran


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,k,n", [
    (1, 512, 256), (16, 2048, 2048), (17, 1040, 200), (64, 6144, 2048), (256, 1024, 512), (300, 512, 384), (33, 16, 128),
    (16, 8192, 1024),   # thread-block clusters, K split across their CTAs: int32 partial sums through shared memory
    (64, 2048, 12288),  # whole tiles
    (16, 4096, 24576),  # stream-K ranges: int32 partial sums through the workspace
    (64, 25600, 5120),  # sums beyond 2^24: the single conversion to fp32 rounds
])
def test_int8_operands_accumulate_in_int32_bit_exact(m, k, n, out_dtype):
    """The integer form (pretuned_kernels/scaled_mm/scaled_mm.py:53): int32 accumulation is exact, so the result is
    the oracle's, bit for bit, whatever the split of the K range."""
    g = torch.Generator().manual_seed(m + k + n)
    a = torch.randint(-128, 128, (m, k), dtype=torch.int8, generator=g)
    b = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=g).t()
    if k >= 25600:
        a, b = a.abs().clamp(max=127).to(torch.int8), b.abs().clamp(max=127).to(torch.int8)  # large same-sign sums
    sa = (torch.rand(m, 1, generator=g) + 0.5) * 1e-3
    sb = (torch.rand(n, generator=g) + 0.5) * 1e-3
    bias = (torch.rand(n, generator=g) - 0.5).to(out_dtype)
    for s_a, s_b, bb in ((sa, sb, bias), (sa[:1], sb[:1], None)):
        c = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
        hb.scaled_mm(c, a.to(DEV), b.to(DEV), s_a.to(DEV), s_b.to(DEV), None if bb is None else bb.to(DEV))
        assert device_status_ok()
        ref = O.scaled_mm(a, b, s_a, s_b, bb, out_dtype)
        assert torch.equal(c.cpu(), ref)


def test_int8_and_fp8_operands_must_not_be_mixed():
    a = torch.zeros(16, 64, dtype=torch.int8, device=DEV)
    b = torch.zeros(32, 64, dtype=FP8, device=DEV).t()
    c = torch.empty(16, 32, dtype=torch.bfloat16, device=DEV)
    one = torch.ones(1, device=DEV)
    with pytest.raises(AssertionError):
        hb.scaled_mm(c, a, b, one, one)


PREFILL = [(384, 512, 256), (1000, 1040, 520), (2048, 4096, 1024), (513, 208, 1000), (4096, 2048, 2304), (640, 144, 130)]


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,k,n", PREFILL)
def test_prefill_shapes_on_cta_pairs(m, k, n, out_dtype):
    """From 384 tokens on the activations ride the M side of 256 x 256 CTA-pair tiles; ragged M, N and K edges, and
    an output pitch the TMA stores cannot take (n = 130: the decode kernel runs instead)."""
    a, b, g = random_case(m, k, n, seed=m + k + n)
    sa = (torch.rand(m, 1, generator=g) + 0.5).to(DEV)
    sb = (torch.rand(n, generator=g) + 0.5).to(DEV)
    bias = (torch.rand(n, generator=g) - 0.5).to(out_dtype).to(DEV)
    c = torch.full((m + 3, n), float("nan"), dtype=out_dtype, device=DEV)
    hb.scaled_mm(c[:m], a, b, sa, sb, bias)
    assert device_status_ok()
    check(c[:m], a, b, sa, sb, bias)
    assert torch.isnan(c[m:]).all()  # rows past M are not written
    c2 = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    hb.scaled_mm(c2, a, b, sa[:1], sb[:1], None)
    assert device_status_ok()
    check(c2, a, b, sa[:1], sb[:1], None)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,k,n", PREFILL)
def test_prefill_shapes_int8_bit_exact(m, k, n, out_dtype):
    g = torch.Generator().manual_seed(m + k + n)
    a = torch.randint(-128, 128, (m, k), dtype=torch.int8, generator=g)
    b = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=g).t()
    sa = (torch.rand(m, 1, generator=g) + 0.5) * 1e-3
    sb = (torch.rand(n, generator=g) + 0.5) * 1e-3
    bias = (torch.rand(n, generator=g) - 0.5).to(out_dtype)
    c = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
    hb.scaled_mm(c, a.to(DEV), b.to(DEV), sa.to(DEV), sb.to(DEV), bias.to(DEV))
    assert device_status_ok()
    assert torch.equal(c.cpu(), O.scaled_mm(a, b, sa, sb, bias, out_dtype))


def test_prefill_is_deterministic_and_replays_from_a_graph():
    m, k, n = 1024, 2048, 1536
    a, b, g = random_case(m, k, n, seed=77)
    sa = (torch.rand(m, 1, generator=g) + 0.5).to(DEV)
    sb = (torch.rand(n, generator=g) + 0.5).to(DEV)
    c = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    hb.scaled_mm(c, a, b, sa, sb)
    first = c.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        hb.scaled_mm(c, a, b, sa, sb)
    a2, _, _ = random_case(m, k, n, seed=78)
    a.copy_(a2)
    graph.replay()
    assert device_status_ok()
    assert not torch.equal(c, first)
    check(c, a, b, sa, sb, None)


def test_a_chain_of_calls_whose_tokens_the_kernel_before_wrote():
    """Every call's tokens are written by the kernel just before it on the stream, and the next call reuses the
    shared workspace (partial sums, arrival counters) at once; eagerly and replayed from a graph."""
    m, k, n = 16, 4096, 24576  # stream-K: partial sums and arrival counters in the shared workspace
    a, b, g = random_case(m, k, n, seed=91)
    sa = (torch.rand(m, 1, generator=g) + 0.5).to(DEV)
    sb = (torch.rand(n, generator=g) + 0.5).to(DEV)
    srcs = [random_case(m, k, 16, seed=92 + i)[0] for i in range(6)]
    outs = [torch.empty(m, n, dtype=torch.bfloat16, device=DEV) for _ in srcs]
    torch.cuda.synchronize()
    for src, c in zip(srcs, outs):
        a.copy_(src)            # a kernel that writes the tokens ...
        hb.scaled_mm(c, a, b, sa, sb)  # ... directly followed by their consumer
    assert device_status_ok()
    for src, c in zip(srcs, outs):
        check(c, src, b, sa, sb, None)
    # the same chain replayed from a graph
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for src, c in zip(srcs, outs):
            a.copy_(src)
            hb.scaled_mm(c, a, b, sa, sb)
    firsts = [c.clone() for c in outs]
    for c in outs:
        c.fill_(float("nan"))
    graph.replay()
    assert device_status_ok()
    for c, first in zip(outs, firsts):
        assert torch.equal(c, first)
