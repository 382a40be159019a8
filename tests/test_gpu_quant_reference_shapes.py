"""Every shape the reference's own ``correctness_check()`` functions walk, for all six FP8 producers.

The grids are the ``_bench_shapes()`` of the pretuned modules (per_token_group_fp8_quant.py:147-151,
rms_norm_dynamic_per_token_quant.py:204-208, silu_and_mul_per_block_quant.py:190-194,
rms_norm_per_block_quant.py:262-272, dynamic_per_token_scaled_fp8_quant.py:133-138, silu_mul_fp8.py:99-103).  The
reference checks its kernels against its torch functions evaluated on the GPU.  Here the oracle's functions (the
same torch expressions) run on the GPU where every operation in them is exactly rounded on both sides (SiLU-mul as the
reference's own protocol has it, the dynamic per-token quantiser, silu_mul_fp8) and on the CPU otherwise (log2 / exp2
in the group quantiser's power-of-two scales, rsqrt and the order of the sum of squares in the RMSNorm producers, whose
rows must equal the oracle or the oracle with that row's fp32 rms moved by at most two units in the last place).
"""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
FP8 = torch.float8_e4m3fn


def bits(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().contiguous()
    return t.view(torch.uint8) if t.element_size() == 1 else t.view(torch.int32)


def same(a: torch.Tensor, b: torch.Tensor) -> bool:
    return bool(torch.equal(bits(a).to(DEV), bits(b).to(DEV)))


GROUP_SHAPES = [(t, h) for h in (2048, 4096, 5120) for t in (1, 4, 16, 64, 256, 1024, 2048, 8192)]
RMS_SHAPES = [(t, h) for h in (2048, 4096, 5120) for t in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048)]
SILU_SHAPES = [(t, i) for i in (6144, 12288, 25600) for t in (1, 8, 32, 64, 128, 256, 1024, 4096)]
RMS_BLOCK_SHAPES = [(t, h) for h in (2048, 4096, 5120) for t in (1, 8, 32, 64, 128, 256, 1024, 4096)]
DYN_SHAPES = [(t, h) for h in (2048, 4096, 5120) for t in (1, 4, 16, 64, 256, 1024, 2048, 4096)]
SILU_FP8_SHAPES = [(t, i) for i in (2048, 2880, 4096, 8192, 11008, 14336) for t in (1, 8, 32, 64, 128, 256)]


def test_per_token_group_fp8_quant_on_the_reference_grid():
    torch.manual_seed(0)
    for t, h in GROUP_SHAPES:
        x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
        for ue in (False, True):
            q = torch.empty(t, h, device=DEV, dtype=FP8)
            s = torch.empty(t, h // 128, device=DEV)
            hb.per_token_group_fp8_quant(x, q, s, 128, 1e-10, -448.0, 448.0, ue)
            qo, so = O.per_token_group_fp8_quant(x.cpu(), 128, 1e-10, -448.0, 448.0, ue)
            assert same(s, so) and same(q, qo), (t, h, ue)


def test_silu_and_mul_per_block_quant_on_the_reference_grid():
    torch.manual_seed(0)
    for t, i in SILU_SHAPES:
        x = torch.randn(t, 2 * i, device=DEV, dtype=torch.bfloat16)
        q = torch.empty(t, i, device=DEV, dtype=FP8)
        s = torch.empty(t, i // 128, device=DEV)
        hb.silu_and_mul_per_block_quant(q, x, s, 128)
        qo, so = O.silu_and_mul_per_block_quant(x, 128)
        assert same(s, so) and same(q, qo), (t, i)
        del x, q, s, qo, so


def test_dynamic_per_token_scaled_fp8_quant_on_the_reference_grid():
    torch.manual_seed(0)
    for t, h in DYN_SHAPES:
        x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
        q = torch.empty(t, h, device=DEV, dtype=FP8)
        s = torch.empty(t, 1, device=DEV)
        hb.dynamic_per_token_scaled_fp8_quant(q, x, s)
        qo, so = O.dynamic_per_token_scaled_fp8_quant(x)
        assert same(s, so) and same(q, qo), (t, h)


def test_silu_mul_fp8_on_the_reference_grid():
    torch.manual_seed(0)
    scale = torch.tensor([0.37], device=DEV)
    for t, i in SILU_FP8_SHAPES:
        x = torch.randn(t, 2 * i, device=DEV, dtype=torch.bfloat16)
        got = hb.silu_mul_fp8(x, scale)
        r = (torch.nn.functional.silu(x[:, :i]) * x[:, i:]).to(torch.float32)
        want = (r * (1.0 / scale.reshape(()))).clamp(-448.0, 448.0).to(FP8)
        assert same(got, want), (t, i)


def _rows_explained_by_the_rms(q, s, oracle_with_nudge, tokens):
    """Rows that equal the oracle, or the oracle with that row's fp32 rms moved by at most two units in the last
    place (the order of the sum of squares is the only freedom in the chain)."""
    qo, so = oracle_with_nudge(None)
    bad = (bits(q) != bits(qo).to(DEV)).any(dim=1) | (bits(s) != bits(so).to(DEV)).reshape(tokens, -1).any(dim=1)
    for nudge in (-1, 1, -2, 2):
        if not bool(bad.any()):
            break
        qn, sn = oracle_with_nudge(torch.full((tokens,), nudge, dtype=torch.int32))
        bad &= (bits(q) != bits(qn).to(DEV)).any(dim=1) | (bits(s) != bits(sn).to(DEV)).reshape(tokens, -1).any(dim=1)
    return int(bad.sum())


def test_rms_norm_dynamic_per_token_quant_on_the_reference_grid():
    torch.manual_seed(0)
    for t, h in RMS_SHAPES:
        x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
        w = (torch.rand(h, device=DEV) + 0.5).to(torch.bfloat16)
        q = torch.empty(t, h, device=DEV, dtype=FP8)
        s = torch.empty(t, 1, device=DEV)
        hb.rms_norm_dynamic_per_token_quant(q, x, w, s, 1e-6)

        xc, wc = x.cpu(), w.cpu()

        def oracle(nudge):
            qo, so, _ = O.rms_norm_dynamic_per_token_quant(xc, wc, 1e-6, None, None, nudge)
            return qo, so

        assert _rows_explained_by_the_rms(q, s, oracle, t) == 0, (t, h)


def test_rms_norm_per_block_quant_on_the_reference_grid():
    torch.manual_seed(0)
    for t, h in RMS_BLOCK_SHAPES:
        x = torch.randn(t, h, device=DEV, dtype=torch.bfloat16)
        w = (torch.rand(h, device=DEV) + 0.5).to(torch.bfloat16)
        q = torch.empty(t, h, device=DEV, dtype=FP8)
        s = torch.empty(t, h // 128, device=DEV)
        hb.rms_norm_per_block_quant(q, x, w, s, 1e-6, None, None, 128, False)

        xc, wc = x.cpu(), w.cpu()

        def oracle(nudge):
            qo, so, _ = O.rms_norm_per_block_quant(xc, wc, 1e-6, 128, None, None, nudge)
            return qo, so

        assert _rows_explained_by_the_rms(q, s, oracle, t) == 0, (t, h)
