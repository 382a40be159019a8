"""Grouped NVFP4 GEMM and the NVFP4 MoE layer against the CPU oracle."""

from __future__ import annotations

import pytest
import torch

import helion_b200 as hb
from helion_b200 import _lib
from helion_b200 import moe as M
from oracle import checks as C
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(y, ref):
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    assert torch.isfinite(y).all()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    return float(((y - ref).abs() / torch.maximum(ref.abs(), floor)).max())


def oracle_weights(w: torch.Tensor):
    """Quantise ``[E, N, K]`` with the oracle, one global scale per expert; returns oracle-side lists and the device-side bundle."""
    packed, scales, gs = [], [], []
    for e in range(w.shape[0]):
        p, s, g = O.nvfp4_quantize(w[e])
        packed.append(p)
        scales.append(s)
        gs.append(g)
    bundle = M.GroupedNvfp4Weight(
        torch.stack(packed).to(DEV), torch.stack([s.view(torch.uint8) for s in scales]).to(DEV).view(torch.float8_e4m3fn),
        torch.stack(gs).to(DEV),
    )
    return torch.stack(packed), scales, torch.stack(gs), bundle


@pytest.mark.parametrize("padding", [128, 256])
@pytest.mark.parametrize("counts", [[5, 0, 130, 1, 0, 128, 256, 3], [0, 0, 0, 7], [128], [1, 1, 1, 1, 1]])
def test_schedule_edge_cases(counts, padding):
    """Ragged groups incl. empty, single-row, exactly-full and multi-tile experts
    (the cases of test/test_cute_grouped_gemm_split_sizes.py:620-745 that apply to a routing result)."""
    e = len(counts)
    experts = torch.cat([torch.full((c,), i, dtype=torch.int64) for i, c in enumerate(counts)])
    experts = experts[torch.randperm(experts.numel(), generator=torch.Generator().manual_seed(0))]
    sched = M.build_schedule(experts.to(DEV).reshape(-1, 1), e, padding)
    torch.cuda.synchronize()
    pad = [0]
    for c in counts:
        pad.append(pad[-1] + (c + padding - 1) // padding * padding)
    assert sched.padded_offsets.cpu().tolist() == pad
    info = sched.tile_info.cpu().tolist()
    assert len(info) >= (sum(counts) + 127) // 128 + e * (padding // 128) and len(info) % (padding // 128) == 0
    for t, (g, rows) in enumerate(info):
        row0 = t * 128
        if row0 >= pad[-1]:
            assert (g, rows) == (-1, 0)
        else:
            exp_g = max(i for i in range(e) if pad[i] <= row0 and counts[i] > 0 and row0 < pad[i + 1])
            # a 256-padded expert may end with a tile that holds padding only
            assert g == exp_g and rows == max(0, min(128, counts[g] - (row0 - pad[g])))
    # stable order: inside an expert rows follow the original pair order
    order, _, offsets = O.moe_sort(experts.reshape(-1, 1), e)
    assert torch.equal(sched.sorted_pairs.cpu(), order)
    rows = sched.row_of_sorted.cpu()
    for i, c in enumerate(counts):
        assert rows[offsets[i] : offsets[i] + c].tolist() == list(range(pad[i], pad[i] + c))
    assert torch.equal(sched.row_of_pair.cpu()[order.long()], rows)


@pytest.mark.parametrize("padding,n", [(128, 384), (256, 512), (256, 384)])
def test_grouped_matmul_against_oracle(padding, n):
    torch.manual_seed(0)
    e, k = 6, 512
    counts = [70, 0, 200, 1, 128, 33]
    w = torch.randn(e, n, k) * 0.02
    wp, ws, wg, bundle = oracle_weights(w)
    experts = torch.cat([torch.full((c,), i, dtype=torch.int64) for i, c in enumerate(counts)])
    experts = experts[torch.randperm(experts.numel())]
    x = torch.randn(experts.numel(), k).to(torch.bfloat16)
    sched = M.build_schedule(experts.to(DEV).reshape(-1, 1), e, padding)
    a, sf, g = M._quantize_rows(x.to(DEV), k, sched, 1, None, False, gather=True)
    out = M.grouped_matmul(a, sf, bundle, sched, g, torch.float32)
    out16 = M.grouped_matmul(a, sf, bundle, sched, g)  # bf16: CTA pairs when padded to 256 and N % 256 == 0
    torch.cuda.synchronize()
    assert _lib.load().hb200_device_status(1) == 0
    rows = sched.row_of_pair.cpu().long()
    assert rel_err(out16.float().cpu()[rows], out.cpu()[rows]) <= 1e-2
    ap, asc, ag = O.nvfp4_quantize(x, per_token=True)
    aq = O.dequant_scaled_k_major(ap, asc) * ag.reshape(-1, 1)
    ref = torch.empty(x.shape[0], n)
    for i in range(e):
        idx = (experts == i).nonzero(as_tuple=True)[0]
        ref[idx] = aq[idx] @ (O.dequant_scaled_k_major(wp[i], ws[i]) * wg[i]).t()
    assert rel_err(out.cpu()[rows], ref) <= 1e-4


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("t,h,inter,e,k", [(64, 256, 128, 8, 2), (300, 512, 384, 16, 4), (128, 256, 256, 4, 1)])
def test_moe_layer_against_oracle(t, h, inter, e, k, interleaved):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    w_gu = torch.randn(e, 2 * inter, h, generator=g) * 0.02
    w_d = torch.randn(e, h, inter, generator=g) * 0.02
    gp, gsc, gg, gu_bundle = oracle_weights(w_gu)
    dp, dsc, dg, d_bundle = oracle_weights(w_d)
    ref = O.nvfp4_moe(x, logits, k, gp, gsc, gg, dp, dsc, dg)
    got = {}
    y = M.nvfp4_moe(x.to(DEV), logits.to(DEV), k, M.interleave_gate_up(gu_bundle) if interleaved else gu_bundle,
                    d_bundle, intermediates=got)
    torch.cuda.synchronize()
    assert _lib.load().hb200_device_status(1) == 0
    assert y.shape == (t, h) and y.dtype is torch.bfloat16
    # Bound: 1e-2 per element.  Two quantisation steps sit between input and output: a last-place difference of
    # the first GEMM's fp32 sum can flip one bf16 rounding of the intermediate and with it one 4-bit code by one
    # step, which moves single outputs of that token by about a percent.  Such an element is accepted only when
    # it is explained: its token's intermediate differs from the oracle's (by one step, never more) and the
    # oracle's second half fed with the CUDA path's own intermediate reproduces the CUDA output within 1e-2.
    rep = C.moe_sample_report(x, logits, k, gu_bundle, d_bundle, y, got, torch.arange(t))
    assert rep["routing_same"]
    assert abs(rep["max_rel_err"] - rel_err(y, ref)) <= 1e-3  # the report runs the oracle on the CUDA path's routing
    assert rep["max_rel_err_given_cuda_intermediate"] <= 1e-2
    assert rep["intermediate_codes_differing_by_more_than_one_step"] == 0
    assert rep["intermediate_scales_differing_by_more_than_one_step"] == 0
    assert rep["elements_over_1e-2_in_tokens_without_intermediate_difference"] == 0
    assert rep["max_rel_err"] <= 2e-2 and rep["rms_rel_err"] <= 5e-3


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
@pytest.mark.parametrize("pairs,experts", [(0, 4), (1, 1), (1000, 7), (70000, 128), (5000, 1024), (3333, 3)])
def test_device_sort_matches_stable_argsort(pairs, experts, dtype):
    g = torch.Generator().manual_seed(pairs + experts)
    e = torch.randint(0, experts, (pairs,), generator=g).to(dtype).to(DEV)
    sorted_pairs = torch.full((pairs,), -1, dtype=torch.int32, device=DEV)
    counts = torch.full((experts,), -1, dtype=torch.int32, device=DEV)
    scratch = torch.empty(max(1, -(-pairs // 1024)) * experts, dtype=torch.int32, device=DEV)
    _lib.call("hb200_moe_sort_pairs", e.data_ptr(), int(dtype is torch.int64), pairs, experts, sorted_pairs.data_ptr(),
              counts.data_ptr(), scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(sorted_pairs.cpu().long(), torch.argsort(e.cpu().long(), stable=True))
    assert torch.equal(counts.cpu().long(), torch.bincount(e.cpu().long(), minlength=experts))


def test_silu_epilogue_is_bit_identical_to_the_two_kernel_form():
    t, h, inter, e, k = 512, 512, 256, 8, 2
    g = torch.Generator().manual_seed(11)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16).to(DEV)
    logits = torch.randn(t, e, generator=g).to(DEV)
    w_gu = M.quantize_expert_weights((torch.randn(e, 2 * inter, h, generator=g) * 0.02).to(DEV))
    w_d = M.quantize_expert_weights((torch.randn(e, h, inter, generator=g) * 0.02).to(DEV))
    plain = M.nvfp4_moe(x, logits, k, w_gu, w_d)
    fused = M.nvfp4_moe(x, logits, k, M.interleave_gate_up(w_gu), w_d)
    torch.cuda.synchronize()
    assert _lib.load().hb200_device_status(1) == 0
    assert torch.equal(plain, fused)
    # and the pieces: y and the row maxima against the SiLU-mul of the quantiser kernel
    _, experts = M.route_top_k(logits, k)
    sched = M.build_schedule(experts, e)
    a1, sf1, g1 = M._quantize_and_gather(x, sched, k)
    h1 = M.grouped_matmul(a1, sf1, w_gu, sched, g1)
    y, amax = M.grouped_matmul_silu(a1, sf1, M.interleave_gate_up(w_gu), sched, g1)
    rows = sched.row_of_pair.long()
    hg, hu = h1[rows, :inter].float(), h1[rows, inter:].float()
    want = ((hg / (1.0 + torch.exp(-hg))) * hu).to(torch.bfloat16)
    assert torch.equal(y[rows], want)
    assert torch.equal(amax[rows], want.float().abs().amax(dim=1))


def test_pair_tiles_over_256_row_padding_give_the_same_layer_bit_for_bit(monkeypatch):
    """CTA-pair grouped GEMMs (SiLU-mul epilogue included) over experts padded to 256 rows, against the 128-row form;
    skewed routing, so some experts are empty and some 256-row tiles hold one valid half only."""
    t, h, inter, e, k = 1024, 512, 256, 8, 2
    g = torch.Generator().manual_seed(12)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16).to(DEV)
    logits = torch.randn(t, e, generator=g).to(DEV)
    logits[:, 5] = -30.0
    logits[:, 0] += 1.5
    w_gu = M.interleave_gate_up(M.quantize_expert_weights((torch.randn(e, 2 * inter, h, generator=g) * 0.02).to(DEV)))
    w_d = M.quantize_expert_weights((torch.randn(e, h, inter, generator=g) * 0.02).to(DEV))
    monkeypatch.delenv("HB200_MOE_PAD", raising=False)
    got128 = {}
    y128 = M.nvfp4_moe(x, logits, k, w_gu, w_d, intermediates=got128)
    monkeypatch.setenv("HB200_MOE_PAD", "256")
    got256 = {}
    y256 = M.nvfp4_moe(x, logits, k, w_gu, w_d, intermediates=got256)
    torch.cuda.synchronize()
    assert _lib.load().hb200_device_status(1) == 0
    assert got128["sched"].pad == 128 and got256["sched"].pad == 256
    r128, r256 = got128["sched"].row_of_pair.long(), got256["sched"].row_of_pair.long()
    assert torch.equal(got128["y"][r128], got256["y"][r256])
    assert torch.equal(got128["a2"][r128], got256["a2"][r256])
    assert torch.equal(y128, y256)


def test_layer_replays_from_a_cuda_graph_after_its_inputs_change():
    """Capture the whole layer (routing, sort, schedule, both grouped GEMMs, combine), then change tokens and router
    logits in place and replay: the routing, the per-expert row counts and the tile list all change on the device,
    nothing is read back (the pattern of test/test_cute_deepgemm_selected.py:391-405)."""
    t, h, inter, e, k = 384, 512, 256, 8, 2
    g = torch.Generator().manual_seed(13)
    w_gu = M.interleave_gate_up(M.quantize_expert_weights((torch.randn(e, 2 * inter, h, generator=g) * 0.02).to(DEV)))
    w_d = M.quantize_expert_weights((torch.randn(e, h, inter, generator=g) * 0.02).to(DEV))
    x = torch.randn(t, h, generator=g).to(torch.bfloat16).to(DEV)
    logits = torch.randn(t, e, generator=g).to(DEV)
    for _ in range(2):
        M.nvfp4_moe(x, logits, k, w_gu, w_d)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = M.nvfp4_moe(x, logits, k, w_gu, w_d)
    for seed, skew in ((14, None), (15, 3), (16, 0)):
        g2 = torch.Generator().manual_seed(seed)
        x.copy_(torch.randn(t, h, generator=g2).to(torch.bfloat16))
        new_logits = torch.randn(t, e, generator=g2)
        if skew is not None:
            new_logits[:, skew] += 4.0  # most tokens now take this expert: other experts shrink or empty out
        logits.copy_(new_logits)
        graph.replay()
        torch.cuda.synchronize()
        replayed = y.clone()
        eager = M.nvfp4_moe(x, logits, k, w_gu, w_d)
        torch.cuda.synchronize()
        assert _lib.load().hb200_device_status(1) == 0
        assert torch.equal(replayed, eager)


def test_device_weight_quantiser_matches_oracle():
    torch.manual_seed(5)
    w = torch.randn(3, 128, 256) * 0.02
    wp, ws, wg, _ = oracle_weights(w.to(torch.bfloat16).float())
    b = M.quantize_expert_weights(w.to(DEV))
    assert torch.equal(b.packed.cpu(), wp)
    assert torch.equal(b.global_scale.cpu(), wg)
    assert torch.equal(b.scales.cpu().view(torch.uint8), torch.stack([s.view(torch.uint8) for s in ws]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens,experts,k", [(1, 8, 2), (300, 128, 8), (64, 100, 5), (17, 1024, 33), (5, 32, 32), (0, 16, 2)])
def test_fused_routing_matches_softmax_then_topk(tokens, experts, k, dtype):
    g = torch.Generator().manual_seed(tokens + experts + k)
    logits = (torch.randn(tokens, experts, generator=g) * 2).to(dtype)
    w, e = M.route_top_k(logits.to(DEV), k)
    torch.cuda.synchronize()
    assert w.shape == (tokens, k) and e.shape == (tokens, k) and w.dtype is torch.float32 and e.dtype is torch.int64
    ow, oe = O.moe_route(logits, k)
    w, e = w.cpu(), e.cpu()
    torch.testing.assert_close(w, ow, rtol=2e-6, atol=1e-9)
    # the same experts in the same order, except where two probabilities are equal to within the last places
    differs = e != oe
    if bool(differs.any()):
        probs = torch.softmax(logits.float(), dim=-1)
        assert torch.allclose(probs.gather(1, e)[differs], probs.gather(1, oe)[differs], rtol=4e-6, atol=0)
    assert bool((w[:, :-1] >= w[:, 1:]).all())  # descending
    assert all(len(set(row.tolist())) == k for row in e)  # no expert twice


def test_fused_routing_breaks_ties_by_expert_index():
    logits = torch.zeros(3, 64, device=DEV)
    logits[1, 40] = 1.0
    w, e = M.route_top_k(logits, 4)
    assert e[0].tolist() == [0, 1, 2, 3] and e[1].tolist() == [40, 0, 1, 2]
    assert torch.allclose(w[0], torch.full((4,), 1 / 64, device=DEV))


@pytest.mark.parametrize("t,h,e,k", [(300, 512, 16, 4), (1000, 4096, 32, 8), (77, 2048, 8, 2), (64, 256, 8, 1)])
def test_fused_quantise_and_scatter_equals_quantiser_plus_gather(t, h, e, k):
    """The one-pass dispatch (quantise a token once, write its row to all its pairs' rows) writes the same bytes as
    the quantiser followed by the row gather, in every row a pair owns."""
    g = torch.Generator().manual_seed(t + h)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16).to(DEV)
    logits = torch.randn(t, e, generator=g).to(DEV)
    _, experts = M.route_top_k(logits, k)
    sched = M.build_schedule(experts, e)
    c1, s1, g1 = M._quantize_and_gather(x, sched, k, fused=True)
    c2, s2, g2 = M._quantize_and_gather(x, sched, k, fused=False)
    torch.cuda.synchronize()
    rows = sched.row_of_pair.long()
    assert torch.equal(c1[rows], c2[rows]) and torch.equal(g1[rows], g2[rows])
    cols = h // 16
    u1 = C.swizzled_rows(s1.cpu(), rows.cpu(), cols)
    u2 = C.swizzled_rows(s2.cpu(), rows.cpu(), cols)
    assert torch.equal(u1, u2)
    assert bool((g1[rows] > 0).all())
