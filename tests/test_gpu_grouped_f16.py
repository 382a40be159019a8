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


def _graph(fn, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    torch.cuda.synchronize()
    return g, out


@pytest.mark.parametrize("split_dtype,split_stride", [(torch.int64, 2), (torch.int32, 1)])
def test_split_sizes_edges_and_graph_replay(split_dtype, split_stride):
    """The ragged edge cases and the capture -> mutate -> replay protocol of
    test/test_cute_grouped_gemm_split_sizes.py:628-745: zero-row and one-row groups, then, by replaying one captured
    launch after overwriting the device-resident sizes, another partition, an oversized size, negative sizes and
    (int64) a size beyond int32.  Sizes are clipped, never trusted; rows no group covers keep their contents."""
    from helion_b200 import grouped as G

    gen = torch.Generator().manual_seed(5)
    sizes0 = (0, 224, 17, 0, 449, 1, 256, 1101)
    m, n, k, groups = sum(sizes0), 224, 128, len(sizes0)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(DEV)
    b = torch.randn(groups, n, k, generator=gen).to(torch.bfloat16).to(DEV)
    storage = torch.zeros(groups * split_stride, dtype=split_dtype, device=DEV)
    split = storage[::split_stride]
    assert split.stride() == (split_stride,)
    out = torch.full((m, n), -7.0, dtype=torch.bfloat16, device=DEV)

    def set_sizes(sizes):
        split.copy_(torch.tensor(sizes, dtype=split_dtype, device=DEV))

    def expected(sizes):
        want = torch.full((m, n), -7.0)
        prefix = 0
        for g, raw in enumerate(sizes):
            length = min(max(raw, 0), m)
            lo, hi = min(max(prefix, 0), m), min(max(prefix + length, 0), m)
            if hi > lo:
                want[lo:hi] = a[lo:hi].float().cpu() @ b[g].float().cpu().t()
            prefix += raw
        return want

    set_sizes(sizes0)
    graph, captured = _graph(lambda: G.grouped_gemm_split_sizes(a, b, split, out=out))
    assert captured is out
    cases = [sizes0, (113, 0, 224, 200, 0, 1, 300, 1210), (m + 1, 0, 0, 0, 0, 0, 0, 0), (-100, 50, m + 50, 0, 0, 0, 0, 0)]
    if split_dtype is torch.int64:
        huge = torch.iinfo(torch.int32).max + 17
        cases.append((huge, m - huge, 0, 0, 0, 0, 0, 0))
    for sizes in cases:
        a.normal_(generator=None)
        set_sizes(sizes)
        out.fill_(-7.0)
        graph.replay()
        assert status_ok()
        want = expected(sizes)
        got = out.float().cpu()
        untouched = want == -7.0
        assert torch.equal(got[untouched], want[untouched]), sizes  # nothing outside the groups' visible rows
        assert rel_err(torch.where(untouched, torch.zeros_like(got), got),
                       torch.where(untouched, torch.zeros_like(want), want)) <= 1e-2, sizes
        if sizes[0] == -100:
            # the reference's reading of negative sizes: the third group starts at -50 and writes rows [0, m - 50)
            assert bool((out[m - 50 :].float() == -7.0).all()) and bool((out[: m - 50].float() != -7.0).any())


def test_worklist_items_are_clipped_not_trusted():
    """Worklist entries come from device memory: negative starts or groups drop the item, store_m is clipped to the
    rows that exist, valid_m to store_m; unsorted items are fine."""
    gen = torch.Generator().manual_seed(9)
    m_total, n, k = 640, 256, 64
    a = torch.randn(m_total, k, generator=gen).to(torch.float16)
    b = torch.randn(3, n, k, generator=gen).to(torch.float16)
    wl = torch.tensor([[2, 384, 100, 128], [0, 0, 128, 128], [1, 512, 300, 9999], [1, -128, 5, 128], [-1, 128, 7, 128],
                       [0, 128, 200, 100], [2, 700, 1, 1]], dtype=torch.int32)
    y = hb.grouped_gemm_deepgemm(a.to(DEV), b.to(DEV), wl.to(DEV))
    assert status_ok()
    want = torch.zeros(m_total, n)
    af, bf = a.float(), b.float()
    want[384:484] = af[384:484] @ bf[2].t()          # rows 484..511 of the item are stored as zero
    want[0:128] = af[0:128] @ bf[0].t()
    want[512:640] = af[512:640] @ bf[1].t()          # store and valid clipped to the 128 rows that exist
    want[128:228] = af[128:228] @ bf[0].t()          # valid (200) clipped to store (100)
    assert rel_err(y, want) <= 1e-2
    assert float(y[228:384].float().abs().max()) == 0.0 and float(y[484:512].float().abs().max()) == 0.0


def test_grouped_gemm_graph_replay_after_mutating_inputs():
    """Capture -> mutate inputs and metadata -> replay (test/test_cute_deepgemm_selected.py:391-405)."""
    gen = torch.Generator().manual_seed(12)
    m_total, n, k = 512, 384, 128
    a = torch.randn(m_total, k, generator=gen).to(torch.bfloat16).to(DEV)
    b = torch.randn(4, n, k, generator=gen).to(torch.bfloat16).to(DEV)
    wl = torch.tensor([[0, 0, 128, 128], [1, 128, 60, 128], [2, 256, 128, 128], [3, 384, 1, 128]], dtype=torch.int32, device=DEV)
    graph, y = _graph(lambda: hb.grouped_gemm_deepgemm(a, b, wl))
    a.normal_()
    b.normal_()
    wl.copy_(torch.tensor([[3, 0, 100, 128], [3, 128, 128, 128], [0, 256, 0, 128], [1, 384, 128, 128]], dtype=torch.int32))
    graph.replay()
    assert status_ok()
    assert rel_err(y, O.grouped_gemm_worklist(a.cpu(), b.cpu(), wl.cpu())) <= 1e-2
    offs = torch.tensor([0, 100, 100, 357, 512], dtype=torch.int32, device=DEV)
    bj = torch.randn(k, n, generator=gen).to(torch.bfloat16).to(DEV)
    graph2, yj = _graph(lambda: hb.grouped_gemm_jagged(a, bj, offs))
    a.normal_()
    offs.copy_(torch.tensor([0, 0, 300, 301, 512], dtype=torch.int32))
    graph2.replay()
    assert status_ok()
    assert rel_err(yj, O.grouped_gemm_jagged(a.cpu(), bj.cpu(), offs.cpu())) <= 1e-2


# the seven cases of benchmarks/cute/compare_grouped_gemm_backends.py:102-116 (M, N, K per group): the default small
# parity case and the CUTLASS-example shapes with M and N tails
def _doc_case(m1, n3):
    return ((8192, 1280, 32), (m1, 384, 1536), (640, 1280, 16), (640, n3, 16))


DIRECT_CASES = {
    "default_small_parity": ((128, 128, 128), (512, 128, 128), (128, 256, 128)),
    "doc_no_mn_tail": _doc_case(128, 128), "doc_no_mn_g3_192_extra_full": _doc_case(128, 192),
    "doc_original": _doc_case(16, 160), "doc_mtail_g1_g3_192_extra_full": _doc_case(16, 192),
    "doc_mtail_g1_only": _doc_case(16, 128), "doc_ntail_g3_160": _doc_case(128, 160),
}


def _reference_args(problems, group_a, group_b, outputs):
    """The arguments _prepare_helion builds (pretuned_kernels/grouped_gemm/grouped_gemm.py:261-327)."""
    dev = group_a[0].device
    aligned = [(m + 127) // 128 * 128 for m, _, _ in problems]
    layout = torch.cat([torch.cat([torch.full((m,), g, dtype=torch.int32), torch.full((am - m,), -1, dtype=torch.int32)])
                        for g, ((m, _, _), am) in enumerate(zip(problems, aligned))]).to(dev)
    max_n, max_k = max(p[1] for p in problems), max(p[2] for p in problems)

    def placeholder(shape):
        base = torch.empty(max(1, shape[-1]), device=dev, dtype=group_a[0].dtype)
        return torch.as_strided(base, shape, (0,) * (len(shape) - 1) + (1,))

    pointers = torch.tensor([(a.data_ptr(), b.data_ptr(), o.data_ptr()) for a, b, o in zip(group_a, group_b, outputs)],
                            dtype=torch.int64, device=dev)
    strides = torch.tensor([(tuple(a.stride()), tuple(b.stride()), tuple(o.stride())) for a, b, o in zip(group_a, group_b, outputs)],
                           dtype=torch.int32, device=dev)
    signature = (len(problems),) + tuple(v for p in problems for v in p)
    return (placeholder((sum(aligned), max_k)), placeholder((len(problems), max_n, max_k)), layout,
            torch.tensor([p[1] for p in problems], dtype=torch.int32, device=dev),
            torch.tensor([p[2] for p in problems], dtype=torch.int32, device=dev),
            placeholder((sum(aligned), max_n)), pointers, strides, signature)


@pytest.mark.parametrize("case", sorted(DIRECT_CASES))
def test_direct_mode_heterogeneous_groups(case):
    """Per-group M, N and K with separate operand and output tensors, through the reference's own call signature
    (device pointer and stride tables) and through the list form; checked as check_correctness does (fp32 matmul of
    the same operands), then replayed from a CUDA graph after the inputs changed."""
    problems = DIRECT_CASES[case]
    gen = torch.Generator().manual_seed(0)
    group_a = [torch.randn(m, k, generator=gen).to(torch.float16).to(DEV) for m, _, k in problems]
    group_b = [torch.randn(n, k, generator=gen).to(torch.float16).to(DEV) for _, n, k in problems]
    outputs = [torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV) for m, n, _ in problems]

    def check():
        assert status_ok()
        for a, b, o in zip(group_a, group_b, outputs):
            assert rel_err(o, (a.float() @ b.float().t()).half()) <= 1e-2

    args = _reference_args(problems, group_a, group_b, outputs)
    out = hb.grouped_gemm(*args)
    assert out is args[5]
    check()
    for o in outputs:
        o.fill_(float("nan"))
    hb.grouped_gemm_direct(group_a, group_b, outputs)
    check()
    graph, _ = _graph(lambda: hb.grouped_gemm(*args))
    for t in group_a + group_b:
        t.normal_()
    for o in outputs:
        o.fill_(float("nan"))
    graph.replay()
    check()


def test_direct_mode_views_empty_groups_and_bf16():
    gen = torch.Generator().manual_seed(4)
    big_a = torch.randn(300, 512, generator=gen).to(torch.bfloat16).to(DEV)
    big_o = torch.full((300, 1024), -7.0, dtype=torch.bfloat16, device=DEV)
    group_a = [big_a[:130, 64:192], big_a[130:, 256:320], torch.empty(0, 64, dtype=torch.bfloat16, device=DEV)]
    group_b = [torch.randn(200, 128, generator=gen).to(torch.bfloat16).to(DEV), torch.randn(72, 64, generator=gen).to(torch.bfloat16).to(DEV),
               torch.randn(16, 64, generator=gen).to(torch.bfloat16).to(DEV)]
    outputs = [big_o[:130, 8:208], big_o[130:, 512:584], torch.empty(0, 16, dtype=torch.bfloat16, device=DEV)]
    hb.grouped_gemm_direct(group_a, group_b, outputs)
    assert status_ok()
    for a, b, o in zip(group_a[:2], group_b[:2], outputs[:2]):
        assert rel_err(o, (a.float() @ b.float().t()).to(torch.bfloat16)) <= 1e-2
    untouched = torch.ones_like(big_o, dtype=torch.bool)
    untouched[:130, 8:208] = False
    untouched[130:, 512:584] = False
    assert bool((big_o[untouched] == -7.0).all())  # views: nothing outside a group's own columns is written
    with pytest.raises(_lib.HelionB200Error):
        hb.grouped_gemm_direct([big_a[:8, :12]], [group_b[0][:8, :12]], [big_o[:8, :8]])  # K % 8 != 0
