"""Parity checks that pair the CUDA path's outputs with the CPU oracle on a sample (test infrastructure only:
imported by ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s parity legs, never by the product)."""

from __future__ import annotations

import torch
from torch import Tensor

from . import oracle as O


def rel_err_elements(y: Tensor, ref: Tensor) -> Tensor:
    """``|y - ref| / max(|ref|, rms(ref))`` per element (the floating-point parity measure of this repository)."""
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    return (y - ref).abs() / torch.maximum(ref.abs(), floor)


def _signed_index(codes: Tensor) -> Tensor:
    """4-bit e2m1 code -> position on the value ladder -6 ... -0.5, 0, 0.5 ... 6 (both zeros at 0)."""
    c = codes.to(torch.int16)
    mag = c & 7
    return torch.where((c & 8) != 0, -mag, mag)


def swizzled_rows(flat: Tensor, rows: Tensor, cols: int) -> Tensor:
    """Rows ``rows`` of a SWIZZLE_32_4_4 scale buffer for logical ``[*, cols]`` (bytes, ``[len(rows), cols]``),
    by the layout's formula (examples/nvfp4_gemv.py:68-79) without materialising the whole offset table."""
    col_tiles = (cols + 3) // 4
    r = rows.to(torch.int64).reshape(-1, 1)
    c = torch.arange(cols, dtype=torch.int64).reshape(1, -1)
    off = ((r // 128) * col_tiles + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    return flat.reshape(-1).view(torch.uint8)[off]


def moe_sample_report(x: Tensor, logits: Tensor, top_k: int, w_gu, w_d, y_gpu: Tensor, inter: dict,
                      tokens: Tensor) -> dict:
    """Compare the NVFP4 MoE layer's CUDA result with the oracle on the sampled ``tokens`` of a (possibly
    full-size) problem.  Tokens are independent, so the oracle runs on the sample alone with the experts it
    touches, one expert at a time.

    ``w_gu`` / ``w_d`` are the expert weight bundles (``packed [E, N, K/2]``, ``scales [E, ...]``,
    ``global_scale [E]``, gate rows first, NOT interleaved) on any device; ``inter`` is what
    ``nvfp4_moe(..., intermediates=inter)`` filled.

    Returns counts and maxima: the end-to-end error, the same with the oracle's second half fed the CUDA path's
    own intermediate codes (what remains is the arithmetic of the second GEMM and the combine alone), and how the
    intermediate codes / scales differ (a last-place difference of the first GEMM's fp32 sum can flip a bf16
    rounding of the intermediate and with it a 4-bit code by one step).
    """
    tokens = tokens.cpu().long()
    xs, ls = x[tokens.to(x.device)].cpu(), logits[tokens.to(logits.device)].cpu()
    w_gpu = inter["weights"][tokens.to(inter["weights"].device)].cpu()
    e_gpu = inter["experts"][tokens.to(inter["experts"].device)].cpu()
    w_ref, e_ref = O.moe_route(ls, top_k)
    routing_same = bool(torch.equal(e_ref, e_gpu))
    routing_weight_err = float(((w_ref - w_gpu).abs() / w_ref.abs().clamp(min=1e-30)).max()) if routing_same else None

    experts = w_gu.packed.shape[0]
    need = sorted(set(e_gpu.reshape(-1).tolist()))

    def host(bundle):
        packed, scales = [None] * experts, [None] * experts
        for e in need:
            packed[e] = bundle.packed[e].cpu()
            scales[e] = bundle.scales[e].cpu()
        return packed, scales, bundle.global_scale.cpu()

    gp, gs, gg = host(w_gu)
    dp, ds, dg = host(w_d)
    ref, pairs = O.nvfp4_moe(xs, ls, top_k, gp, gs, gg, dp, ds, dg, return_pairs=True, routing=(w_gpu, e_gpu))
    y_s = y_gpu[tokens.to(y_gpu.device)].cpu()
    err = rel_err_elements(y_s, ref)

    # the CUDA path's intermediate for the same (token, slot) pairs
    sched = inter["sched"]
    inter_dim = pairs["codes"].shape[1]
    pair_id = tokens[pairs["tok"]] * top_k + pairs["slot"]
    rows = sched.row_of_pair.cpu().long()[pair_id]
    dev = inter["a2"].device
    codes_gpu = O.unpack_codes_k_major(inter["a2"][rows.to(dev)].cpu())
    scales_gpu = swizzled_rows(inter["sf2"].cpu(), rows, inter_dim // 16)
    g_gpu = inter["g2"][rows.to(dev)].cpu()

    step = (_signed_index(codes_gpu) - _signed_index(pairs["codes"])).abs()
    codes_diff = step > 0
    scales_diff = scales_gpu != pairs["scales"].view(torch.uint8)
    scale_steps = (scales_gpu.to(torch.int16) - pairs["scales"].view(torch.uint8).to(torch.int16)).abs()
    g_err = float(((g_gpu - pairs["g"]).abs() / pairs["g"].abs().clamp(min=1e-30)).max())
    pair_differs = codes_diff.any(dim=1) | scales_diff.any(dim=1) | (g_gpu != pairs["g"])
    token_differs = torch.zeros(tokens.numel(), dtype=torch.bool)
    token_differs[pairs["tok"][pair_differs]] = True

    y_inter = None
    if inter.get("y") is not None:
        y_g = inter["y"][rows.to(dev)].cpu()
        d = (y_g.float() - pairs["y"].float()).abs()
        row_max = pairs["y"].float().abs().amax(dim=1, keepdim=True).clamp(min=1e-30)
        y_inter = {"elements": int(d.numel()), "elements_differing": int((d > 0).sum()),
                   "max_abs_diff_over_row_amax": float((d / row_max).max())}

    # second half of the oracle on the CUDA path's own intermediate
    ref2 = O.nvfp4_moe_down(codes_gpu, scales_gpu.view(torch.float8_e4m3fn), g_gpu, pairs["tok"], pairs["slot"],
                            pairs["expert"], w_gpu, dp, ds, dg, tokens.numel())
    err2 = rel_err_elements(y_s, ref2)

    over = err > 1e-2
    return {
        "tokens": int(tokens.numel()), "pairs": int(rows.numel()), "experts_touched": len(need),
        "routing_same": routing_same, "routing_weight_max_rel_err": routing_weight_err,
        "max_rel_err": float(err.max()), "rms_rel_err": float((y_s.float() - ref.float()).pow(2).mean().sqrt()
                                                              / ref.float().pow(2).mean().sqrt()),
        "elements_over_1e-2": int(over.sum()),
        "elements_over_1e-2_in_tokens_without_intermediate_difference": int((over & ~token_differs[:, None]).sum()),
        "max_rel_err_given_cuda_intermediate": float(err2.max()),
        "intermediate_codes": int(codes_diff.numel()), "intermediate_codes_differing": int(codes_diff.sum()),
        "intermediate_codes_differing_by_more_than_one_step": int((step > 1).sum()),
        "intermediate_scales_differing": int(scales_diff.sum()),
        "intermediate_scales_differing_by_more_than_one_step": int((scale_steps > 1).sum()),
        "intermediate_row_scale_max_rel_err": g_err,
        "pairs_with_intermediate_difference": int(pair_differs.sum()),
        "intermediate_y": y_inter,
    }


def _bits(t: Tensor) -> Tensor:
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8) if t.element_size() == 1 else t.view(torch.int32)


def rms_quant_report(x: Tensor, w: Tensor, eps: float, q: Tensor, s: Tensor, scale_ub: Tensor | None = None,
                     residual: Tensor | None = None, chunk: int = 4096) -> dict:
    """``rms_norm_dynamic_per_token_quant`` outputs ``q`` / ``s`` against the CPU oracle, row by row: exact counts of
    differing rows, codes and scales, and how many differing rows are NOT explained by moving that row's fp32
    ``rms`` by at most two units in the last place (the sum of squares is order dependent; nothing else is)."""
    x, w, q, s = x.cpu(), w.cpu(), q.cpu(), s.cpu()
    rows_bad = codes_bad = scales_bad = unexplained = 0
    for r0 in range(0, x.shape[0], chunk):
        xs = x[r0 : r0 + chunk]
        rs = None if residual is None else residual[r0 : r0 + chunk].cpu()
        qs, ss = _bits(q[r0 : r0 + chunk]), _bits(s[r0 : r0 + chunk]).reshape(-1)
        qo, so, _ = O.rms_norm_dynamic_per_token_quant(xs, w, eps, scale_ub, rs)
        dq, ds = qs != _bits(qo), ss != _bits(so).reshape(-1)
        bad = dq.any(dim=1) | ds
        rows_bad += int(bad.sum())
        codes_bad += int(dq.sum())
        scales_bad += int(ds.sum())
        left = bad.clone()
        for nudge in (-1, 1, -2, 2):
            if not left.any():
                break
            idx = left.nonzero(as_tuple=True)[0]
            qn, sn, _ = O.rms_norm_dynamic_per_token_quant(
                xs[idx], w, eps, scale_ub, None if rs is None else rs[idx],
                rms_ulp_nudge=torch.full((idx.numel(),), nudge, dtype=torch.int32))
            ok = ~((qs[idx] != _bits(qn)).any(dim=1) | (ss[idx] != _bits(sn).reshape(-1)))
            left[idx[ok]] = False
        unexplained += int(left.sum())
    return {"rows": int(x.shape[0]), "rows_differing": rows_bad, "codes_differing": codes_bad,
            "scales_differing": scales_bad, "rows_not_explained_by_2ulp_of_rms": unexplained}
