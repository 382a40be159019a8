"""Benchmark driver: ``python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]``.

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of synthetic input, with the
inputs already resident in HBM; ``e2e`` repeats it through the public operator API from pinned host buffers.

Workloads (``--workload``):
  gemm   (default) dense NVFP4 GEMM, M=N=K=8192: A ~ N(0,1) bf16 and B ~ N(0,0.02), both quantised to NVFP4
         (16-wide blocks, e4m3 scales, fp32 global scale); bf16 output; metric TFLOP/s.  With N GPUs the
         rows of B (output columns) are split evenly and the outputs all-gathered.
  gemv   the four NVFP4 matrices of a 70B-class dense layer applied to M activation rows (--batch, default 1);
         metric TB/s of HBM traffic the step must move; column-parallel over N GPUs.
  moe    NVFP4 MoE layer: 8192 tokens, hidden 4096, 128 experts, top-8, intermediate 1536; metric TFLOP/s;
         expert-parallel over N GPUs.
  quant  the fused FP8 quant producers at 16384 tokens (RMSNorm hidden 7168 as the headline; the others in
         ``ops``); metric TB/s.
  scaled_mm  the row-wise scaled FP8 GEMM on the twelve (K, N) decode weight shapes the reference tunes it on,
         --batch tokens each (default 16; the reference sweeps 16 and 64), bias and per-tensor scales as in its
         sweep; a step is one pass over all twelve (715 MB of weights); metric TB/s; replicas only over N GPUs.

Timing: every step is bracketed by its own CUDA-event pair on the launching stream and the L2 is flushed
(a 256 MB write followed, on one GPU, by a 256 MB read of another buffer, which pushes the write's dirty lines
out) between steps, outside the pairs; ms_per_step is the mean over K steps and the max over
ranks.  Steps whose launch sequence is fixed are replayed from a CUDA graph so that the host does not sit
between kernels.  ``--impl reference`` times the CPU port of the reference's PyTorch reference functions on
a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path
import sys
import threading
import time

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYER_70B = {"qkv": (10240, 8192), "o": (8192, 8192), "gate_up": (57344, 8192), "down": (8192, 28672)}
MOE_CFG = dict(tokens=8192, hidden=4096, experts=128, top_k=8, inter=1536)
GEMM_CFG = dict(m=8192, n=8192, k=8192)
# (K, N) of the reference's scaled_mm sweep (pretuned_kernels/scaled_mm/scaled_mm.py:167-180)
SCALED_MM_KN = [(2048, 4096), (2048, 2048), (2048, 12288), (6144, 2048), (4096, 6144), (4096, 4096), (4096, 24576),
                (12288, 4096), (5120, 10240), (5120, 5120), (5120, 51200), (25600, 5120)]


def gemv_bytes(n: int, k: int, m: int = 1) -> int:
    """Algorithmic HBM bytes of one NVFP4 GEMV: packed codes + block scales + activations + outputs."""
    return n * k // 2 + n * k // 16 + 2 * m * k + 2 * m * n


def scaled_mm_bytes(m: int, k: int, n: int) -> int:
    """Algorithmic HBM bytes of one FP8 scaled_mm with a bf16 output and bias: weight, activations, bias, output."""
    return n * k + m * k + 2 * n + 2 * m * n


def moe_flops(c=MOE_CFG) -> int:
    pairs = c["tokens"] * c["top_k"]
    return 2 * pairs * c["hidden"] * 2 * c["inter"] + 2 * pairs * c["inter"] * c["hidden"]


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the headline kernels, from the
# `ncu --set full` captures summarised under profiles/ (same bench command, same sizes).
NCU_TRAFFIC = {
    "gemm_8192": 212.1e6,           # profiles/nvfp4_gemm_pair_kernel_8192x8192x8192.md
    "gemv_gate_up_m1": 268.5e6,     # profiles/nvfp4_gemv_kernels_70b_decode_layer.md
    "gemv_gate_up_m8": 274.9e6,     # tensor-core kernel
    "rms_norm_16384x7168": 315.0e6,      # profiles/quant_producers_16384_tokens.md
    "scaled_mm_16x5120x51200": 271.6e6,  # profiles/fp8_scaled_mm_kernel_decode_shapes.md
}


def ncu_traffic(key: str):
    return NCU_TRAFFIC.get(key)


# ------------------------------------------------------------------ timing
class Timer:
    profile_region = 0  # index of the timed region bracketed by cudaProfilerStart/Stop (--profile-region)
    flush_read = True   # --flush write+read (default) or write
    regions_seen = 0

    def __init__(self, dev, world: int):
        self.dev = dev
        self.world = world
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.sweep_buf = torch.zeros(256 << 18, dtype=torch.int32, device=dev)  # 256 MB, only ever read

    def sync(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def run(self, step, steps: int, warmup: int) -> float:
        """Mean milliseconds per step (max over ranks): per-step event pairs, L2 flushed between steps."""
        # (flush = write 256 MB, then read 256 MB: see the loop)
        for _ in range(warmup):
            step()
        self.sync()
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        profiled = Timer.profile_region == Timer.regions_seen  # `ncu --profile-from-start off` sees this region only
        Timer.regions_seen += 1
        if profiled:
            torch.cuda.profiler.start()
        for s, e in pairs:
            # L2 flush: a 256 MB write, then a 256 MB read of another buffer, so that the step neither finds its
            # inputs in L2 nor pays for writing back the flush's dirty lines
            self.flush_buf.zero_()
            # (one GPU only: with peers the extra eager kernels let the ranks drift apart between steps, and a
            # step's peer barriers then time the other rank's lateness: 135-155 us against 112 us on two GPUs)
            if Timer.flush_read and self.world == 1:
                self.sweep_buf.sum()
            s.record()
            step()
            e.record()
        self.sync()
        if profiled:
            torch.cuda.profiler.stop()
        ms = sum(s.elapsed_time(e) for s, e in pairs) / steps
        if self.world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms


def graphed(fn, warmup: int = 3):
    """Capture ``fn`` (fixed launch sequence, static buffers) in a CUDA graph; returns (replay, outputs)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    return g.replay, out


def graphed_ring(fn, turns: int = 2):
    """One graph per buffer of an output ring (``fn`` advances the ring by one per call); replays alternate."""
    replays = [graphed(fn, warmup=turns)[0] for _ in range(turns)]
    state = {"i": 0}

    def replay():
        replays[state["i"]]()
        state["i"] = (state["i"] + 1) % turns

    return replay


def rel_err(y, ref) -> float:
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    floor = ref.pow(2).mean().sqrt().clamp(min=1e-30)
    return float(((y - ref).abs() / torch.maximum(ref.abs(), floor)).max())


# ------------------------------------------------------------- CPU baselines
def cpu_gemm(seconds: float = 8.0):
    """Oracle port of reference_nvfp4_w4a4_matmul semantics (dequantise -> fp32 matmul) on a 1024x1024x8192 slice."""
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    m = n = 1024
    k = GEMM_CFG["k"]
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g)
    sa = O.swizzle_scales((torch.rand(m, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
    sb = O.swizzle_scales((torch.rand(n, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))

    def step():
        return O.nvfp4_scaled_matmul(a, b, sa, sb)

    return step, 2 * m * n * k, f"{m}x{n}x{k} slice of the 8192^3 GEMM (dequantise -> fp32 matmul -> bf16)"


def cpu_gemv():
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    k, rows = 8192, 1024
    g = torch.Generator().manual_seed(4)
    w = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, generator=g)
    x = torch.randn(k, generator=g).to(torch.bfloat16)
    s = O.swizzle_scales((torch.rand(rows, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
    return (lambda: O.nvfp4_gemv_bf16in(w, x, s, 1.0)), gemv_bytes(rows, k), f"{rows}x{k} slice of the O projection"


def cpu_quant():
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    t, h = 2048, 7168
    g = torch.Generator().manual_seed(2)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    w = (torch.rand(h, generator=g) + 0.5).to(torch.bfloat16)
    return (lambda: O.rms_norm_dynamic_per_token_quant(x, w, 1e-6)), 2 * t * h + 2 * h + t * h + 4 * t, f"{t} of 16384 tokens"


def cpu_moe():
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    t, h, inter, e, k = 256, MOE_CFG["hidden"], MOE_CFG["inter"], 8, 2
    g = torch.Generator().manual_seed(3)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16)
    logits = torch.randn(t, e, generator=g)
    gu = [O.nvfp4_quantize(torch.randn(2 * inter, h, generator=g) * 0.02) for _ in range(e)]
    dn = [O.nvfp4_quantize(torch.randn(h, inter, generator=g) * 0.02) for _ in range(e)]
    gp, gs, gg = torch.stack([p for p, _, _ in gu]), [s for _, s, _ in gu], torch.stack([q for _, _, q in gu])
    dp, ds, dg = torch.stack([p for p, _, _ in dn]), [s for _, s, _ in dn], torch.stack([q for _, _, q in dn])
    flops = 2 * t * k * h * 2 * inter + 2 * t * k * inter * h
    return (lambda: O.nvfp4_moe(x, logits, k, gp, gs, gg, dp, ds, dg)), flops, f"{t} tokens, {e} experts, top-{k} (same hidden/intermediate sizes)"


def cpu_scaled_mm():
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    m, k, n = 16, 4096, 4096
    g = torch.Generator().manual_seed(6)
    a = ((0.5 + torch.rand(m, k, generator=g)) / 64).to(torch.float8_e4m3fn)
    b = ((0.5 + torch.rand(n, k, generator=g)) / 64).to(torch.float8_e4m3fn).t()
    sa, sb = torch.rand(1, 1, generator=g) + 0.5, torch.rand(1, 1, generator=g) + 0.5
    bias = (torch.rand(n, generator=g) - 0.5).to(torch.bfloat16)
    return (lambda: O.scaled_mm(a, b, sa, sb, bias)), scaled_mm_bytes(m, k, n), f"the {m}x{k}x{n} shape of the twelve"


CPU_WORKLOADS = {"gemm": (cpu_gemm, 1e12, "TFLOP/s"), "gemv": (cpu_gemv, 1e12, "TB/s"), "quant": (cpu_quant, 1e12, "TB/s"),
                 "moe": (cpu_moe, 1e12, "TFLOP/s"), "scaled_mm": (cpu_scaled_mm, 1e12, "TB/s")}
METRICS = {"gemm": "nvfp4_gemm_tflops", "gemv": "nvfp4_gemv_hbm_throughput", "quant": "fp8_quant_producer_hbm_throughput",
           "moe": "nvfp4_moe_tflops", "scaled_mm": "fp8_scaled_mm_hbm_throughput"}


def time_cpu(workload: str, budget_s: float = 10.0, steps: int | None = None, warmup: int = 1):
    make, scale, unit = CPU_WORKLOADS[workload]
    step, work, sample = make()
    for _ in range(max(1, warmup)):
        step()
    t0 = time.perf_counter()
    reps = 0
    while True:
        step()
        reps += 1
        if steps is not None:
            if reps >= steps:
                break
        elif time.perf_counter() - t0 > budget_s or reps >= 50:
            break
    dt = (time.perf_counter() - t0) / reps
    return work / dt / scale, unit, torch.get_num_threads(), f"{sample}; {reps} calls", dt


def reference_config(args) -> dict:
    """The configuration of the matching GPU arm (the CPU arm times a bounded sample of it, see cpu_baseline.sample)."""
    if args.workload == "gemm":
        cfg = {"workload": "gemm", **GEMM_CFG}
    elif args.workload == "gemv":
        cfg = {"workload": "gemv", "layer": "qkv 10240x8192, o 8192x8192, gate_up 57344x8192, down 8192x28672", "batch": args.batch}
    elif args.workload == "moe":
        cfg = {"workload": "moe", **MOE_CFG}
    elif args.workload == "scaled_mm":
        cfg = {"workload": "scaled_mm", "tokens": args.batch if args.batch > 1 else 16, "kn_shapes": len(SCALED_MM_KN)}
    else:
        cfg = {"workload": "quant", "tokens": 16384, "hidden": 7168, "op": "rms_norm_dynamic_per_token_quant"}
    cfg["parallelism"] = "host cores (rank 0 only)"
    cfg["sampled"] = True
    return cfg


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    value, unit, cores, sample, dt = time_cpu(args.workload, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRICS[args.workload], "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": reference_config(args),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ workloads
def random_nvfp4(rows: int, k: int, dev, seed: int, sigma: float):
    """N(0, sigma) matrix quantised to NVFP4 by the CUDA quantiser in row chunks (keeps device memory small)."""
    import helion_b200 as hb

    gen = torch.Generator(device=dev).manual_seed(seed)
    codes = torch.empty(rows, k // 2, dtype=torch.uint8, device=dev)
    chunks = []
    g = torch.tensor(sigma * 6.0 / (6.0 * 448.0), device=dev, dtype=torch.float32)  # amax taken as 6 sigma
    for r0 in range(0, rows, 2048):
        r1 = min(rows, r0 + 2048)
        w = (torch.randn(r1 - r0, k, generator=gen, device=dev) * sigma).to(torch.bfloat16)
        c, s, _ = hb.nvfp4_quantize(w, g)
        codes[r0:r1] = c
        chunks.append(s.view(torch.uint8))
    return codes, torch.cat(chunks).view(torch.float8_e4m3fn), float(g)


def wl_gemm(args, dev, rank, world, timer):
    import helion_b200 as hb
    from helion_b200 import dist as D
    from oracle import oracle as O

    m, n, k = GEMM_CFG["m"], GEMM_CFG["n"], GEMM_CFG["k"]
    n_local = n // world
    host_a = torch.randn(m, k, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).pin_memory()
    a_dev = host_a.to(dev)
    ga = hb.layouts.nvfp4_global_scale(a_dev).reshape(1)
    a_codes, a_scales, _ = hb.nvfp4_quantize(a_dev, ga)
    b_codes, b_scales, gb = random_nvfp4(n_local, k, dev, 1000 + rank, 0.02)
    alpha = float(ga) * gb

    def gemm_only():
        return hb.nvfp4_scaled_matmul(a_codes, b_codes.t(), a_scales, b_scales, alpha=alpha)

    tp = ring = None
    if world > 1:
        tp = D.TensorParallel(dev)
        ring = tp.gathered_output(m, n, torch.bfloat16)

    def step():
        if world > 1:  # the GEMM's epilogue stores its columns into every rank's buffer; then a barrier kernel
            return tp.matmul(a_codes, a_scales, b_codes, b_scales, ring, alpha)
        return gemm_only()

    # parity on a slice, against the oracle
    y = gemm_only()
    ref = O.nvfp4_scaled_matmul(a_codes[:256].cpu(), b_codes[:256].cpu(), a_scales[: 256 * (k // 16)].cpu(),
                                b_scales[: 256 * (k // 16)].cpu(), torch.float32, alpha=alpha)
    parity = rel_err(y[:256, :256], ref)

    extra = {}
    if world > 1:
        extra["fused_equals_collective"] = bool(torch.equal(step(), D.all_gather_columns(y)))
    replay = graphed_ring(step) if world > 1 else graphed(step)[0]
    ms = timer.run(replay, args.steps, args.warmup)
    flops = 2 * m * n * k
    if world > 1:
        ms_gemm = timer.run(graphed(gemm_only)[0], args.steps, args.warmup)
        extra["gemm_only_ms"] = ms_gemm
        extra["nccl_gather_ms"] = timer.run(lambda: D.all_gather_columns(gemm_only()), max(3, args.steps // 4), 3)

    host_out = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        a = host_a.to(dev, non_blocking=True)
        c, s, _ = hb.nvfp4_quantize(a, ga)
        if world > 1:
            y = tp.matmul(c, s, b_codes, b_scales, ring, alpha)
        else:
            y = hb.nvfp4_scaled_matmul(c, b_codes.t(), s, b_scales, alpha=alpha)
        host_out.copy_(y, non_blocking=True)

    e2e_ms = timer.run(e2e_step, max(3, args.steps // 10), 3)
    peaks = measured_peaks()
    ach = 2 * m * n_local * k / (extra.get("gemm_only_ms", ms) * 1e-3) / 1e12
    roof = {
        "bound": "tensor", "kernel": "nvfp4_gemm_kernel", "launch": f"{m}x{n_local}x{k}",
        "achieved": ach, "peak": 4 * peaks["bf16_tflops"],
        "peak_kind": f"4 x {peaks['kind']} dense bf16 burst (e2m1 runs at four times the bf16 rate of the same pipe); nominal dense FP4 is 9000",
        "unit": "TFLOP/s", "frac": ach / (4 * peaks["bf16_tflops"]), "frac_of_nominal": ach / 9000.0,
        "traffic": ncu_traffic("gemm_8192"),
    }
    return dict(value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms=ms, e2e_value=flops / (e2e_ms * 1e-3) / 1e12,
                e2e_ms=e2e_ms, h2d=host_a.numel() * 2, d2h=host_out.numel() * 2, launches=1 + (1 if world > 1 else 0),
                roofline=roof, parity=parity, extra=extra,
                dtype="e2m1 x e2m1 with e4m3 block scales, fp32 accumulate, bf16 out",
                config={"workload": "gemm", "m": m, "n": n, "k": k, "parallelism": f"column-tp{world}" if world > 1 else "single",
                        "l2": "flushed between steps"})


def wl_gemv(args, dev, rank, world, timer):
    import helion_b200 as hb
    from helion_b200 import dist as D
    from oracle import oracle as O

    batch = args.batch
    # the kernel family the step runs on: with peers a single row stays on the SIMT kernel (dist.TensorParallel.gemv)
    used_path = "simt" if (world > 1 and batch == 1) else hb.ops._gemv_path(args.path, 57344 // world, 8192, batch)
    mats = {}
    for i, (name, (n, k)) in enumerate(LAYER_70B.items()):
        c, s, g = random_nvfp4(n // world, k, dev, 4000 + 16 * i + rank, 0.02)
        mats[name] = (c, s, g, n, k)
    gen = torch.Generator().manual_seed(4)
    host_x = {nm: torch.randn(batch, k, generator=gen).to(torch.bfloat16).pin_memory() for nm, (_, k) in LAYER_70B.items()}
    dev_x = {nm: t.to(dev) for nm, t in host_x.items()}

    def one(name, x):
        c, s, g, n, k = mats[name]
        path = used_path if world > 1 else args.path  # with peers: the family the fused kernels run on
        if batch == 1:
            return hb.nvfp4_gemv_bf16in(c, x.reshape(-1), s, g, path=path).reshape(1, -1)
        return hb.nvfp4_gemv_bf16in_batched(c, x, s, g, path=path)

    tp = None
    rings = {}
    if world > 1:
        tp = D.TensorParallel(dev)
        rings = {nm: tp.gathered_output(batch, n, torch.bfloat16) for nm, (n, _) in LAYER_70B.items()}

    def layer(xs):
        outs = {}
        for name in mats:
            if world > 1:  # the kernel stores its slice into every rank's buffer; a barrier kernel follows
                c, s, g, n, k = mats[name]
                outs[name] = tp.gemv(c, s, xs[name], rings[name], g)
            else:
                outs[name] = one(name, xs[name])
        return outs

    c, s, g, n, k = mats["o"]
    y = one("o", dev_x["o"])[0, :256]
    ref = O.nvfp4_gemv_bf16in(c[:256].cpu(), host_x["o"][0], s[: 256 * (k // 16)].cpu(), g) if batch == 1 else \
        O.nvfp4_gemm_bf16in(c[:256].cpu(), host_x["o"], s[: 256 * (k // 16)].cpu(), g)[0]
    parity = rel_err(y, ref)

    extra = {}
    if world > 1:
        fused = layer(dev_x)
        extra["fused_equals_collective"] = all(
            bool(torch.equal(fused[nm], D.all_gather_columns(one(nm, dev_x[nm])))) for nm in mats)
    step = graphed_ring(lambda: layer(dev_x)) if world > 1 else graphed(lambda: layer(dev_x))[0]
    ms = timer.run(step, args.steps, args.warmup)
    layer_bytes = sum(gemv_bytes(n, k, batch) for n, k in LAYER_70B.values())

    per_matrix = {}
    if world == 1:
        for name, (n, k) in LAYER_70B.items():
            r = graphed(lambda name=name: one(name, dev_x[name]))[0]
            t = timer.run(r, max(10, args.steps // 4), 3)
            per_matrix[name] = {"us": t * 1e3, "GBps": gemv_bytes(n, k, batch) / (t * 1e-3) / 1e9}

    host_out = {nm: torch.empty(batch, n, dtype=torch.bfloat16).pin_memory() for nm, (n, _) in LAYER_70B.items()}

    def e2e_step():
        outs = layer({nm: t.to(dev, non_blocking=True) for nm, t in host_x.items()})
        for nm, y in outs.items():
            host_out[nm].copy_(y, non_blocking=True)

    e2e_ms = timer.run(e2e_step, args.steps, 3)
    peaks = measured_peaks()
    roof = None
    if per_matrix:
        ach = per_matrix["gate_up"]["GBps"]
        roof = {"bound": "hbm", "kernel": {"simt": "nvfp4_gemv_kernel", "mma": "nvfp4_gemv_batched_kernel", "tc": "nvfp4_gemv_tc_kernel"}[
                    used_path] if not (batch > 1 and args.path == "simt") else "nvfp4_gemv_batched_kernel",
                "launch": f"gate_up 57344x8192 M={batch}", "achieved": ach, "peak": peaks["hbm_gbs"],
                "peak_kind": f"{peaks['kind']} copy bandwidth", "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                # the tensor-core kernel was captured with 8 rows; the weights are all but 0.1 % of its traffic
                "traffic": ncu_traffic("gemv_gate_up_m8" if used_path == "tc"
                                       else f"gemv_gate_up_m{batch}")}
    return dict(value=layer_bytes / (ms * 1e-3) / 1e12, unit="TB/s", ms=ms, e2e_value=layer_bytes / (e2e_ms * 1e-3) / 1e12,
                e2e_ms=e2e_ms, h2d=sum(2 * batch * k for _, k in LAYER_70B.values()),
                d2h=sum(2 * batch * n for n, _ in LAYER_70B.values()), launches=4 * ((2 if world > 1 else 1) + (1 if used_path == "tc" else 0)),
                roofline=roof, parity=parity, extra={"per_matrix": per_matrix, **extra},
                dtype=("e2m1 x e2m1 block-scaled tensor-core products, fp32 accumulate (bf16 activations as four NVFP4 "
                       "terms, bf16 out)" if used_path == "tc"
                       else "fp16 products, fp32 accumulate (e2m1 x e4m3 weights, bf16 in/out)"),
                config={"workload": "gemv", "layer": "qkv 10240x8192, o 8192x8192, gate_up 57344x8192, down 8192x28672",
                        "batch": batch, "path": args.path, "parallelism": f"column-tp{world}" if world > 1 else "single",
                        "l2": "flushed between steps; 481 MB of weights per step", "bytes_per_step": layer_bytes})


def wl_quant(args, dev, rank, world, timer):
    import helion_b200 as hb
    from oracle import oracle as O

    t, h = 16384, 7168
    g = torch.Generator().manual_seed(2)
    host_x = torch.randn(t, h, generator=g).to(torch.bfloat16).pin_memory()
    w = (torch.rand(h, generator=g) + 0.5).to(torch.bfloat16).to(dev)
    x = host_x.to(dev)
    q = torch.empty(t, h, dtype=torch.float8_e4m3fn, device=dev)
    s = torch.empty(t, 1, dtype=torch.float32, device=dev)

    def step():
        hb.rms_norm_dynamic_per_token_quant(q, x, w, s, 1e-6)

    step()
    qo, so, _ = O.rms_norm_dynamic_per_token_quant(host_x[:64], w.cpu(), 1e-6)
    parity = float((q[:64].cpu().view(torch.uint8) != qo.view(torch.uint8)).float().mean())
    ms = timer.run(graphed(step)[0], args.steps, args.warmup)
    nbytes = 2 * t * h + 2 * h + t * h + 4 * t

    ops = {}
    i = 18432
    xs = torch.randn(t, 2 * i, device=dev, dtype=torch.bfloat16)
    qs = torch.empty(t, i, dtype=torch.float8_e4m3fn, device=dev)
    ss = torch.empty(t, i // 128, dtype=torch.float32, device=dev)
    r = graphed(lambda: hb.silu_and_mul_per_block_quant(qs, xs, ss, 128))[0]
    tm = timer.run(r, max(10, args.steps // 4), 3)
    b = 2 * t * 2 * i + t * i + 4 * t * (i // 128)
    ops["silu_and_mul_per_block_quant_16384x18432"] = {"us": tm * 1e3, "GBps": b / (tm * 1e-3) / 1e9}
    one = torch.tensor([0.5], device=dev)
    r = graphed(lambda: hb.silu_mul_fp8(xs, one))[0]
    tm = timer.run(r, max(10, args.steps // 4), 3)
    b = 2 * t * 2 * i + t * i
    ops["silu_mul_fp8_16384x18432"] = {"us": tm * 1e3, "GBps": b / (tm * 1e-3) / 1e9}
    del xs, qs, ss
    sg = torch.empty(t, h // 128, dtype=torch.float32, device=dev)
    r = graphed(lambda: hb.per_token_group_fp8_quant(x, q, sg, 128, 1e-10, -448.0, 448.0, False))[0]
    tm = timer.run(r, max(10, args.steps // 4), 3)
    b = 2 * t * h + t * h + 4 * t * (h // 128)
    ops["per_token_group_fp8_quant_16384x7168"] = {"us": tm * 1e3, "GBps": b / (tm * 1e-3) / 1e9}

    sb = torch.empty(t, h // 128, dtype=torch.float32, device=dev)
    r = graphed(lambda: hb.rms_norm_per_block_quant(q, x, w, sb, 1e-6, None, None, 128, False))[0]
    tm = timer.run(r, max(10, args.steps // 4), 3)
    b = 2 * t * h + 2 * h + t * h + 4 * t * (h // 128)
    ops["rms_norm_per_block_quant_16384x7168"] = {"us": tm * 1e3, "GBps": b / (tm * 1e-3) / 1e9}
    r = graphed(lambda: hb.dynamic_per_token_scaled_fp8_quant(q, x, s))[0]
    tm = timer.run(r, max(10, args.steps // 4), 3)
    b = 2 * t * h + t * h + 4 * t
    ops["dynamic_per_token_scaled_fp8_quant_16384x7168"] = {"us": tm * 1e3, "GBps": b / (tm * 1e-3) / 1e9}

    host_q = torch.empty(t, h, dtype=torch.uint8).pin_memory()

    def e2e_step():
        xd = host_x.to(dev, non_blocking=True)
        hb.rms_norm_dynamic_per_token_quant(q, xd, w, s, 1e-6)
        host_q.copy_(q.view(torch.uint8), non_blocking=True)

    e2e_ms = timer.run(e2e_step, max(3, args.steps // 10), 3)
    peaks = measured_peaks()
    ach = nbytes / (ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": "rms_norm_token_quant_kernel", "launch": f"{t}x{h}", "achieved": ach,
            "peak": peaks["hbm_gbs"], "peak_kind": f"{peaks['kind']} copy bandwidth", "unit": "GB/s",
            "frac": ach / peaks["hbm_gbs"], "traffic": ncu_traffic("rms_norm_16384x7168")}
    return dict(value=world * nbytes / (ms * 1e-3) / 1e12, unit="TB/s", ms=ms, e2e_value=world * nbytes / (e2e_ms * 1e-3) / 1e12,
                e2e_ms=e2e_ms, h2d=host_x.numel() * 2, d2h=host_q.numel(), launches=1, roofline=roof,
                parity=parity, extra={"ops": ops}, dtype="fp32 arithmetic, bf16 in, e4m3 out",
                config={"workload": "quant", "op": "rms_norm_dynamic_per_token_quant", "tokens": t, "hidden": h,
                        "parallelism": "replicas only" if world > 1 else "single", "l2": "flushed between steps"})


def wl_scaled_mm(args, dev, rank, world, timer):
    import math

    import helion_b200 as hb
    from oracle import oracle as O

    m = args.batch if args.batch > 1 else 16
    g = torch.Generator(device=dev).manual_seed(7)
    cases = []
    for k, n in SCALED_MM_KN:
        sc = 1.0 / math.sqrt(k)
        a = (sc * (0.5 + torch.rand(m, k, device=dev, generator=g))).to(torch.float8_e4m3fn)
        b = (sc * (0.5 + torch.rand(n, k, device=dev, generator=g))).to(torch.float8_e4m3fn).t()
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        sa = torch.rand(1, 1, device=dev, generator=g) + 0.5
        sb = torch.rand(1, 1, device=dev, generator=g) + 0.5
        bias = (0.5 * (torch.rand(n, device=dev, generator=g) - 0.5)).to(torch.bfloat16)
        cases.append((a, b, c, sa, sb, bias))
    nbytes = sum(scaled_mm_bytes(m, k, n) for k, n in SCALED_MM_KN)

    def step():
        for a, b, c, sa, sb, bias in cases:
            hb.scaled_mm(c, a, b, sa, sb, bias)

    step()
    a, b, c, sa, sb, bias = cases[1]
    parity = rel_err(c, O.scaled_mm(a.cpu(), b.cpu(), sa.cpu(), sb.cpu(), bias.cpu()))
    ms = timer.run(graphed(step)[0], args.steps, args.warmup)

    # the largest weight (5120 x 51200, 262 MB: larger than the L2) alone, for the roofline of the kernel
    big = cases[10]
    def four_big():
        for _ in range(4):
            hb.scaled_mm(big[2], big[0], big[1], big[3], big[4], big[5])

    big_ms = timer.run(graphed(four_big)[0], max(10, args.steps // 2), 3) / 4
    big_bytes = scaled_mm_bytes(m, *SCALED_MM_KN[10])
    # The same step through the library (torch._scaled_mm: cuBLASLt), and every shape eight times back to back
    # (weights under 126 MB stay in L2 there), ours and the library's, as context for the numbers above.
    def library_step():
        for a, b, c, sa, sb, bias in cases:
            torch._scaled_mm(a, b, scale_a=sa, scale_b=sb, bias=bias, out_dtype=torch.bfloat16)

    library_ms = timer.run(graphed(library_step)[0], args.steps, args.warmup)
    per_shape = {}
    for (k, n), cs in zip(SCALED_MM_KN, cases):
        def ours8(cs=cs):
            for _ in range(8):
                hb.scaled_mm(cs[2], cs[0], cs[1], cs[3], cs[4], cs[5])

        def library8(cs=cs):
            for _ in range(8):
                torch._scaled_mm(cs[0], cs[1], scale_a=cs[3], scale_b=cs[4], bias=cs[5], out_dtype=torch.bfloat16)

        t_ours = timer.run(graphed(ours8)[0], max(10, args.steps // 4), 3) / 8
        t_lib = timer.run(graphed(library8)[0], max(10, args.steps // 4), 3) / 8
        per_shape[f"{m}x{k}x{n}"] = {"us": t_ours * 1e3, "library_us": t_lib * 1e3}

    host_a = [cs[0].cpu().view(torch.uint8).pin_memory() for cs in cases]
    host_c = [torch.empty(m, n, dtype=torch.bfloat16).pin_memory() for _, n in SCALED_MM_KN]

    def e2e_step():
        for ha, hc, (a, b, c, sa, sb, bias) in zip(host_a, host_c, cases):
            a.view(torch.uint8).copy_(ha, non_blocking=True)
            hb.scaled_mm(c, a, b, sa, sb, bias)
            hc.copy_(c, non_blocking=True)

    e2e_ms = timer.run(e2e_step, max(3, args.steps // 5), 3)
    peaks = measured_peaks()
    ach = big_bytes / (big_ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": "fp8_scaled_mm_kernel", "launch": f"{m}x5120x51200, four back to back", "achieved": ach,
            "peak": peaks["hbm_gbs"], "peak_kind": f"{peaks['kind']} copy bandwidth", "unit": "GB/s",
            "frac": ach / peaks["hbm_gbs"], "traffic": ncu_traffic(f"scaled_mm_{m}x5120x51200")}
    return dict(value=world * nbytes / (ms * 1e-3) / 1e12, unit="TB/s", ms=ms,
                e2e_value=world * nbytes / (e2e_ms * 1e-3) / 1e12, e2e_ms=e2e_ms,
                h2d=sum(h.numel() for h in host_a), d2h=sum(h.numel() * 2 for h in host_c), launches=len(cases),
                roofline=roof, parity=parity,
                extra={"library_ms_per_step": library_ms, "shapes_back_to_back": per_shape}, dtype="e4m3 operands, fp32 accumulate, bf16 out",
                config={"workload": "scaled_mm", "tokens": m, "kn_shapes": len(SCALED_MM_KN),
                        "parallelism": "replicas only" if world > 1 else "single", "l2": "flushed between steps"})


def wl_moe(args, dev, rank, world, timer):
    import helion_b200 as hb  # noqa: F401
    from helion_b200 import dist as D
    from helion_b200 import moe as M

    c = MOE_CFG
    e_local = c["experts"] // world
    t_local = c["tokens"] // world

    def bundle(n, k, seed):
        codes, scales, g = random_nvfp4(e_local * n, k, dev, seed, 0.02)
        per = hb.swizzled_scale_numel(n, k // 16)
        assert scales.numel() == e_local * per
        return M.GroupedNvfp4Weight(codes.reshape(e_local, n, k // 2), scales.reshape(e_local, per),
                                    torch.full((e_local,), g, dtype=torch.float32, device=dev))

    # gate/up rows interleaved in blocks of 128: the first expert GEMM applies SiLU-mul in its epilogue
    w_gu = M.interleave_gate_up(bundle(2 * c["inter"], c["hidden"], 3000 + rank))
    w_d = bundle(c["hidden"], c["inter"], 3500 + rank)
    g = torch.Generator().manual_seed(3 + 97 * rank)
    host_x = torch.randn(t_local, c["hidden"], generator=g).to(torch.bfloat16).pin_memory()
    host_l = torch.randn(t_local, c["experts"], generator=g).pin_memory()
    x, logits = host_x.to(dev), host_l.to(dev)

    if world == 1:
        def step():
            return M.nvfp4_moe(x, logits, c["top_k"], w_gu, w_d)
    else:
        fn = D.make_nvfp4_expert_fn(w_gu, w_d)

        def step():
            return D.expert_parallel_moe(x, logits, c["top_k"], c["experts"], fn)

    y = step()
    parity = 0.0 if bool(torch.isfinite(y.float()).all()) else 1.0  # full parity is the test suite's; here: finite
    ms = timer.run(step, args.steps, args.warmup)
    host_out = torch.empty(t_local, c["hidden"], dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        xd, ld = host_x.to(dev, non_blocking=True), host_l.to(dev, non_blocking=True)
        if world == 1:
            out = M.nvfp4_moe(xd, ld, c["top_k"], w_gu, w_d)
        else:
            out = D.expert_parallel_moe(xd, ld, c["top_k"], c["experts"], fn)
        host_out.copy_(out, non_blocking=True)

    e2e_ms = timer.run(e2e_step, max(3, args.steps // 4), 3)
    flops = moe_flops()
    peaks = measured_peaks()
    ach = flops / world / (ms * 1e-3) / 1e12
    roof = {"bound": "tensor", "kernel": "nvfp4_gemm_kernel (grouped)", "launch": "whole MoE step (2 grouped GEMMs + quantisers + combine)",
            "achieved": ach, "peak": 4 * peaks["bf16_tflops"], "peak_kind": f"4 x {peaks['kind']} dense bf16 burst",
            "unit": "TFLOP/s", "frac": ach / (4 * peaks["bf16_tflops"]), "traffic": None}
    return dict(value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms=ms, e2e_value=flops / (e2e_ms * 1e-3) / 1e12, e2e_ms=e2e_ms,
                h2d=host_x.numel() * 2 + host_l.numel() * 4, d2h=host_out.numel() * 2, launches=9, roofline=roof,
                parity=parity, extra={}, dtype="e2m1 x e2m1 with e4m3 block scales, fp32 accumulate, bf16 activations",
                config={"workload": "moe", **c, "parallelism": f"ep{world}" if world > 1 else "single", "l2": "flushed between steps"})


WORKLOADS = {"gemm": wl_gemm, "gemv": wl_gemv, "quant": wl_quant, "moe": wl_moe, "scaled_mm": wl_scaled_mm}


def run_gpu(args) -> None:
    from helion_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    timer = Timer(dev, world)
    with ClockSampler(local) as clocks:
        r = WORKLOADS[args.workload](args, dev, rank, world, timer)
    torch.cuda.synchronize()
    status = lib.hb200_device_status(0)

    if rank == 0:
        cpu_v, cpu_unit, cores, sample, _ = time_cpu(args.workload)
        line = {
            "metric": METRICS[args.workload], "value": r["value"], "unit": r["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms"], "higher_is_better": True,
            "scaling": "strong" if args.workload not in ("quant", "scaled_mm") else "weak", "vs_baseline": None, "dtype": r["dtype"],
            "data": "synthetic", "config": r["config"],
            "e2e": {"value": r["e2e_value"], "unit": r["unit"], "h2d_bytes_per_step": r["h2d"],
                    "d2h_bytes_per_step": r["d2h"], "ms_per_step": r["e2e_ms"]},
            "gpu_launches": args.steps * r["launches"], "roofline": r["roofline"],
            "cpu_baseline": {"value": cpu_v, "unit": cpu_unit, "cores": cores, "kind": "port", "sample": sample},
            "clocks": clocks.summary(), "parity": {"max_rel_err_or_mismatch": r["parity"]}, "device_status": status,
        }
        line.update(r["extra"])
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "mma", "tc"],
                    help="GEMV kernel family (gemv workload): auto = tensor cores for 1..32 rows of a large weight")
    ap.add_argument("--profile-region", type=int, default=0,
                    help="which timed region (0 = the headline one) cudaProfilerStart/Stop brackets, for "
                         "`ncu --profile-from-start off`")
    ap.add_argument("--flush", default="write+read", choices=["write+read", "write"],
                    help="L2 flush between steps: a 256 MB write followed by a 256 MB read (no dirty lines left), or the write alone")
    args = ap.parse_args()
    Timer.profile_region = args.profile_region
    Timer.flush_read = args.flush == "write+read"
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(3, args.warmup)
    run_gpu(args)


if __name__ == "__main__":
    main()
