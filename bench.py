"""Benchmark driver: ``python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]``.

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of synthetic input, with the
inputs already resident in HBM; ``e2e`` repeats it through the public operator API from pinned host buffers.

Workloads (``--workload``):
  all    (default) the headline is ``gemm``; the same JSON line carries a ``workloads`` object with every other
         configuration measured in the same run (the 8192 x 4096 GEMV, the decode sweep over 1..32 rows, the
         shapes the reference publishes GEMV times for, the quant producers, the MoE layer, scaled_mm), each
         with microseconds (mean and median), achieved throughput, roofline fraction, a parity figure against
         the oracle and, where a library kernel exists, its time under the same protocol.
  gemm   dense NVFP4 GEMM, M=N=K=8192 (seed 1): A ~ N(0,1) bf16 and B ~ N(0,0.02) fp32, both quantised to NVFP4
         (16-wide blocks, e4m3 scales, fp32 global scale amax / (6 * 448)); bf16 output; metric TFLOP/s.  With N
         GPUs the rows of B (output columns) are split evenly and the outputs all-gathered.
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
ranks; the median over the K steps (the reference's protocol: median of CUDA-graph replays with the L2 cleared
before each, pretuned_kernels/_bench.py:50-64) is reported beside it.  Steps whose launch sequence is fixed are replayed from a CUDA graph so that the host does not sit
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


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the headline kernels are read from the
# ncu summaries kept under profiles/: each holds a line "dram_bytes_per_launch[<key>] = <bytes>".
def ncu_traffic(key: str):
    import re

    pat = re.compile(r"dram_bytes_per_launch\[" + re.escape(key) + r"\]\s*=\s*([0-9.eE+]+)")
    for f in sorted((ROOT / "profiles").glob("*.md")):
        m = pat.search(f.read_text())
        if m:
            return float(m.group(1))
    return None


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
        self.last_median = None  # median milliseconds of the last run() (max over ranks)

    def run2(self, step, steps: int, warmup: int) -> tuple[float, float]:
        """(mean, median) milliseconds per step."""
        mean = self.run(step, steps, warmup)
        return mean, self.last_median

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
        times = sorted(s.elapsed_time(e) for s, e in pairs)
        ms = sum(times) / steps
        med = times[steps // 2] if steps % 2 else 0.5 * (times[steps // 2 - 1] + times[steps // 2])
        if self.world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms, med], device=self.dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, med = float(t[0]), float(t[1])
        self.last_median = med
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
def config1_operands():
    """Config 1's operands as the configuration states them: seed 1, A ~ N(0,1) bf16 [8192, 8192], then
    B ~ N(0, 0.02) fp32 [8192, 8192], drawn from one CPU generator so that the oracle and the GPU see identical bits."""
    g = torch.Generator().manual_seed(1)
    a = torch.randn(GEMM_CFG["m"], GEMM_CFG["k"], generator=g).to(torch.bfloat16)
    b = torch.randn(GEMM_CFG["n"], GEMM_CFG["k"], generator=g) * 0.02
    return a, b


def cpu_gemm(seconds: float = 8.0):
    """Oracle port of reference_nvfp4_w4a4_matmul semantics (dequantise -> fp32 matmul) on the first 1024 rows of
    config 1's seeded A and B, quantised by the oracle with the whole tensors' global scales."""
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    m = n = 1024
    k = GEMM_CFG["k"]
    a_full, b_full = config1_operands()
    ga = a_full.float().abs().amax() / (6.0 * 448.0)
    gb = b_full.abs().amax() / (6.0 * 448.0)
    a, sa, _ = O.nvfp4_quantize(a_full[:m], ga)
    b, sb, _ = O.nvfp4_quantize(b_full[:n], gb)
    alpha = float(ga) * float(gb)
    del a_full, b_full

    def step():
        return O.nvfp4_scaled_matmul(a, b, sa, sb, alpha=alpha)

    return step, 2 * m * n * k, (f"rows [0, {m}) of the seeded A and B of the 8192^3 GEMM ({m}x{n}x{k}: dequantise -> "
                                 "fp32 matmul -> bf16)")


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


CPU_WORKLOADS = {"all": (cpu_gemm, 1e12, "TFLOP/s"), "gemm": (cpu_gemm, 1e12, "TFLOP/s"), "gemv": (cpu_gemv, 1e12, "TB/s"), "quant": (cpu_quant, 1e12, "TB/s"),
                 "moe": (cpu_moe, 1e12, "TFLOP/s"), "scaled_mm": (cpu_scaled_mm, 1e12, "TB/s")}
METRICS = {"all": "nvfp4_gemm_tflops", "gemm": "nvfp4_gemm_tflops", "gemv": "nvfp4_gemv_hbm_throughput", "quant": "fp8_quant_producer_hbm_throughput",
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
    """The configuration of the matching GPU arm, key for key (the CPU arm times a bounded sample of it, described in
    cpu_baseline.sample)."""
    world = max(1, args.gpus)
    if args.workload in ("all", "gemm"):
        return {"workload": "gemm", **GEMM_CFG, "seed": 1,
                "parallelism": f"column-tp{world}" if world > 1 else "single", "l2": "flushed between steps"}
    if args.workload == "gemv":
        cfg = {"workload": "gemv", "layer": "qkv 10240x8192, o 8192x8192, gate_up 57344x8192, down 8192x28672", "batch": args.batch}
    elif args.workload == "moe":
        cfg = {"workload": "moe", **MOE_CFG}
    elif args.workload == "scaled_mm":
        cfg = {"workload": "scaled_mm", "tokens": args.batch if args.batch > 1 else 16, "kn_shapes": len(SCALED_MM_KN)}
    else:
        cfg = {"workload": "quant", "tokens": 16384, "hidden": 7168, "op": "rms_norm_dynamic_per_token_quant"}
    cfg["parallelism"] = "host cores (rank 0 only)"
    return cfg


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    value, unit, cores, sample, dt = time_cpu(args.workload, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRICS[args.workload], "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (dequantise, then fp32 matmul)", "data": "synthetic",
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


def quantize_weight_rows(w_fp32_cpu: torch.Tensor, g: torch.Tensor, dev, chunk: int = 1024):
    """fp32 weight rows -> NVFP4 (codes, swizzled scales) on the device with the tensor-code quantiser of
    helion_b200.layouts (weight preparation, not a timed path), in row chunks to bound temporaries."""
    import helion_b200 as hb

    rows, k = w_fp32_cpu.shape
    codes = torch.empty(rows, k // 2, dtype=torch.uint8, device=dev)
    scales = []
    gd = g.to(dev)
    for r0 in range(0, rows, chunk):
        c, sc, _ = hb.layouts.nvfp4_quantize_host(w_fp32_cpu[r0 : r0 + chunk].to(dev), gd)
        codes[r0 : r0 + chunk] = c
        scales.append(sc.view(torch.uint8))
    return codes, torch.cat(scales).view(torch.float8_e4m3fn)


def library_nvfp4_gemm(a_codes, b_codes, a_scales, b_scales):
    """The library kernel for the same operands: torch._scaled_mm (cuBLASLt block-scaled FP4), as the reference's
    nvfp4_scaled_matmul calls it (examples/nvfp4_gemm.py:358-364).  Returns a callable or None when unavailable."""
    fp4 = getattr(torch, "float4_e2m1fn_x2", None)
    if fp4 is None:
        return None
    a, bt = a_codes.view(fp4), b_codes.view(fp4).t()

    def call():
        return torch._scaled_mm(a, bt, a_scales.reshape(-1), b_scales.reshape(-1), out_dtype=torch.bfloat16)

    try:
        call()
        torch.cuda.synchronize()
    except Exception:
        return None
    return call


def wl_gemm(args, dev, rank, world, timer):
    import helion_b200 as hb
    from helion_b200 import dist as D
    from oracle import oracle as O

    m, n, k = GEMM_CFG["m"], GEMM_CFG["n"], GEMM_CFG["k"]
    n_local = n // world
    a_cpu, b_cpu = config1_operands()
    host_a = a_cpu.pin_memory()
    a_dev = host_a.to(dev)
    ga = hb.layouts.nvfp4_global_scale(a_dev).reshape(1)
    a_codes, a_scales, _ = hb.nvfp4_quantize(a_dev, ga)
    gb = b_cpu.abs().amax() / torch.tensor(6.0 * 448.0)
    lo = rank * n_local
    b_codes, b_scales = quantize_weight_rows(b_cpu[lo : lo + n_local], gb, dev)
    alpha = float(ga) * float(gb)

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

    # parity: the quantised operands against the oracle's quantiser on the same seeded rows (bit for bit), and a
    # 256 x 256 block of the product against dequantise-then-fp32-matmul
    y = gemm_only()
    oa, osa, _ = O.nvfp4_quantize(a_cpu[:256], ga.cpu().reshape(()))
    ob, osb, _ = O.nvfp4_quantize(b_cpu[lo : lo + 256], gb)
    cs = 256 * (k // 16)
    operands_exact = bool(torch.equal(oa, a_codes[:256].cpu()) and torch.equal(ob, b_codes[:256].cpu())
                          and torch.equal(osa.view(torch.uint8), a_scales.view(torch.uint8)[:cs].cpu())
                          and torch.equal(osb.view(torch.uint8), b_scales.view(torch.uint8)[:cs].cpu()))
    ref = O.nvfp4_scaled_matmul(oa, ob, osa, osb, torch.float32, alpha=alpha)
    parity = rel_err(y[:256, :256], ref)
    del a_cpu, b_cpu

    extra = {"operands_bit_identical_to_oracle_quantiser": operands_exact}
    if world > 1:
        extra["fused_equals_collective"] = bool(torch.equal(step(), D.all_gather_columns(y)))
    replay = graphed_ring(step) if world > 1 else graphed(step)[0]
    ms, med = timer.run2(replay, args.steps, args.warmup)
    flops = 2 * m * n * k
    extra["median_ms_per_step"] = med
    if world > 1:
        ms_gemm = timer.run(graphed(gemm_only)[0], args.steps, args.warmup)
        extra["gemm_only_ms"] = ms_gemm
        extra["nccl_gather_ms"] = timer.run(lambda: D.all_gather_columns(gemm_only()), max(3, args.steps // 4), 3)

    # the library on the same operands, same protocol (this rank's slice)
    lib_call = library_nvfp4_gemm(a_codes, b_codes, a_scales, b_scales)
    lib_ms = None
    if lib_call is not None:
        lib_ms, lib_med = timer.run2(graphed(lib_call)[0], args.steps, args.warmup)
        extra["library"] = {"kernel": "torch._scaled_mm (cuBLASLt NVFP4)", "launch": f"{m}x{n_local}x{k}", "ms": lib_ms,
                            "median_ms": lib_med, "tflops": 2 * m * n_local * k / (lib_ms * 1e-3) / 1e12,
                            "max_abs_diff_vs_ours": float((lib_call().float() * alpha - y.float()).abs().max())}

    host_out = torch.empty(m, n_local, dtype=torch.bfloat16).pin_memory()
    m_slice = m // world
    a_part = torch.empty(m_slice, k, dtype=torch.bfloat16, device=dev)
    gathered_codes = torch.empty(m, k // 2, dtype=torch.uint8, device=dev)
    gathered_scales = torch.empty(a_scales.numel(), dtype=torch.uint8, device=dev)

    host_pipeline = hb.HostPipelinedMatmul(b_codes, b_scales, ga, alpha, m, chunks=8) if world == 1 else None

    def e2e_step():
        # whole job: A crosses PCIe once (every rank takes m / world rows, quantises them and the ranks all-gather
        # the packed rows over NVLink), D crosses once (every rank copies back the columns it computed)
        if world > 1:
            import torch.distributed as dist

            a_part.copy_(host_a[rank * m_slice : (rank + 1) * m_slice], non_blocking=True)
            c, sc, _ = hb.nvfp4_quantize(a_part, ga)
            dist.all_gather_into_tensor(gathered_codes, c)
            dist.all_gather_into_tensor(gathered_scales, sc.view(torch.uint8))
            y = tp.matmul(gathered_codes, gathered_scales.view(torch.float8_e4m3fn), b_codes, b_scales, ring, alpha)
            host_out.copy_(y[:, lo : lo + n_local], non_blocking=True)
        else:
            # rows in eight chunks: the copy in of the next chunk, quantiser + GEMM of this one and the copy out of the
            # one before overlap on three streams (every byte still crosses PCIe inside the timed region)
            host_pipeline(host_a, host_out)

    if world > 1:
        e2e_step()
        extra["e2e_equals_resident"] = bool(torch.equal(ring.locals[(ring.turn - 1) % len(ring.locals)], step()))
    else:
        e2e_step()
        torch.cuda.synchronize()
        extra["e2e_equals_resident"] = bool(torch.equal(host_out.to(dev), step()))
    e2e_ms = timer.run(e2e_step, max(3, args.steps // 10), 3)
    peaks = measured_peaks()
    ach = 2 * m * n_local * k / (extra.get("gemm_only_ms", ms) * 1e-3) / 1e12
    roof = {
        "bound": "tensor", "kernel": "nvfp4_gemm_pair_kernel", "launch": f"{m}x{n_local}x{k}",
        "achieved": ach, "peak": 4 * peaks["bf16_tflops"],
        "peak_kind": f"4 x {peaks['kind']} dense bf16 burst (e2m1 runs at four times the bf16 rate of the same pipe); "
                     "nominal dense FP4 is 9000; no FP4 figure is in MEASURED_PEAKS.json",
        "unit": "TFLOP/s", "frac": ach / (4 * peaks["bf16_tflops"]), "frac_of_nominal_fp4": ach / 9000.0,
        "frac_of_library": (lib_ms / extra.get("gemm_only_ms", ms)) if lib_ms else None,
        "traffic": ncu_traffic("nvfp4_gemm_pair_kernel 8192x8192x8192") if world == 1 else None,
    }
    return dict(value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms=ms, e2e_value=flops / (e2e_ms * 1e-3) / 1e12,
                e2e_ms=e2e_ms, h2d=host_a.numel() * 2, d2h=m * n * 2, launches=1 + (1 if world > 1 else 0),
                roofline=roof, parity=parity, extra=extra,
                dtype="e2m1 x e2m1 with e4m3 block scales, fp32 accumulate, bf16 out",
                config={"workload": "gemm", "m": m, "n": n, "k": k, "seed": 1,
                        "parallelism": f"column-tp{world}" if world > 1 else "single", "l2": "flushed between steps"})


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

    # The reference gates these kernels on their speed-up over the best of torch eager and torch.compile
    # (test/test_pretuned_kernels.py:325-346, H100 figures only).  torch eager, the modules' own torch expressions
    # written out here, is timed beside each operator on this device at the same size (its fp32 temporaries take a
    # few GB).
    fp8 = torch.float8_e4m3fn
    te, scale_up = t, 1.0

    def eager_rms():
        xf = x[:te].float()
        xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * w
        sc = (xn.float().abs().amax(-1, keepdim=True) * (1.0 / 448.0)).clamp(min=1.0 / (448.0 * 512.0))
        return (xn.float() / sc).clamp(-448.0, 448.0).to(fp8), sc

    def eager_group():
        xg = x[:te].float().reshape(te, h // 128, 128)
        sc = xg.abs().amax(-1, keepdim=True).clamp(min=1e-10) / 448.0
        return (xg / sc).clamp(-448.0, 448.0).to(fp8), sc

    xs_e = torch.randn(te, 2 * i, device=dev, dtype=torch.bfloat16)

    def eager_silu():
        a, bb = xs_e[:, :i].float(), xs_e[:, i:].float()
        y = (a * torch.sigmoid(a) * bb).reshape(te, i // 128, 128)
        sc = (y.abs().amax(-1) * (1.0 / 448.0)).clamp(min=1.0 / (448.0 * 512.0))
        return (y / sc[:, :, None]).clamp(-448.0, 448.0).to(fp8), sc

    def eager_dyn():
        xf = x[:te].float()
        sc = (xf.abs().amax(-1, keepdim=True) * (1.0 / 448.0)).clamp(min=1.0 / (448.0 * 512.0))
        return (xf * (1.0 / sc)).clamp(-448.0, 448.0).to(fp8), sc

    eager = {}
    for name, fn, ours_us in (("rms_norm_dynamic_per_token_quant_16384x7168", eager_rms, ms * 1e3),
                              ("per_token_group_fp8_quant_16384x7168", eager_group, None),
                              ("silu_and_mul_per_block_quant_16384x18432", eager_silu, None),
                              ("dynamic_per_token_scaled_fp8_quant_16384x7168", eager_dyn, None)):
        tm = timer.run(graphed(fn)[0], 5, 2) * 1e3 * scale_up
        ours = ours_us if ours_us is not None else ops[name]["us"]
        eager[name] = {"torch_eager_us": tm, "ours_us": ours, "speedup": tm / ours}
    del xs_e

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
                parity=parity, extra={"ops": ops, "vs_torch_eager": eager}, dtype="fp32 arithmetic, bf16 in, e4m3 out",
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
    # a prefill-sized call (8192 tokens: the CTA-pair kernel), two launches per step; timed region 3
    pm, pk, pn = SCALED_MM_PREFILL[-1]
    pa = (torch.randn(pm, pk, device=dev, generator=g) / math.sqrt(pk)).to(torch.float8_e4m3fn)
    pb = (torch.randn(pn, pk, device=dev, generator=g) / math.sqrt(pk)).to(torch.float8_e4m3fn).t()
    psa, psb = torch.rand(pm, 1, device=dev, generator=g) + 0.5, torch.rand(pn, device=dev, generator=g) + 0.5
    pc = torch.empty(pm, pn, dtype=torch.bfloat16, device=dev)

    def two_prefill():
        hb.scaled_mm(pc, pa, pb, psa, psb)
        hb.scaled_mm(pc, pa, pb, psa, psb)

    prefill_ms = timer.run(graphed(two_prefill)[0], max(5, args.steps // 4), 3) / 2
    prefill = {"shape": f"{pm}x{pk}x{pn}", "us": prefill_ms * 1e3, "TFLOPs": 2.0 * pm * pn * pk / (prefill_ms * 1e-3) / 1e12,
               "traffic": ncu_traffic(f"scaled_mm_prefill_{pm}x{pk}x{pn}")}
    del pa, pb, pc
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
                extra={"library_ms_per_step": library_ms, "shapes_back_to_back": per_shape, "prefill": prefill},
                dtype="e4m3 operands, fp32 accumulate, bf16 out",
                config={"workload": "scaled_mm", "tokens": m, "kn_shapes": len(SCALED_MM_KN),
                        "parallelism": "replicas only" if world > 1 else "single", "l2": "flushed between steps"})


def wl_moe(args, dev, rank, world, timer):
    """Config 3 as the headline: one GPU (sampled comparison with the oracle) or expert-parallel (compared, on
    rank 0, with the one-GPU layer on all tokens and experts)."""
    import helion_b200 as hb  # noqa: F401
    from helion_b200 import dist as D
    from helion_b200 import moe as M

    c = MOE_CFG
    rec = sub_moe(args, dev, timer) if world == 1 else sub_ep_moe(args, dev, rank, world, timer)
    ms = rec["us"] * 1e-3
    # end to end: tokens and logits from pinned host memory, the result back
    t_local = c["tokens"] // world
    g = torch.Generator().manual_seed(3 + 97 * rank)
    host_x = torch.randn(t_local, c["hidden"], generator=g).to(torch.bfloat16).pin_memory()
    host_l = torch.randn(t_local, c["experts"], generator=g).pin_memory()
    e_local = c["experts"] // world
    w_gu = M.interleave_gate_up(seeded_expert_bundle(e_local, 2 * c["inter"], c["hidden"], 3000 + rank, dev))
    w_d = seeded_expert_bundle(e_local, c["hidden"], c["inter"], 3500 + rank, dev)
    ep = D.ExpertParallel(dev, t_local, c["hidden"], c["top_k"], c["experts"]) if world > 1 else None
    host_out = torch.empty(t_local, c["hidden"], dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        xd, ld = host_x.to(dev, non_blocking=True), host_l.to(dev, non_blocking=True)
        out = M.nvfp4_moe(xd, ld, c["top_k"], w_gu, w_d) if world == 1 else ep.moe(xd, ld, w_gu, w_d)
        host_out.copy_(out, non_blocking=True)

    e2e_ms = timer.run(e2e_step, max(3, args.steps // 4), 3)
    flops = moe_flops()
    peaks = measured_peaks()
    ach = flops / world / (ms * 1e-3) / 1e12
    roof = {"bound": "tensor", "kernel": "nvfp4_gemm_kernel (grouped)", "launch": "whole MoE step (2 grouped GEMMs + quantisers + combine)",
            "achieved": ach, "peak": 4 * peaks["bf16_tflops"], "peak_kind": f"4 x {peaks['kind']} dense bf16 burst",
            "unit": "TFLOP/s", "frac": ach / (4 * peaks["bf16_tflops"]), "frac_of_nominal_fp4": ach / 9000.0, "traffic": None}
    parity = rec.get("parity") or {}
    return dict(value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s", ms=ms, e2e_value=flops / (e2e_ms * 1e-3) / 1e12, e2e_ms=e2e_ms,
                h2d=world * (host_x.numel() * 2 + host_l.numel() * 4), d2h=world * host_out.numel() * 2, launches=14, roofline=roof,
                parity=parity.get("max_rel_err", parity.get("max_rel_err_vs_one_gpu")), extra={"moe": rec},
                dtype="e2m1 x e2m1 with e4m3 block scales, fp32 accumulate, bf16 activations",
                config={"workload": "moe", **c, "seed": 3, "parallelism": f"ep{world}" if world > 1 else "single", "l2": "flushed between steps"})


# ------------------------------------------------------------------ the other configurations, as sub-records
HBM_NOMINAL_GBS = 8000.0  # the "about 8 TB/s" the target is quoted against
# (N, K) the reference publishes GEMV times for, with its figures in microseconds (Helion Triton kernels, B200,
# CUDA graph, L2 cleared per replay, median): pretuned_kernels/nvfp4_gemv/_helion_aot_nvfp4_gemv_cuda_sm100.py:20-22,
# 30-31, 65, 93, 104
PUBLISHED_GEMV = {
    (8192, 28672): {"w4a16_us": 58.04, "w4a4_us": 38.8},
    (15360, 5120): {"w4a16_us": 17.70, "w4a4_us": 15.32},
    (28672, 4096): {"w4a16_us": 28.12, "w4a4_us": None},
}


def protocol_floor_us(timer) -> float:
    """What this timing protocol reads for a kernel that does nothing (one graph replay of a one-element add between
    an event pair, L2 flushed before): the part of every small figure that is not the kernel's."""
    t = torch.zeros(1, device=timer.dev)
    _, med = timer.run2(graphed(lambda: t.add_(1))[0], 30, 3)
    return med * 1e3


def in_graph_us(timer, fn, reps: int = 10, rounds: int = 7) -> float:
    """Per-call microseconds under the reference's protocol (tritonbench's CUDA-graph timer as
    pretuned_kernels/_bench.py:50-64 uses it): ONE graph holds `reps` x (L2 clear, call), its time minus that of a
    graph with the clears alone, divided by `reps`; median over `rounds` replays.  Launch and event overheads of a
    single replay are not charged to the kernel."""
    def with_calls():
        for _ in range(reps):
            timer.flush_buf.zero_()
            fn()

    def clears_only():
        for _ in range(reps):
            timer.flush_buf.zero_()

    g_calls, g_clear = graphed(with_calls)[0], graphed(clears_only)[0]

    def med(replay):
        ts = []
        for _ in range(rounds):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[rounds // 2]

    return (med(g_calls) - med(g_clear)) / reps * 1e3


def hbm_record(ms: float, med: float, nbytes: int, **more) -> dict:
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"us": ms * 1e3, "median_us": med * 1e3, "bytes": nbytes, "GBps": gbs,
            "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "frac_of_8TBps": gbs / HBM_NOMINAL_GBS, **more}


def tensor_record(ms: float, med: float, flops: int, **more) -> dict:
    peaks = measured_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    return {"us": ms * 1e3, "median_us": med * 1e3, "flops": flops, "TFLOPs": tf,
            "frac_of_4x_measured_bf16": tf / (4 * peaks["bf16_tflops"]), "frac_of_nominal_fp4": tf / 9000.0, **more}


def cpu_port(workload: str, budget_s: float = 3.0) -> dict:
    v, unit, cores, sample, _ = time_cpu(workload, budget_s=budget_s)
    return {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample}


def sub_gemv_config0(args, dev, timer) -> dict:
    """Config 0: W fp32 [8192, 4096] ~ N(0, 0.02) quantised as stated, x bf16 [4096] ~ N(0, 1), seed 0."""
    import helion_b200 as hb
    from oracle import oracle as O

    n, k = 8192, 4096
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g) * 0.02
    gw = w.abs().amax() / torch.tensor(6.0 * 448.0)
    codes, scales = quantize_weight_rows(w, gw, dev)
    xd = x.reshape(-1).to(dev)
    steps = max(20, args.steps)
    out = {"shape": f"{n}x{k}", "seed": 0, "empty_kernel_under_this_protocol_us": protocol_floor_us(timer)}
    ref = O.nvfp4_gemv_bf16in(codes[:1024].cpu(), x.reshape(-1), scales.reshape(-1)[: 1024 * (k // 16)].cpu(), float(gw))
    for path in ("auto", "simt"):
        y = hb.nvfp4_gemv_bf16in(codes, xd, scales, float(gw), path=path)
        ms, med = timer.run2(graphed(lambda path=path: hb.nvfp4_gemv_bf16in(codes, xd, scales, float(gw), path=path))[0], steps, 3)
        out[f"bf16in_{path}"] = hbm_record(
            ms, med, gemv_bytes(n, k), parity_max_rel_err=rel_err(y[:1024], ref), kernel=hb.ops._gemv_path(path, n, k, 1),
            in_graph_protocol_us=in_graph_us(timer, lambda path=path: hb.nvfp4_gemv_bf16in(codes, xd, scales, float(gw), path=path)))
    xq, xs, gx = hb.nvfp4_quantize(xd.reshape(1, -1), hb.layouts.nvfp4_global_scale(xd).reshape(1))
    alpha = float(gw) * float(gx)
    y4 = hb.nvfp4_gemv_fp4in(codes, xq.reshape(-1), scales, xs, alpha)
    ref4 = O.nvfp4_gemv_fp4in(codes[:1024].cpu(), xq.reshape(-1).cpu(), scales.reshape(-1)[: 1024 * (k // 16)].cpu(), xs.cpu(), alpha)
    ms, med = timer.run2(graphed(lambda: hb.nvfp4_gemv_fp4in(codes, xq.reshape(-1), scales, xs, alpha))[0], steps, 3)
    out["fp4in"] = hbm_record(ms, med, gemv_bytes(n, k) - k - k // 2 + k // 16, parity_max_rel_err=rel_err(y4[:1024], ref4),
                              in_graph_protocol_us=in_graph_us(timer, lambda: hb.nvfp4_gemv_fp4in(codes, xq.reshape(-1), scales, xs, alpha)))
    return out


def sub_gemv_published_shapes(args, dev, timer) -> dict:
    import helion_b200 as hb

    out = {}
    steps = max(20, args.steps)
    for i, ((n, k), pub) in enumerate(PUBLISHED_GEMV.items()):
        codes, scales, gw = random_nvfp4(n, k, dev, 7000 + i, 0.02)
        x = torch.randn(k, generator=torch.Generator().manual_seed(70 + i)).to(torch.bfloat16).to(dev)
        xq, xs, gx = hb.nvfp4_quantize(x.reshape(1, -1), hb.layouts.nvfp4_global_scale(x).reshape(1))
        ms, med = timer.run2(graphed(lambda: hb.nvfp4_gemv_bf16in(codes, x, scales, gw))[0], steps, 3)
        rec = {"w4a16": hbm_record(ms, med, gemv_bytes(n, k), reference_published_us=pub["w4a16_us"],
                                   in_graph_protocol_us=in_graph_us(timer, lambda: hb.nvfp4_gemv_bf16in(codes, x, scales, gw)))}
        alpha4 = gw * float(gx)
        ms, med = timer.run2(graphed(lambda: hb.nvfp4_gemv_fp4in(codes, xq.reshape(-1), scales, xs, alpha4))[0], steps, 3)
        rec["w4a4"] = hbm_record(ms, med, gemv_bytes(n, k) - k - k // 2 + k // 16, reference_published_us=pub["w4a4_us"],
                                 in_graph_protocol_us=in_graph_us(
                                     timer, lambda: hb.nvfp4_gemv_fp4in(codes, xq.reshape(-1), scales, xs, alpha4)))
        out[f"{n}x{k}"] = rec
        del codes, scales
    out["note"] = ("reference_published_us: the reference's own Triton kernels on a B200 as its heuristics file records "
                   "them (tritonbench CUDA-graph timer: the comparable figure here is in_graph_protocol_us); they are not "
                   "re-timed on this box (the reference cannot be installed offline: its build backend is absent)")
    return out


def sub_gemv_decode_sweep(args, dev, timer) -> dict:
    """Config 4: the four NVFP4 matrices of a 70B-class layer for 1..32 activation rows (seed 4)."""
    import helion_b200 as hb
    from oracle import oracle as O

    mats = {}
    for i, (name, (n, k)) in enumerate(LAYER_70B.items()):
        c, sc, g = random_nvfp4(n, k, dev, 4000 + 16 * i, 0.02)
        mats[name] = (c, sc, g, n, k)
    gen = torch.Generator().manual_seed(4)
    host_x = {nm: torch.randn(32, k, generator=gen).to(torch.bfloat16) for nm, (_, k) in LAYER_70B.items()}
    dev_x = {nm: t.to(dev) for nm, t in host_x.items()}
    out = {}
    c, sc, g, n, k = mats["o"]
    oc, osc = c[:256].cpu(), sc.reshape(-1)[: 256 * (k // 16)].cpu()
    for batch in (1, 2, 4, 8, 16, 32):
        def one(name, batch=batch):
            c, sc, g, n, k = mats[name]
            x = dev_x[name][:batch]
            if batch == 1:
                return hb.nvfp4_gemv_bf16in(c, x.reshape(-1), sc, g).reshape(1, -1)
            return hb.nvfp4_gemv_bf16in_batched(c, x, sc, g)

        y = one("o")[:, :256]
        ref = O.nvfp4_gemm_bf16in(oc, host_x["o"][:batch], osc, g)
        ms, med = timer.run2(graphed(lambda: [one(nm) for nm in mats])[0], max(20, args.steps), 3)
        nbytes = sum(gemv_bytes(n, k, batch) for n, k in LAYER_70B.values())
        rec = hbm_record(ms, med, nbytes, parity_max_rel_err=rel_err(y, ref))
        if batch in (1, 8):
            per = {}
            for name, (n, k) in LAYER_70B.items():
                t, tm = timer.run2(graphed(lambda name=name: one(name))[0], 20, 3)
                per[name] = {"us": t * 1e3, "median_us": tm * 1e3, "GBps": gemv_bytes(n, k, batch) / (t * 1e-3) / 1e9}
            rec["per_matrix"] = per
        out[f"M={batch}"] = rec
    return out


def sub_quant(args, dev, timer) -> dict:
    """Config 2 (seed 2): 16384 tokens through the three producers the target names and their siblings."""
    import helion_b200 as hb
    from oracle import checks as C
    from oracle import oracle as O

    t, h, i = 16384, 7168, 18432
    fp8 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(2)
    x_cpu = torch.randn(t, h, generator=g).to(torch.bfloat16)
    w_cpu = (torch.rand(h, generator=g) + 0.5).to(torch.bfloat16)
    x, w = x_cpu.to(dev), w_cpu.to(dev)
    q = torch.empty(t, h, dtype=fp8, device=dev)
    s = torch.empty(t, 1, dtype=torch.float32, device=dev)
    steps = max(20, args.steps)
    out = {}
    hb.rms_norm_dynamic_per_token_quant(q, x, w, s, 1e-6)
    rep = C.rms_quant_report(x_cpu[:512], w_cpu, 1e-6, q[:512], s[:512])
    ms, med = timer.run2(graphed(lambda: hb.rms_norm_dynamic_per_token_quant(q, x, w, s, 1e-6))[0], steps, 3)
    out["rms_norm_dynamic_per_token_quant_16384x7168"] = hbm_record(
        ms, med, 2 * t * h + 2 * h + t * h + 4 * t, parity={"rows_checked": 512, **rep})
    sg = torch.empty(t, h // 128, dtype=torch.float32, device=dev)
    hb.per_token_group_fp8_quant(x, q, sg, 128, 1e-10, -448.0, 448.0, False)
    qo, so = O.per_token_group_fp8_quant(x_cpu[:512], 128, 1e-10, -448.0, 448.0, False)
    mism = int((q[:512].cpu().view(torch.uint8) != qo.view(torch.uint8)).sum()) + int((sg[:512].cpu() != so).sum())
    ms, med = timer.run2(graphed(lambda: hb.per_token_group_fp8_quant(x, q, sg, 128, 1e-10, -448.0, 448.0, False))[0], steps, 3)
    out["per_token_group_fp8_quant_16384x7168"] = hbm_record(
        ms, med, 2 * t * h + t * h + 4 * t * (h // 128), parity={"rows_checked": 512, "codes_and_scales_differing": mism})
    ms, med = timer.run2(graphed(lambda: hb.rms_norm_per_block_quant(q, x, w, sg, 1e-6, None, None, 128, False))[0], steps, 3)
    out["rms_norm_per_block_quant_16384x7168"] = hbm_record(ms, med, 2 * t * h + 2 * h + t * h + 4 * t * (h // 128))
    ms, med = timer.run2(graphed(lambda: hb.dynamic_per_token_scaled_fp8_quant(q, x, s))[0], steps, 3)
    out["dynamic_per_token_scaled_fp8_quant_16384x7168"] = hbm_record(ms, med, 2 * t * h + t * h + 4 * t)
    del x, q, sg
    xs = torch.randn(t, 2 * i, device=dev, dtype=torch.bfloat16, generator=torch.Generator(device=dev).manual_seed(2))
    qs = torch.empty(t, i, dtype=fp8, device=dev)
    ss = torch.empty(t, i // 128, dtype=torch.float32, device=dev)
    hb.silu_and_mul_per_block_quant(qs, xs, ss, 128)
    qd, sd = O.silu_and_mul_per_block_quant(xs[:512], 128)  # the reference function evaluated by torch on this device
    mism = int((qs[:512].view(torch.uint8) != qd.view(torch.uint8)).sum()) + int((ss[:512] != sd).sum())
    ms, med = timer.run2(graphed(lambda: hb.silu_and_mul_per_block_quant(qs, xs, ss, 128))[0], steps, 3)
    out["silu_and_mul_per_block_quant_16384x18432"] = hbm_record(
        ms, med, 2 * t * 2 * i + t * i + 4 * t * (i // 128),
        parity={"rows_checked": 512, "codes_and_scales_differing_from_torch_on_this_device": mism})
    one = torch.tensor([0.5], device=dev)
    ms, med = timer.run2(graphed(lambda: hb.silu_mul_fp8(xs, one))[0], steps, 3)
    out["silu_mul_fp8_16384x18432"] = hbm_record(ms, med, 2 * t * 2 * i + t * i)
    return out


def seeded_expert_bundle(experts: int, n: int, k: int, seed: int, dev, chunk: int = 16):
    """``[E, N, K]`` ~ N(0, 0.02), drawn on the device in chunks, NVFP4 with one global scale per expert."""
    from helion_b200 import moe as M

    g = torch.Generator(device=dev).manual_seed(seed)
    parts = []
    for e0 in range(0, experts, chunk):
        parts.append(M.quantize_expert_weights(torch.randn(min(chunk, experts - e0), n, k, device=dev, generator=g) * 0.02))
    return M.GroupedNvfp4Weight(torch.cat([p.packed for p in parts]),
                                torch.cat([p.scales.view(torch.uint8) for p in parts]).view(torch.float8_e4m3fn),
                                torch.cat([p.global_scale for p in parts]))


def sub_moe(args, dev, timer) -> dict:
    """Config 3 (seed 3) on one GPU, with the sampled comparison against the oracle."""
    from helion_b200 import moe as M
    from oracle import checks as C

    c = MOE_CFG
    g = torch.Generator().manual_seed(3)
    x = torch.randn(c["tokens"], c["hidden"], generator=g).to(torch.bfloat16).to(dev)
    logits = torch.randn(c["tokens"], c["experts"], generator=g).to(dev)
    w_gu = seeded_expert_bundle(c["experts"], 2 * c["inter"], c["hidden"], 3000, dev)
    w_d = seeded_expert_bundle(c["experts"], c["hidden"], c["inter"], 3500, dev)
    w_gu_i = M.interleave_gate_up(w_gu)
    got = {}
    y = M.nvfp4_moe(x, logits, c["top_k"], w_gu_i, w_d, intermediates=got)
    sample = torch.randperm(c["tokens"], generator=g)[:6]
    rep = C.moe_sample_report(x, logits, c["top_k"], w_gu, w_d, y, got, sample)
    del got
    ms, med = timer.run2(graphed(lambda: M.nvfp4_moe(x, logits, c["top_k"], w_gu_i, w_d))[0], max(10, args.steps // 2), 3)
    return tensor_record(ms, med, moe_flops(), parity=rep,
                         weight_bytes=int(w_gu.packed.numel() + w_gu.scales.numel() + w_d.packed.numel() + w_d.scales.numel()))


def sub_scaled_mm(args, dev, timer) -> dict:
    import math

    import helion_b200 as hb

    m = 16
    g = torch.Generator(device=dev).manual_seed(7)
    cases = []
    for k, n in SCALED_MM_KN:
        sc = 1.0 / math.sqrt(k)
        a = (sc * (0.5 + torch.rand(m, k, device=dev, generator=g))).to(torch.float8_e4m3fn)
        b = (sc * (0.5 + torch.rand(n, k, device=dev, generator=g))).to(torch.float8_e4m3fn).t()
        cc = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        sa = torch.rand(1, 1, device=dev, generator=g) + 0.5
        sb = torch.rand(1, 1, device=dev, generator=g) + 0.5
        bias = (0.5 * (torch.rand(n, device=dev, generator=g) - 0.5)).to(torch.bfloat16)
        cases.append((a, b, cc, sa, sb, bias))
    nbytes = sum(scaled_mm_bytes(m, k, n) for k, n in SCALED_MM_KN)

    def ours():
        for a, b, cc, sa, sb, bias in cases:
            hb.scaled_mm(cc, a, b, sa, sb, bias)

    def library():
        for a, b, cc, sa, sb, bias in cases:
            torch._scaled_mm(a, b, scale_a=sa, scale_b=sb, bias=bias, out_dtype=torch.bfloat16)

    steps = max(20, args.steps)
    ms, med = timer.run2(graphed(ours)[0], steps, 3)
    lms, lmed = timer.run2(graphed(library)[0], steps, 3)
    rec = hbm_record(ms, med, nbytes, tokens=m, shapes=len(SCALED_MM_KN), library_us=lms * 1e3, library_median_us=lmed * 1e3)
    del cases
    # prefill shapes (tensor-bound): the CTA-pair kernel, FP8 and int8, the library's FP8 kernel beside them
    peaks = measured_peaks()
    rec["prefill"] = {}
    for pm, pk, pn in SCALED_MM_PREFILL:
        sc = 1.0 / math.sqrt(pk)
        a = (sc * torch.randn(pm, pk, device=dev, generator=g)).to(torch.float8_e4m3fn)
        b = (sc * torch.randn(pn, pk, device=dev, generator=g)).to(torch.float8_e4m3fn).t()
        ai = torch.randint(-128, 128, (pm, pk), dtype=torch.int8, device=dev, generator=g)
        bi = torch.randint(-128, 128, (pn, pk), dtype=torch.int8, device=dev, generator=g).t()
        sa = torch.rand(pm, 1, device=dev, generator=g) + 0.5
        sb = torch.rand(1, pn, device=dev, generator=g) + 0.5
        cc = torch.empty(pm, pn, dtype=torch.bfloat16, device=dev)
        t8, m8 = timer.run2(graphed(lambda: hb.scaled_mm(cc, a, b, sa, sb.reshape(-1)))[0], 10, 3)
        ti, mi = timer.run2(graphed(lambda: hb.scaled_mm(cc, ai, bi, sa, sb.reshape(-1)))[0], 10, 3)
        tl, ml = timer.run2(graphed(lambda: torch._scaled_mm(a, b, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16))[0], 10, 3)
        flops = 2.0 * pm * pn * pk
        rec["prefill"][f"{pm}x{pk}x{pn}"] = {
            "fp8_us": t8 * 1e3, "fp8_median_us": m8 * 1e3, "int8_us": ti * 1e3, "library_fp8_us": tl * 1e3,
            "fp8_TFLOPs": flops / (t8 * 1e-3) / 1e12,
            "frac_of_2x_measured_bf16": flops / (t8 * 1e-3) / 1e12 / (2 * peaks["bf16_tflops"])}
        del a, b, ai, bi, cc
    return rec


# (M, K, N): prefill-sized calls of the same operator (the reference tunes it on 16 and 64 tokens only)
SCALED_MM_PREFILL = [(1024, 4096, 4096), (4096, 4096, 4096), (8192, 4096, 6144), (8192, 8192, 8192)]

# (groups, expected rows per group, N, K) of the reference's bf16 grouped-GEMM manifest
# (benchmarks/cute/deepgemm_selected_path.py:62-71); the real group sizes are expected * U(0.7, 1.3) from
# random.Random(0), aligned to 128 rows, as official_actual_ms / make_case (:104-113, 209-238) draw them
GROUPED_F16_SHAPES = [(4, 8192, 6144, 7168), (4, 8192, 7168, 3072), (4, 8192, 4096, 4096), (4, 8192, 4096, 2048),
                      (8, 4096, 6144, 7168), (8, 4096, 7168, 3072), (8, 4096, 4096, 4096), (8, 4096, 4096, 2048)]
# (M, N, K) per group of the direct-mode cases (benchmarks/cute/compare_grouped_gemm_backends.py:102-116)
GROUPED_DIRECT_CASES = {"default_small_parity": ((128, 128, 128), (512, 128, 128), (128, 256, 128)),
                        "doc_original": ((8192, 1280, 32), (16, 384, 1536), (640, 1280, 16), (640, 160, 16)),
                        "doc_no_mn_tail": ((8192, 1280, 32), (128, 384, 1536), (640, 1280, 16), (640, 128, 16))}


def sub_grouped_f16(args, dev, timer) -> dict:
    """The bf16 / fp16 grouped GEMM on the reference's manifests: the worklist form on its eight large shapes and
    the direct (heterogeneous) form on three of its small cases; cuBLAS, one matmul per group, under the same
    protocol beside each."""
    import random

    import helion_b200 as hb

    peaks = measured_peaks()
    rng = random.Random(0)
    out = {"worklist": {}, "direct": {}}
    gen = torch.Generator(device=dev).manual_seed(8)
    for groups, expect, n, k in GROUPED_F16_SHAPES:
        actual = [int(expect * rng.uniform(0.7, 1.3)) for _ in range(groups)]
        aligned = [(m + 127) // 128 * 128 for m in actual]
        total = sum(aligned)
        a = torch.randn(total, k, device=dev, dtype=torch.bfloat16, generator=gen)
        b = torch.randn(groups, n, k, device=dev, dtype=torch.bfloat16, generator=gen)
        rows, start = [], 0
        for grp, (m, am) in enumerate(zip(actual, aligned)):
            a[start + m : start + am] = 0
            rows.append((grp, start, m, am))
            start += am
        wl = torch.tensor(rows, dtype=torch.int32, device=dev)
        y = hb.grouped_gemm_deepgemm(a, b, wl)
        grp, s0, m, _ = rows[-1]
        parity = rel_err(y[s0 : s0 + 256], (a[s0 : s0 + 256].float() @ b[grp].float().t()))

        def library():
            return [a[s0_ : s0_ + am_] @ b[g_].t() for g_, s0_, _, am_ in rows]

        ms, med = timer.run2(graphed(lambda: hb.grouped_gemm_deepgemm(a, b, wl))[0], 5, 3)
        lms, _ = timer.run2(graphed(library)[0], 5, 3)
        flops = 2 * sum(actual) * n * k
        tf = flops / (ms * 1e-3) / 1e12
        out["worklist"][f"{groups}x{expect}x{n}x{k}"] = {
            "us": ms * 1e3, "median_us": med * 1e3, "TFLOPs": tf, "frac_of_measured_bf16": tf / peaks["bf16_tflops"],
            "library_us": lms * 1e3, "parity_max_rel_err": parity}
        del a, b, y
    # the dense CTA-pair kernel (the one-GPU form of the fused matmul + collective kernels) beside cuBLAS
    out["dense_pair"] = {}
    from helion_b200 import dist as D

    for dm, dn, dk in ((4096, 6656, 16384), (8192, 8192, 8192)):
        a = torch.randn(dm, dk, device=dev, dtype=torch.bfloat16, generator=gen)
        b = (torch.randn(dn, dk, device=dev, dtype=torch.float32, generator=gen) / dk**0.5).to(torch.bfloat16).t()
        cc = torch.empty(dm, dn, dtype=torch.bfloat16, device=dev)
        parity = rel_err(D.dense_matmul(a, b)[:256], a[:256].float() @ b.float())
        ms, med = timer.run2(graphed(lambda: D.dense_matmul(a, b, out=cc))[0], 10, 3)
        lms, _ = timer.run2(graphed(lambda: torch.matmul(a, b, out=cc))[0], 10, 3)
        tf = 2.0 * dm * dn * dk / (ms * 1e-3) / 1e12
        out["dense_pair"][f"{dm}x{dn}x{dk}"] = {"us": ms * 1e3, "median_us": med * 1e3, "TFLOPs": tf,
                                                "frac_of_measured_bf16": tf / peaks["bf16_tflops"],
                                                "library_us": lms * 1e3, "parity_max_rel_err": parity}
        del a, b, cc
    for name, problems in GROUPED_DIRECT_CASES.items():
        ga = [torch.randn(m, k, device=dev, dtype=torch.float16, generator=gen) for m, _, k in problems]
        gb = [torch.randn(nn, k, device=dev, dtype=torch.float16, generator=gen) for _, nn, k in problems]
        go = [torch.empty(m, nn, device=dev, dtype=torch.float16) for m, nn, _ in problems]
        hb.grouped_gemm_direct(ga, gb, go)
        parity = max(rel_err(o, a_.float() @ b_.float().t()) for a_, b_, o in zip(ga, gb, go))
        ms, med = timer.run2(graphed(lambda: hb.grouped_gemm_direct(ga, gb, go))[0], 20, 3)
        lms, _ = timer.run2(graphed(lambda: [torch.matmul(a_, b_.t(), out=o) for a_, b_, o in zip(ga, gb, go)])[0], 20, 3)
        out["direct"][name] = {"us": ms * 1e3, "median_us": med * 1e3, "library_us": lms * 1e3, "parity_max_rel_err": parity,
                               "TFLOPs": 2 * sum(m * nn * k for m, nn, k in problems) / (ms * 1e-3) / 1e12}
    return out


def sub_tp_decode_layer(args, dev, rank, world, timer) -> dict:
    """Config 4 column-parallel over the ranks (fused peer-store gather), 1 and 8 rows."""
    import helion_b200 as hb
    from helion_b200 import dist as D

    tp = D.TensorParallel(dev)
    mats = {}
    for i, (name, (n, k)) in enumerate(LAYER_70B.items()):
        c, sc, g = random_nvfp4(n // world, k, dev, 4000 + 16 * i + rank, 0.02)
        mats[name] = (c, sc, g, n, k)
    gen = torch.Generator().manual_seed(4)
    dev_x = {nm: torch.randn(8, k, generator=gen).to(torch.bfloat16).to(dev) for nm, (_, k) in LAYER_70B.items()}
    out = {}
    for batch in (1, 8):
        rings = {nm: tp.gathered_output(batch, n, torch.bfloat16) for nm, (n, _) in LAYER_70B.items()}

        def layer(batch=batch, rings=rings):
            return {nm: tp.gemv(mats[nm][0], mats[nm][1], dev_x[nm][:batch], rings[nm], mats[nm][2]) for nm in mats}

        fused = layer()
        same = True
        for nm in mats:
            c, sc, g, n, k = mats[nm]
            x = dev_x[nm][:batch]
            path = "simt" if batch == 1 else "auto"  # the kernel family tp.gemv runs a single row on
            local = hb.nvfp4_gemv_bf16in(c, x.reshape(-1), sc, g, path=path).reshape(1, -1) if batch == 1 else \
                hb.nvfp4_gemv_bf16in_batched(c, x, sc, g)
            same &= bool(torch.equal(fused[nm], D.all_gather_columns(local)))
        ms, med = timer.run2(graphed_ring(layer), max(20, args.steps), 3)
        nbytes = sum(gemv_bytes(n, k, batch) for n, k in LAYER_70B.values())
        out[f"M={batch}"] = hbm_record(ms, med, nbytes, fused_equals_collective=same)
    return out


def sub_ep_moe(args, dev, rank, world, timer) -> dict:
    """Config 3 expert-parallel: rank r owns experts [r E / g, (r + 1) E / g) and T / g of the tokens; the result is
    compared, on rank 0, with the one-GPU layer on all tokens and all experts."""
    import torch.distributed as dist

    from helion_b200 import dist as D
    from helion_b200 import moe as M

    c = MOE_CFG
    e_local, t_local = c["experts"] // world, c["tokens"] // world

    def shards(r):
        return (seeded_expert_bundle(e_local, 2 * c["inter"], c["hidden"], 3000 + r, dev),
                seeded_expert_bundle(e_local, c["hidden"], c["inter"], 3500 + r, dev))

    w_gu, w_d = shards(rank)
    w_gu_i = M.interleave_gate_up(w_gu)
    g = torch.Generator().manual_seed(3 + 97 * rank)
    x = torch.randn(t_local, c["hidden"], generator=g).to(torch.bfloat16).to(dev)
    logits = torch.randn(t_local, c["experts"], generator=g).to(dev)
    ep = D.ExpertParallel(dev, t_local, c["hidden"], c["top_k"], c["experts"])

    def step():
        return ep.moe(x, logits, w_gu_i, w_d)

    y = step()
    ys = [torch.empty_like(y) for _ in range(world)]
    xs = [torch.empty_like(x) for _ in range(world)]
    ls = [torch.empty_like(logits) for _ in range(world)]
    dist.all_gather(ys, y)
    dist.all_gather(xs, x)
    dist.all_gather(ls, logits)
    parity = None
    if rank == 0:
        parts = [shards(r) if r else (w_gu, w_d) for r in range(world)]

        def cat(bundles):
            return M.GroupedNvfp4Weight(torch.cat([b.packed for b in bundles]),
                                        torch.cat([b.scales.view(torch.uint8) for b in bundles]).view(torch.float8_e4m3fn),
                                        torch.cat([b.global_scale for b in bundles]))

        full_gu, full_d = cat([p[0] for p in parts]), cat([p[1] for p in parts])
        del parts
        single = M.nvfp4_moe(torch.cat(xs), torch.cat(ls), c["top_k"], M.interleave_gate_up(full_gu), full_d)
        got = torch.cat(ys)
        parity = {"max_rel_err_vs_one_gpu": rel_err(got, single), "bit_identical_to_one_gpu": bool(torch.equal(got, single))}
        del full_gu, full_d, single
    # the step is a fixed sequence of launches (two barrier kernels included): replayed from a CUDA graph
    ms, med = timer.run2(graphed(step)[0], max(10, args.steps // 2), 3)
    return tensor_record(ms, med, moe_flops(), parity=parity, phases_us=ep.phase_times(x, logits, w_gu_i, w_d))


def sub_fused_matmul(args, dev, rank, world, timer) -> dict:
    """The reference's distributed examples at the all-gather example's shape (M = 4096, N = 6656, K = 16384, bf16:
    examples/distributed/all_gather_matmul.py:258): all-gather + matmul and matmul + reduce-scatter as single
    kernels over peer memory, beside the process group's collective plus the same GEMM kernel.  Eager launches
    (the all-gather form takes a call number per launch)."""
    import torch.distributed as dist

    from helion_b200 import dist as D

    m, n, k = 4096, 6656, 16384
    peaks = measured_peaks()
    fm = D.FusedMatmulCollectives(dev)
    g = torch.Generator(device=dev).manual_seed(40 + rank)
    out = {}
    # all-gather + matmul: every rank holds M / world rows of a, and all of b
    rows = m // world
    splits = 1  # more chunks per rank cost more system-scope fences than they gain in overlap (measured)
    shard = torch.randn(rows, k, device=dev, dtype=torch.bfloat16, generator=g)
    gb = torch.Generator(device=dev).manual_seed(39)
    b = (torch.randn(n, k, device=dev, dtype=torch.float32, generator=gb) / k**0.5).to(torch.bfloat16).t()
    full = torch.empty(m, k, dtype=torch.bfloat16, device=dev)

    def unfused_ag():
        dist.all_gather_into_tensor(full, shard)
        return D.dense_matmul(full, b)

    _, c = fm.all_gather_matmul(shard, b, splits_per_rank=splits)
    same = bool(torch.equal(c, unfused_ag()))
    ms, med = timer.run2(lambda: fm.all_gather_matmul(shard, b, splits_per_rank=splits), 10, 3)
    ums, umed = timer.run2(unfused_ag, 10, 3)
    gms, _ = timer.run2(lambda: D.dense_matmul(full, b), 10, 3)
    flops = 2.0 * m * n * k
    out["all_gather_matmul"] = {
        "us": ms * 1e3, "median_us": med * 1e3, "collective_then_matmul_us": ums * 1e3, "matmul_alone_us": gms * 1e3,
        "TFLOPs": flops / (ms * 1e-3) / 1e12, "frac_of_measured_bf16": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "fused_equals_collective": same, "splits_per_rank": splits,
        "nvlink_bytes_in_per_rank": (world - 1) * rows * k * 2}
    del full, c, shard
    # matmul + reduce-scatter: every rank holds a K shard of a and of b
    k_local = k // world
    a = torch.randn(m, k_local, device=dev, dtype=torch.bfloat16, generator=g)
    bl = (torch.randn(n, k_local, device=dev, dtype=torch.float32, generator=g) / k**0.5).to(torch.bfloat16).t()
    recv = torch.empty(m // world, n, dtype=torch.bfloat16, device=dev)

    def unfused_rs():
        dist.reduce_scatter_tensor(recv, D.dense_matmul(a, bl))
        return recv

    got = fm.matmul_reduce_scatter(a, bl)
    parts = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    dist.all_gather(parts, D.dense_matmul(a, bl))
    want = sum(p.float() for p in parts)[rank * (m // world) : (rank + 1) * (m // world)].to(torch.bfloat16)
    same = bool(torch.equal(got, want))
    del parts, want
    ms, med = timer.run2(lambda: fm.matmul_reduce_scatter(a, bl), 10, 3)
    ums, umed = timer.run2(unfused_rs, 10, 3)
    gms, _ = timer.run2(lambda: D.dense_matmul(a, bl), 10, 3)
    flops = 2.0 * m * n * k_local
    out["matmul_reduce_scatter"] = {
        "us": ms * 1e3, "median_us": med * 1e3, "matmul_then_collective_us": ums * 1e3, "matmul_alone_us": gms * 1e3,
        "TFLOPs": flops / (ms * 1e-3) / 1e12, "frac_of_measured_bf16": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "equals_ordered_sum_of_partials": same, "nvlink_bytes_out_per_rank": (world - 1) * (m // world) * n * 2}
    return out


def guarded(fn, *a) -> dict:
    """A failing side workload must not cost the run its headline: record the error instead."""
    try:
        return fn(*a)
    except Exception as exc:  # noqa: BLE001
        import traceback

        return {"error": f"{type(exc).__name__}: {exc}"[:400], "where": traceback.format_exc().strip().splitlines()[-3:]}


def wl_all(args, dev, rank, world, timer):
    """Headline: the dense GEMM.  Every other configuration rides along in ``workloads``."""
    r = wl_gemm(args, dev, rank, world, timer)
    subs = {}
    torch.cuda.empty_cache()
    if world == 1:
        for name, fn in (("gemv_config0_8192x4096", sub_gemv_config0), ("gemv_decode_sweep_70b_layer", sub_gemv_decode_sweep),
                         ("gemv_reference_published_shapes", sub_gemv_published_shapes), ("quant_producers_16384_tokens", sub_quant),
                         ("moe_8192_tokens_128_experts_top8", sub_moe), ("scaled_mm_decode_shapes", sub_scaled_mm),
                         ("grouped_gemm_bf16_manifests", sub_grouped_f16)):
            subs[name] = guarded(fn, args, dev, timer)
            torch.cuda.empty_cache()
        for name, cpu in (("gemv_decode_sweep_70b_layer", "gemv"), ("quant_producers_16384_tokens", "quant"),
                          ("moe_8192_tokens_128_experts_top8", "moe")):
            if "error" not in subs[name]:
                subs[name]["cpu_port"] = cpu_port(cpu)
    else:
        subs["gemv_decode_layer_column_parallel"] = guarded(sub_tp_decode_layer, args, dev, rank, world, timer)
        torch.cuda.empty_cache()
        subs["moe_expert_parallel"] = guarded(sub_ep_moe, args, dev, rank, world, timer)
        torch.cuda.empty_cache()
        subs["fused_matmul_collectives_bf16"] = guarded(sub_fused_matmul, args, dev, rank, world, timer)
    r["extra"]["workloads"] = subs
    return r


WORKLOADS = {"all": wl_all, "gemm": wl_gemm, "gemv": wl_gemv, "quant": wl_quant, "moe": wl_moe, "scaled_mm": wl_scaled_mm}


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
    ap.add_argument("--workload", default="all", choices=sorted(WORKLOADS))
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
