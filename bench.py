"""Benchmark driver: ``python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]``.

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of synthetic input:

* ``gemv_decode_layer`` : the four NVFP4 weight matrices of a 70B-class dense layer (QKV 10240x8192,
  O 8192x8192, gate|up 57344x8192, down 8192x28672) applied to one bf16 activation row each (M=1);
  481 MB of weights per step, so every step streams far more than the 126 MB L2 (no flush needed).
  metric = HBM bytes the step must move / time (TB/s).  With N GPUs the rows of every matrix are split
  evenly (column tensor parallelism) and the bf16 outputs are all-gathered over NCCL.

Timing: CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks.
``--impl reference`` times the reference's CPU path (the oracle port of its PyTorch reference functions)
on the host cores, on a bounded sample of the same workload.
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


def gemv_bytes(n: int, k: int, m: int = 1) -> int:
    """Algorithmic HBM bytes of one NVFP4 GEMV: packed codes + block scales + activations + outputs."""
    return n * k // 2 + n * k // 16 + 2 * m * k + 2 * m * n


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x8: "hw_slowdown",
        0x40: "hw_thermal_slowdown",
        0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

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
            self._stop.wait(0.05)

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
        return {
            "sm_mhz": s[len(s) // 2] if s else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(s),
        }


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, dense bf16 TFLOP/s, provenance)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def ncu_traffic(kernel_key: str):
    """DRAM bytes per launch recorded from an ncu capture (profiles/traffic.json), or None."""
    p = ROOT / "profiles" / "traffic.json"
    if p.exists():
        return json.loads(p.read_text()).get(kernel_key)
    return None


# ------------------------------------------------------------- reference arm
def cpu_sample_gemv(seconds_budget: float = 8.0):
    """Times the oracle port of reference_nvfp4_gemv_bf16in on a bounded slice of the O-projection
    (rows x 8192) with all host threads; returns (TB/s, cores, sample description, seconds per call)."""
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    k = 8192
    rows = 1024
    g = torch.Generator().manual_seed(4)
    w = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, generator=g)
    x = torch.randn(k, generator=g).to(torch.bfloat16)
    s = O.swizzle_scales((torch.rand(rows, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
    O.nvfp4_gemv_bf16in(w, x, s, 1.0)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while True:
        O.nvfp4_gemv_bf16in(w, x, s, 1.0)
        reps += 1
        if time.perf_counter() - t0 > seconds_budget or reps >= 50:
            break
    dt = (time.perf_counter() - t0) / reps
    tbs = gemv_bytes(rows, k) / dt / 1e12
    return tbs, torch.get_num_threads(), f"{rows}x{k} slice of the O projection, {reps} calls", dt


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    k, rows = 8192, 1024
    g = torch.Generator().manual_seed(4)
    w = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, generator=g)
    x = torch.randn(k, generator=g).to(torch.bfloat16)
    s = O.swizzle_scales((torch.rand(rows, k // 16, generator=g) + 0.5).to(torch.float8_e4m3fn))
    for _ in range(args.warmup):
        O.nvfp4_gemv_bf16in(w, x, s, 1.0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.nvfp4_gemv_bf16in(w, x, s, 1.0)
    dt = (time.perf_counter() - t0) / args.steps
    value = gemv_bytes(rows, k) / dt / 1e12
    sample = f"each step = reference_nvfp4_gemv_bf16in semantics on a {rows}x{k} slice of the O projection"
    line = {
        "impl": "reference",
        "metric": "nvfp4_gemv_hbm_throughput",
        "value": value,
        "unit": "TB/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": dt * 1e3,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "fp32",
        "data": "synthetic",
        "config": {"workload": "gemv_decode_layer", "batch": 1, "layer": "70B-class dense (cfg 4)", "sampled": True},
        "cpu_baseline": {"value": value, "unit": "TB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ GPU arm
def build_layer(dev, rank: int, world: int):
    """Synthetic 70B-class layer: W ~ N(0, 0.02) quantised to NVFP4 by the CUDA quantiser; each rank keeps
    rows [rank*N/world, (rank+1)*N/world) of every matrix (N/world is a multiple of 128 for world <= 8)."""
    import helion_b200 as hb

    mats = {}
    for i, (name, (n, k)) in enumerate(LAYER_70B.items()):
        n_local = n // world
        gen = torch.Generator(device=dev).manual_seed(4 * 1000 + i * 16 + rank)
        codes = torch.empty(n_local, k // 2, dtype=torch.uint8, device=dev)
        scale_chunks = []
        # global scale from the distribution's expected amax keeps ranks consistent: ~4.9 sigma over 5e8 draws
        g = torch.tensor(0.02 * 6.0 / (6.0 * 448.0), device=dev, dtype=torch.float32)
        chunk = 2048
        for r0 in range(0, n_local, chunk):
            w = (torch.randn(min(chunk, n_local - r0), k, generator=gen, device=dev) * 0.02).to(torch.bfloat16)
            c, s, _ = hb.nvfp4_quantize(w, g)
            codes[r0 : r0 + w.shape[0]] = c
            scale_chunks.append(s.view(torch.uint8))
        scales = torch.cat(scale_chunks).view(torch.float8_e4m3fn)  # chunks are multiples of 128 rows
        mats[name] = (codes, scales, float(g), n, k)
    return mats


def run_gpu(args) -> None:
    import helion_b200 as hb
    from helion_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    batch = args.batch
    mats = build_layer(dev, rank, world)
    gen = torch.Generator().manual_seed(4)
    host_x = {name: torch.randn(batch, k, generator=gen).to(torch.bfloat16).pin_memory() for name, (_, k) in LAYER_70B.items()}
    dev_x = {name: t.to(dev) for name, t in host_x.items()}
    stream = torch.cuda.current_stream()

    def layer_step(xs):
        outs = {}
        for name, (codes, scales, g, n, k) in mats.items():
            if batch == 1:
                y = hb.nvfp4_gemv_bf16in(codes, xs[name].reshape(-1), scales, g).reshape(1, -1)
            else:
                y = hb.nvfp4_gemv_bf16in_batched(codes, xs[name], scales, g)
            if world > 1:
                full = torch.empty(world, batch, n // world, dtype=torch.bfloat16, device=dev)
                dist.all_gather_into_tensor(full, y)
                y = full
            outs[name] = y
        return outs

    # parity spot check against the oracle on a slice of the O projection (outside the timed region)
    from oracle import oracle as O

    codes, scales, g, n, k = mats["o"]
    y = hb.nvfp4_gemv_bf16in(codes[:256], dev_x["o"][0].contiguous(), scales[: 256 * (k // 16)], g)
    ref = O.nvfp4_gemv_bf16in(codes[:256].cpu(), host_x["o"][0], scales[: 256 * (k // 16)].cpu(), g)
    err = ((y.float().cpu() - ref.float()).abs() / torch.maximum(ref.float().abs(), ref.float().pow(2).mean().sqrt())).max()
    parity = {"max_rel_err": float(err), "ok": bool(err <= 1e-2)}

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        layer_step(dev_x)
    sync()

    # ---- device-resident timing (value) + per-matrix launch timing (roofline) ----
    names = list(LAYER_70B)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(args.steps)]
    with ClockSampler(local) as clocks:
        sync()
        t_start = torch.cuda.Event(enable_timing=True)
        t_end = torch.cuda.Event(enable_timing=True)
        t_start.record(stream)
        for s in range(args.steps):
            if world == 1:
                for i, name in enumerate(names):
                    codes, scales, g, n, k = mats[name]
                    ev[s][i].record(stream)
                    if batch == 1:
                        hb.nvfp4_gemv_bf16in(codes, dev_x[name].reshape(-1), scales, g)
                    else:
                        hb.nvfp4_gemv_bf16in_batched(codes, dev_x[name], scales, g)
                ev[s][len(names)].record(stream)
            else:
                layer_step(dev_x)
        t_end.record(stream)
        sync()
        dev_ms = t_start.elapsed_time(t_end)

        # ---- end to end: pinned host activations in, outputs back to the host, every step ----
        host_out = {name: torch.empty(world, batch, n // world, dtype=torch.bfloat16).pin_memory() for name, (n, _) in LAYER_70B.items()}
        for _ in range(min(3, args.warmup)):
            outs = layer_step({name: t.to(dev, non_blocking=True) for name, t in host_x.items()})
        sync()
        e_start = torch.cuda.Event(enable_timing=True)
        e_end = torch.cuda.Event(enable_timing=True)
        e_start.record(stream)
        for _ in range(args.steps):
            xs = {name: t.to(dev, non_blocking=True) for name, t in host_x.items()}
            outs = layer_step(xs)
            for name, y in outs.items():
                host_out[name].view(-1)[: y.numel()].copy_(y.reshape(-1), non_blocking=True)
        e_end.record(stream)
        sync()
        e2e_ms = e_start.elapsed_time(e_end)

    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])

    layer_bytes = sum(gemv_bytes(n, k, batch) for n, k in LAYER_70B.values())
    ms_per_step = dev_ms / args.steps
    value = layer_bytes / (ms_per_step * 1e-3) / 1e12
    e2e_value = layer_bytes / (e2e_ms / args.steps * 1e-3) / 1e12
    h2d = sum(2 * batch * k for _, k in LAYER_70B.values())
    d2h = sum(2 * batch * n for n, _ in LAYER_70B.values())

    hbm_peak, _, peak_kind = measured_peaks()
    roofline = None
    per_matrix = {}
    if world == 1:
        for i, name in enumerate(names):
            ms = sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)) / args.steps
            n, k = LAYER_70B[name]
            per_matrix[name] = {"us": ms * 1e3, "GBps": gemv_bytes(n, k, batch) / (ms * 1e-3) / 1e9}
        dom = "gate_up"
        achieved = per_matrix[dom]["GBps"]
        roofline = {
            "bound": "hbm",
            "kernel": "nvfp4_gemv_kernel" if batch == 1 else "nvfp4_gemv_batched_kernel",
            "launch": f"{dom} {LAYER_70B[dom][0]}x{LAYER_70B[dom][1]} M={batch}",
            "achieved": achieved,
            "peak": hbm_peak,
            "peak_kind": f"{peak_kind} copy bandwidth",
            "unit": "GB/s",
            "frac": achieved / hbm_peak,
            "traffic": ncu_traffic(f"gemv_{dom}_m{batch}"),
        }

    if rank == 0:
        cpu_tbs, cores, sample, _ = cpu_sample_gemv()
        line = {
            "metric": "nvfp4_gemv_hbm_throughput",
            "value": value,
            "unit": "TB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "fp16 products, fp32 accumulate (e2m1 x e4m3 weights, bf16 in/out)",
            "data": "synthetic",
            "config": {
                "workload": "gemv_decode_layer",
                "layer": "70B-class dense: qkv 10240x8192, o 8192x8192, gate_up 57344x8192, down 8192x28672 (cfg 4)",
                "batch": batch,
                "parallelism": f"column-tp{world}" if world > 1 else "single",
                "l2": "inputs larger than L2 (481 MB of weights per step)",
                "bytes_per_step": layer_bytes,
            },
            "e2e": {"value": e2e_value, "unit": "TB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": args.steps * len(names),
            "roofline": roofline,
            "per_matrix": per_matrix,
            "cpu_baseline": {"value": cpu_tbs, "unit": "TB/s", "cores": cores, "kind": "port", "sample": sample},
            "clocks": clocks.summary(),
            "parity": parity,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemv_decode_layer", choices=["gemv_decode_layer"])
    ap.add_argument("--batch", type=int, default=1)
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
