"""Benchmark of the hot path on B200. Prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--sgemm-impl NAME] [--no-extras]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload: FP32 SIMT GEMM, M = N = K = 4096 per GPU, A column-major,
B and C row-major, N(0,1) inputs from seed 0 - the configuration the reference
publishes its numbers on. One step is one `cuda_ai_kernels.gemm` call.

  value     TFLOP/s (2*M*N*K / device time) with inputs resident in HBM, CUDA
            events around exactly K steps on the launching stream; two input
            sets are rotated so that a step never finds its operands in L2.
  e2e       the same metric through the operator API from pinned HOST buffers:
            host->device copies of the operands and the device->host read of C
            are inside the timed region of every step; upload, GEMM and download
            of neighbouring steps overlap on separate streams. With N > 1 every
            rank uploads its rows of A and 1/N of B; B is completed on every GPU
            by an all-gather over NVLink, so each byte of B crosses PCIe once.
  roofline  the dominant kernel against the FP32 FMA peak; `also` carries the
            TF32 tensor-core GEMM (tensor roofline) and the two row operators
            (HBM roofline) measured in the same run, next to cuBLAS, cuBLASLt
            with its fused epilogue and - when its build is present - the
            upstream project's own kernels rebuilt for this GPU.
  cpu_baseline  the reference's CPU-capable path - its FP64 torch matmul oracle,
            with the FP32 product beside it - timed on this host's cores.

N > 1 (one rank per GPU under torchrun): the GEMM is sharded along M - every
rank owns 4096 rows of A and a full B, C stays sharded, no data-path collective
(weak scaling). `also.c5` times the large sharded configuration (M = 32768
split over the ranks, N = K = 8192; strong scaling) on the FP32 and the TF32
path at every N, with the all-gather of C as a separate collective and fused
into the kernels' epilogues.

`--impl reference` times the reference's own CPU implementation of the path
(the FP64 oracle expression) on all host cores, one full 4096^3 product per step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
PACKAGE = REPO / "cuda-ai-infra-kernels_b200"
for _p in (str(PACKAGE / "python"), str(REPO)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

M = N = K = 4096
C5_M, C5_N, C5_K = 32768, 8192, 8192
METRIC = "fp32_simt_gemm_4096_tflops"
UNIT = "TFLOP/s"
FP32_LANES_PER_SM = 128
# The reference's published figure for this metric: split_k at 4096^3 on an
# A800 80GB PCIe, 17.206 TFLOP/s (its README.md:17). Other hardware; per GPU.
PUBLISHED_A800_SPLIT_K_TFLOPS = 17.206
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernels.
# A benchmark cannot run Nsight Compute on itself, so the figures are carried here. Each comes from
# one `ncu` capture of that kernel alone at the benchmark size (a handful of counters, two to four
# launches): the small cases used for the full counter sets keep their operands in L2 and say
# nothing about DRAM, so traffic is not scaled up from them. Beside them stand the algorithmic
# bytes: 201 MB (FP32 4096^3: A + B + C), 268 MB (TF32 4096^3 with a source: A + B + C + D),
# 537 MB (RMSNorm), 268 MB (softmax).
NCU_TRAFFIC_BYTES = {
    "sgemm_4096": 336.2e6 + 53.9e6,
    "tf32_4096": 376.7e6 + 54.4e6,
    "rmsnorm_16384x4096": 481.0e6,   # below the algorithmic bytes: the last written lines are still in L2
    "softmax_32768x1024": 212.0e6,
}


def load_peaks() -> dict:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        peaks["source"] = "measured"
        return peaks
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "sm_max_mhz": 1965.0,
            "source": "fallback"}


def host_threads() -> int:
    """Cores this process may run on (torchrun exports OMP_NUM_THREADS=1, which is not the machine)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def make_config(world: int, impl: str) -> dict:
    """`config` of the JSON line; the same object in both arms (the reference arm times the same workload)."""
    return {"workload": f"fp32_gemm_{M}x{N}x{K}_colmajorA", "impl": impl,
            "sharding": "rows of A per rank, B replicated, C sharded" if world > 1 else "single GPU",
            "rows_per_gpu": M, "global_m": M * world,
            "l2": "two input sets alternate (A+B 256 MB > 126 MB L2), no flush kernel"}


class ClockSampler:
    """Polls SM clock, power and throttle reasons through NVML while a region runs."""

    def __init__(self, device_index: int, period_s: float = 0.002):
        self.samples: list[tuple[int, float, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._handle = None
        self._period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = device_index
            if visible:
                entries = [v.strip() for v in visible.split(",") if v.strip()]
                if device_index < len(entries) and entries[device_index].isdigit():
                    physical = int(entries[device_index])
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: the record says so instead of failing the run
            self._handle = None

    def _loop(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)
                watts = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                self.samples.append((mhz, watts, reasons))
            except Exception:
                pass
            time.sleep(self._period)

    def __enter__(self):
        self.samples = []
        self._stop.clear()
        if self._handle is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def median_mhz(self):
        return statistics.median(s[0] for s in self.samples) if self.samples else None

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"], "samples": 0}
        nv = self._nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        seen = 0
        for _, _, r in self.samples:
            seen |= r
        return {
            "sm_mhz": statistics.median(s[0] for s in self.samples),
            "sm_max_mhz": self.max_mhz,
            "power_w_max": round(max(s[1] for s in self.samples), 1),
            "reasons": [name for name, bit in names.items() if seen & bit],
            "samples": len(self.samples),
        }


def event_time_ms(fn, steps: int) -> float:
    """Device time of `steps` calls of fn(i), CUDA events on the current stream."""
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for i in range(steps):
        fn(i)
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end)


def best_seconds(fn, repeats: int) -> float:
    fn()  # warm-up
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_baseline_block(a_cpu, b_cpu, repeats: int) -> dict:
    """The reference's CPU-capable path on this host: FP64 oracle product, FP32 product beside it."""
    from oracle import oracle

    cores = torch.get_num_threads()
    flop = 2.0 * M * N * K
    fp64_s = best_seconds(lambda: oracle.gemm_fp64(a_cpu, b_cpu), repeats)
    fp32_s = best_seconds(lambda: a_cpu @ b_cpu, repeats)
    return {"value": flop / fp64_s / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "fp32_value": flop / fp32_s / 1e12,
            "sample": f"full {M}x{N}x{K} product, best of {repeats} after 1 warm-up: FP64 torch matmul oracle "
                      f"(A.double() @ B.double()).float() {fp64_s:.3f} s, FP32 A @ B (column-major A) {fp32_s:.3f} s; "
                      f"{cores} threads, host has {os.cpu_count()} logical CPUs"}


def cpu_rowop_seconds() -> dict:
    """The reference's CPU oracle for the row operators at the benchmark shapes, one pass each after a warm-up."""
    from oracle import oracle

    x, w = oracle.rmsnorm_inputs(16384, 4096, seed=0)
    logits = oracle.softmax_inputs(32768, 1024, seed=0)
    out = {"threads": torch.get_num_threads()}
    out["rmsnorm_fp32_s"] = best_seconds(lambda: x * torch.rsqrt(torch.mean(x * x, dim=-1, keepdim=True) + 1e-6) * w, 1)
    out["rmsnorm_fp64_s"] = best_seconds(lambda: oracle.rmsnorm_fp64(x, w, 1e-6), 1)
    out["softmax_fp32_s"] = best_seconds(lambda: torch.softmax(logits, dim=1), 1)
    out["softmax_fp64_s"] = best_seconds(lambda: oracle.softmax_fp64(logits), 1)
    return out


def run_reference(args, rank: int, world: int) -> None:
    """The reference's CPU path (its FP64 torch oracle) on all host cores; rank 0 only."""
    if rank != 0:
        return
    from oracle import oracle

    torch.set_num_threads(host_threads())
    a_cpu, b_cpu = oracle.ladder_inputs(M, N, K, seed=0)
    for _ in range(args.warmup):
        oracle.gemm_fp64(a_cpu, b_cpu)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemm_fp64(a_cpu, b_cpu)
    elapsed = time.perf_counter() - t0
    tflops = 2.0 * M * N * K * args.steps / elapsed / 1e12
    fp32_s = best_seconds(lambda: a_cpu @ b_cpu, 3)
    cores = torch.get_num_threads()
    sample = (f"{args.steps} full {M}x{N}x{K} FP64 products, (A.double() @ B.double()).float(), column-major A; "
              f"FP32 A @ B best of 3: {fp32_s:.3f} s; {cores} threads of {os.cpu_count()} logical CPUs")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": make_config(world, args.sgemm_impl),
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "fp32_value": 2.0 * M * N * K / fp32_s / 1e12},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------ comparisons on one GPU


class Comparator:
    """Times competing implementations of one workload so that the ranking does not depend on the
    order: the arms are interleaved (a, b, c, a, b, c, ...) over `rounds` rounds, every measurement
    records the median SM clock seen while it ran, and the median over the rounds is reported with
    the clock and the clock-normalised time (ms x MHz) beside it."""

    def __init__(self, device_index: int, warmup: int, rounds: int = 3, target_ms: float = 30.0):
        self.sampler = ClockSampler(device_index)
        self.warmup, self.rounds, self.target_ms = warmup, rounds, target_ms

    def run_burst(self, arms: dict, idle_s: float = 0.6, window_ms: float = 8.0) -> dict:
        """Each arm timed ALONE after an idle gap: a short window (a few milliseconds) that starts
        at the clock an idle GPU offers, before power management settles - the regime in which the
        burst peaks of the roofline were measured. Median over the rounds, arms interleaved."""
        steps = {}
        for name, fn in arms.items():
            for i in range(self.warmup):
                fn(i)
            probe = event_time_ms(fn, 3) / 3
            steps[name] = int(min(500, max(3, math.ceil(window_ms / max(probe, 1e-4)))))
        samples = {name: [] for name in arms}
        for _ in range(self.rounds):
            for name, fn in arms.items():
                torch.cuda.synchronize()
                time.sleep(idle_s)
                fn(0), fn(1)
                with self.sampler:
                    ms = event_time_ms(fn, steps[name]) / steps[name]
                samples[name].append((ms, self.sampler.median_mhz()))
        return self._summarise(samples, steps)

    def run(self, arms: dict) -> dict:
        steps = {}
        for name, fn in arms.items():
            for i in range(self.warmup):
                fn(i)
            probe = event_time_ms(fn, 3) / 3
            steps[name] = int(min(2000, max(5, math.ceil(self.target_ms / max(probe, 1e-4)))))
        samples = {name: [] for name in arms}
        for _ in range(self.rounds):
            for name, fn in arms.items():
                fn(0)
                with self.sampler:
                    ms = event_time_ms(fn, steps[name]) / steps[name]
                samples[name].append((ms, self.sampler.median_mhz()))
        return self._summarise(samples, steps)

    def _summarise(self, samples: dict, steps: dict) -> dict:
        out = {}
        for name, vals in samples.items():
            ms = statistics.median(v[0] for v in vals)
            clocks = [v[1] for v in vals if v[1] is not None]
            mhz = statistics.median(clocks) if clocks else None
            out[name] = {"ms": ms, "min_ms": min(v[0] for v in vals), "mhz": mhz,
                         "ms_x_mhz": ms * mhz if mhz else None, "steps": steps[name], "rounds": self.rounds}
        return out


def graph_us(fn) -> dict:
    """The reference's headline method (benchmarks/bench_gemm_all.py:46-77): 10 calls captured in a
    CUDA graph, warm-up 10, 50 timed replays; microseconds per call."""
    from cuda_ai_kernels.benchmark import cuda_graph_benchmark

    t = cuda_graph_benchmark(fn, warmup=10, repeat=50, calls_per_graph=10)
    return {"median_us": 1e3 * t["p50_ms"], "mean_us": 1e3 * t["mean_ms"], "min_us": 1e3 * t["min_ms"]}


def eager_rmsnorm(x, w, eps: float = 1e-6):
    """Eager PyTorch RMSNorm on the GPU, as the reference's benchmark times it (benchmarks/bench_rmsnorm.py:27-29)."""
    return x * torch.rsqrt(torch.mean(x * x, dim=-1, keepdim=True) + eps) * w


def measure_extras(pkg, peaks: dict, device_index: int, warmup: int) -> dict:
    """TF32 GEMM, row operators and library baselines, same process, same GPU."""
    out: dict = {}
    dev = torch.device("cuda", device_index)
    cmp = Comparator(device_index, warmup)
    from cuda_ai_kernels import _C

    def put(prefix: str, result: dict, work: float, unit_scale: float, unit: str):
        """`work / time` under `<prefix>_<unit>` with clock and clock-normalised time beside it."""
        out[f"{prefix}_{unit}"] = work / result["ms"] / unit_scale
        out[f"{prefix}_ms"] = result["ms"]
        out[f"{prefix}_mhz"] = result["mhz"]
        out[f"{prefix}_ms_x_mhz"] = result["ms_x_mhz"]

    # FP32 ladder and cuBLAS strict-FP32 SGEMM through the operator API, same inputs as the headline.
    a_sets = [torch.randn(K, M, device=dev).t() for _ in range(2)]
    b_sets = [torch.randn(K, N, device=dev) for _ in range(2)]
    names = ("cublas", "prefetch_smem", "prefetch_reg", "split_k", "thread_tile_8x8", "warp_tile")
    res = cmp.run({name: (lambda i, name=name: pkg.gemm(a_sets[i & 1], b_sets[i & 1], impl=name)) for name in names})
    for name in names:
        put(f"sgemm_{name}", res[name], 2.0 * M * N * K, 1e9, "tflops")
    # The headline kernel and cuBLAS once more by the reference's own method (graph of 10 calls, 50
    # replays): median, mean and minimum per call.
    for name in ("prefetch_reg", "cublas"):
        g = graph_us(lambda name=name: pkg.gemm(a_sets[0], b_sets[0], impl=name))
        out[f"sgemm_{name}_graph_ms"] = g["median_us"] / 1e3
        out[f"sgemm_{name}_graph_mean_ms"] = g["mean_us"] / 1e3
        out[f"sgemm_{name}_graph_min_ms"] = g["min_us"] / 1e3
        out[f"sgemm_{name}_graph_tflops"] = 2.0 * M * N * K / g["median_us"] / 1e6
    del a_sets, b_sets
    # The other two FP32 benchmark shapes: 1024^3 and 1024 x 4096 x 4096, where tiles do not fill
    # whole rounds of SMs and the stream-K entry (output cleared inside the timed call) matters.
    for (m_, n_, k_) in ((1024, 1024, 1024), (1024, 4096, 4096)):
        a_small = [torch.randn(k_, m_, device=dev).t() for _ in range(2)]
        b_small = [torch.randn(k_, n_, device=dev) for _ in range(2)]
        names = ("cublas", "prefetch_smem", "prefetch_reg", "split_k")
        res = cmp.run({name: (lambda i, name=name: pkg.gemm(a_small[i & 1], b_small[i & 1], impl=name)) for name in names})
        for name in names:
            put(f"sgemm_{name}_{m_}x{n_}x{k_}", res[name], 2.0 * m_ * n_ * k_, 1e9, "tflops")
            g = graph_us(lambda name=name: pkg.gemm(a_small[0], b_small[0], impl=name))
            out[f"sgemm_{name}_{m_}x{n_}x{k_}_graph_us"] = g["median_us"]
            out[f"sgemm_{name}_{m_}x{n_}x{k_}_graph_min_us"] = g["min_us"]
        del a_small, b_small

    # TF32 tcgen05 GEMM with fused epilogue, D = relu(A@B + 0.5*C) and the linear form, against
    # cuBLAS TF32 + a separate ReLU pass (what the reference ships) and cuBLASLt with the ReLU fused
    # by the library (the fair competitor), interleaved.
    tf32_peak = peaks["bf16_tflops"] / 2.0
    for size in (1024, 4096, 8192):   # 1024 and 8192 are the benchmark configuration, 4096 the roofline size
        a = [torch.randn(size, size, device=dev) for _ in range(2)]
        b = [torch.randn(size, size, device=dev) for _ in range(2)]
        c = torch.randn(size, size, device=dev)
        arms = {
            "relu": lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1], c=c, alpha=1.0, beta=0.5, epilogue="relu"),
            "cublaslt_fused_relu": lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1], c=c, alpha=1.0, beta=0.5,
                                                               epilogue="relu", kernel="cublaslt"),
            "linear": lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1], c=c, alpha=1.0, beta=0.5, epilogue="linear"),
            "cublas_unfused_relu": lambda i: torch.relu_(pkg.adaptive_gemm(a[i & 1], b[i & 1], c=c, alpha=1.0, beta=0.5,
                                                                           kernel="cublas")),
        }
        # Two regimes, both interleaved: each arm alone after an idle gap (burst clocks; the key
        # without a suffix, comparable with the burst peak of the roofline) and back to back for
        # tens of milliseconds (`_sustained`: the clock the power cap allows under tensor load).
        res = cmp.run_burst(arms)
        for name in arms:
            put(f"tf32_{name}_{size}", res[name], 2.0 * size ** 3, 1e9, "tflops")
        res = cmp.run(arms)
        for name in arms:
            put(f"tf32_{name}_{size}_sustained", res[name], 2.0 * size ** 3, 1e9, "tflops")
        arms["relu"](0)
        out[f"tf32_relu_{size}_kernel"] = _C.adaptive_gemm_last_kernel()
        if size == 1024:
            # A 10-microsecond call: device time by the reference's method (graph replay) beside the event timings.
            for name in arms:
                g = graph_us(lambda name=name: arms[name](0))
                out[f"tf32_{name}_{size}_graph_us"], out[f"tf32_{name}_{size}_graph_min_us"] = g["median_us"], g["min_us"]
        del a, b, c
    out["tf32_roofline"] = {"bound": "tensor", "achieved": out["tf32_relu_4096_tflops"], "peak": tf32_peak,
                            "unit": "TFLOP/s", "frac": out["tf32_relu_4096_tflops"] / tf32_peak,
                            "peak_source": f"{peaks['source']} bf16 burst / 2",
                            "sustained_achieved": out["tf32_relu_4096_sustained_tflops"],
                            "sustained_peak": peaks.get("bf16_tflops_sustained", 0.0) / 2.0,
                            "sustained_frac": out["tf32_relu_4096_sustained_tflops"] /
                            max(peaks.get("bf16_tflops_sustained", 0.0) / 2.0, 1e-9),
                            "traffic": NCU_TRAFFIC_BYTES["tf32_4096"]}

    # TF32 registry entries for the shapes the tile kernels fit badly, each beside cuBLAS TF32
    # (microseconds per call, alpha = 1, beta = 0): 1024^3 (benchmark configuration), decode-like
    # rows (FP32 stream / split-K cluster), misaligned operands (warp-specialised loader). Event
    # timing through the API (includes the host's launch path) and graph timing (device time).
    for label, (m_, n_, k_) in (("1024", (1024, 1024, 1024)), ("1x4096x4096", (1, 4096, 4096)),
                                ("16x4096x4096", (16, 4096, 4096)), ("1024x1024x8192", (1024, 1024, 8192)),
                                ("4095x4093x4091", (4095, 4093, 4091))):
        a = [torch.randn(m_, k_, device=dev) for _ in range(2)]
        b = [torch.randn(k_, n_, device=dev) for _ in range(2)]
        arms = {"ours": lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1]),
                "cublas": lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1], kernel="cublas")}
        res = cmp.run(arms)
        out[f"tf32_{label}_us"] = 1e3 * res["ours"]["ms"]
        out[f"tf32_{label}_cublas_us"] = 1e3 * res["cublas"]["ms"]
        out[f"tf32_{label}_mhz"] = res["ours"]["mhz"]
        out[f"tf32_{label}_cublas_mhz"] = res["cublas"]["mhz"]
        arms["ours"](0)
        out[f"tf32_{label}_kernel"] = _C.adaptive_gemm_last_kernel()
        if m_ * n_ * k_ <= 1024 * 1024 * 8192:
            g = graph_us(lambda: pkg.adaptive_gemm(a[0], b[0]))
            gc = graph_us(lambda: pkg.adaptive_gemm(a[0], b[0], kernel="cublas"))
            out[f"tf32_{label}_graph_us"], out[f"tf32_{label}_graph_min_us"] = g["median_us"], g["min_us"]
            out[f"tf32_{label}_cublas_graph_us"], out[f"tf32_{label}_cublas_graph_min_us"] = gc["median_us"], gc["min_us"]
        del a, b

    # Automatic dispatch against cuBLASLt with its ReLU fused over mid-sized and long-K shapes, where the
    # choice of registry entry decides: D = relu(A B + 0.5 C), graph-timed, each arm measured twice in
    # turn (the first measurement after fresh allocations runs at a clock that has not settled) and
    # the second measurement reported. The timed measurement of each arm follows 0.6 s of idling: the
    # clock the power cap left behind after the seconds of dense tensor work before it (about
    # 1400 MHz, sw_power_cap) slows a 20 us problem by a third and the two arms unequally; the
    # median SM clock of each arm's measurement is part of the row.
    sweep = []
    for m_, n_, k_ in ((512, 512, 512), (1280, 1280, 1280), (1536, 1536, 1536), (1792, 1792, 1792), (2048, 2048, 2048),
                       (2304, 2304, 2304), (3072, 3072, 3072),
                       (1024, 1024, 4096), (1024, 4096, 4096), (512, 4096, 4096), (64, 4096, 4096), (1280, 1280, 8192),
                       (1024, 2048, 4096), (4096, 4096, 512)):
        a, b, c = (torch.randn(m_, k_, device=dev), torch.randn(k_, n_, device=dev), torch.randn(m_, n_, device=dev))
        ours = lambda: pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, epilogue="relu")
        lt = lambda: pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, epilogue="relu", kernel="cublaslt")
        ours()
        entry = _C.adaptive_gemm_last_kernel()
        graph_us(ours), graph_us(lt)
        timed = {}
        for arm, fn in (("ours", ours), ("lt", lt)):
            time.sleep(0.6)
            with ClockSampler(device_index) as clocks:
                timed[arm] = graph_us(fn)["median_us"]
            timed[arm + "_mhz"] = clocks.median_mhz()
        sweep.append({"shape": f"{m_}x{n_}x{k_}", "kernel": entry, "us": round(timed["ours"], 2),
                      "cublaslt_fused_us": round(timed["lt"], 2), "speed_vs_cublaslt": round(timed["lt"] / timed["ours"], 3),
                      "mhz": timed["ours_mhz"], "cublaslt_mhz": timed["lt_mhz"]})
        del a, b, c
    out["tf32_dispatch_sweep"] = sweep

    # Row operators: bytes = one read of x + one write of y (+ weight once).
    rows, hidden = 16384, 4096
    xs = [torch.randn(rows, hidden, device=dev) for _ in range(2)]
    w = torch.rand(hidden, device=dev) + 0.5
    rms_bytes = 2.0 * rows * hidden * 4 + hidden * 4
    res = cmp.run({"ours": lambda i: pkg.rmsnorm(xs[i & 1], w, 1e-6), "torch": lambda i: eager_rmsnorm(xs[i & 1], w)})
    out["rmsnorm_16384x4096_gbs"] = rms_bytes / res["ours"]["ms"] / 1e6
    out["rmsnorm_torch_gbs"] = rms_bytes / res["torch"]["ms"] / 1e6
    out["rmsnorm_16384x4096_mhz"] = res["ours"]["mhz"]
    del xs
    rows, cols = 32768, 1024
    ls = [2 * torch.randn(rows, cols, device=dev) for _ in range(3)]   # 3 x 128 MiB rotate through L2
    sm_bytes = 2.0 * rows * cols * 4
    res = cmp.run({"ours": lambda i: pkg.softmax(ls[i % 3]), "torch": lambda i: torch.softmax(ls[i % 3], dim=1)})
    out["softmax_32768x1024_gbs"] = sm_bytes / res["ours"]["ms"] / 1e6
    out["softmax_torch_gbs"] = sm_bytes / res["torch"]["ms"] / 1e6
    out["softmax_32768x1024_mhz"] = res["ours"]["mhz"]
    del ls
    for key in ("rmsnorm_16384x4096_gbs", "softmax_32768x1024_gbs"):
        out[key.replace("_gbs", "_roofline")] = {
            "bound": "hbm", "achieved": out[key], "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": out[key] / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth",
            "traffic": NCU_TRAFFIC_BYTES[key.replace("_gbs", "")]}
    return out


def rebuilt_reference_figures() -> dict:
    """The upstream project's own kernels, rebuilt for this GPU, timed in a child process (both
    packages are called `cuda_ai_kernels`). Present only where that build was staged beside the
    repository; otherwise the reason is reported."""
    ref_pkg = REPO / "baseline" / "_ref" / "cuda_ai_kernels"
    if not ref_pkg.is_dir() or not list(ref_pkg.glob("_C*.so")):
        return {"unavailable": "no rebuilt upstream extension under baseline/_ref"}
    script = PACKAGE / "benchmarks" / "compare_reference.py"
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT")}
    try:
        proc = subprocess.run([sys.executable, str(script), "--arm", "reference", "--quick"], capture_output=True,
                              text=True, timeout=600, env=env)
    except subprocess.TimeoutExpired:
        return {"unavailable": "child process exceeded 600 s"}
    line = next((l for l in proc.stdout.splitlines() if l.startswith("RESULT ")), None)
    if line is None:
        return {"unavailable": (proc.stderr or proc.stdout)[-300:]}
    data = json.loads(line[7:])
    out = {"method": "CUDA-graph replay, median", "module": data.get("module")}
    for item in data.get("gemm", []):
        out[f"sgemm_{item['impl']}_{'x'.join(map(str, item['shape']))}_tflops"] = item["tflops_median"]
    for item in data.get("adaptive", []):
        out[f"tf32_{item['case']}_{item['size']}_tflops"] = item["tflops_median"]
    for item in data.get("rows", []):
        out[f"{item['case']}_gbs"] = item["gbs_median"]
    return out


# ------------------------------------------------------------------------ host link


def measure_host_link(dev, world: int, dist) -> dict:
    """Plain pinned cudaMemcpyAsync bandwidth of this rank's host link, all ranks copying at once."""
    nbytes = 256 << 20
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    device = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    device.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    out = {}
    for name, fn in (("h2d", lambda i: device.copy_(host, non_blocking=True)),
                     ("d2h", lambda i: host.copy_(device, non_blocking=True))):
        if world > 1:
            dist.barrier()
        gbs = nbytes * 4 / event_time_ms(fn, 4) / 1e6
        if world > 1:
            t = torch.tensor([gbs], device=dev)
            gathered = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(gathered, t)
            vals = [float(g.item()) for g in gathered]
        else:
            vals = [gbs]
        out[f"{name}_gbs_per_rank"] = round(statistics.fmean(vals), 2)
        out[f"{name}_gbs_per_rank_min"] = round(min(vals), 2)
        out[f"{name}_gbs_aggregate"] = round(sum(vals), 2)
    return out


# ---------------------------------------------------------------- the sharded configuration


def measure_c5(pkg, dev, rank: int, world: int, dist, impl: str, device_index: int) -> dict:
    """M = 32768 split over the ranks, N = K = 8192 (strong scaling): FP32 SIMT and TF32 paths,
    all-gather of C as a separate collective and fused into the kernels' epilogues."""
    from cuda_ai_kernels import _C, sharded

    out: dict = {"m": C5_M, "n": C5_N, "k": C5_K, "n_gpus": world}
    plan = sharded.shard_rows(C5_M, world)
    first, rows = plan[rank]
    out["rows_per_rank"] = rows
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    b = torch.randn(C5_K, C5_N, device=dev, generator=g)          # replicated: same seed on every rank
    g.manual_seed(1000 + rank)
    a_rows = torch.randn(rows, C5_K, device=dev, generator=g)     # TF32 path: contiguous row slab
    a_col = a_rows.t().contiguous().t()                           # FP32 path: column-major shard, made once

    # Parity gate on 48 sampled rows of this rank's shard (a row of C depends on that row of A only).
    sample = torch.randperm(rows, device=dev, generator=g)[:48]
    expected = (a_rows[sample].cpu().double() @ b.cpu().double()).float()
    c = pkg.gemm(a_col, b, impl=impl)
    tol = 1e-4 * C5_K ** 0.5 * float(a_rows.abs().max()) * float(b.abs().max())
    err32 = (c[sample].cpu() - expected).abs().max().item()
    d = pkg.adaptive_gemm(a_rows, b)
    out["tf32_kernel"] = _C.adaptive_gemm_last_kernel()
    rel = float((d[sample].cpu().double() - expected.double()).norm() / expected.double().norm())
    del d
    gate = torch.tensor([int(err32 <= tol and rel <= 5e-3)], device=dev)
    if world > 1:
        dist.all_reduce(gate, op=dist.ReduceOp.MIN)
    out["parity"] = {"fp32_max_abs_error": err32, "fp32_tolerance": tol, "tf32_rel_frobenius": rel, "rows_sampled": 48,
                     "passed_on_every_rank": bool(gate.item())}
    if not bool(gate.item()):
        out["error"] = "parity gate failed; nothing timed"
        return out

    def reduce_max(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    flop = 2.0 * C5_M * C5_N * C5_K
    sampler = ClockSampler(device_index)

    def timed(fn, warm: int, steps: int) -> tuple[float, object]:
        for i in range(warm):
            fn(i)
        if world > 1:
            dist.barrier()
        with sampler:
            ms = event_time_ms(fn, steps) / steps
        return reduce_max(ms), sampler.median_mhz()

    ms, mhz = timed(lambda i: pkg.gemm(a_col, b, impl=impl), 2, 3)
    out.update(fp32_ms=ms, fp32_tflops_total=flop / ms / 1e9, fp32_mhz=mhz)
    ms, mhz = timed(lambda i: pkg.adaptive_gemm(a_rows, b), 3, 10)
    out.update(tf32_ms=ms, tf32_tflops_total=flop / ms / 1e9, tf32_mhz=mhz)
    if world == 1:
        return out

    # All-gather of the 1 GiB C: as a collective on its own, after the GEMM, and fused into the GEMM.
    counts = [count for _, count in plan]
    full = torch.empty(C5_M, C5_N, device=dev)
    ms, _ = timed(lambda i: dist.all_gather_into_tensor(full, c), 2, 5)
    received = (C5_M - rows) * C5_N * 4
    out.update(allgather_c_ms=ms, allgather_c_recv_gbs_per_rank=received / ms / 1e6)
    ms, _ = timed(lambda i: dist.all_gather_into_tensor(full, pkg.gemm(a_col, b, impl=impl)), 1, 3)
    out["fp32_then_allgather_ms"] = ms
    ms, _ = timed(lambda i: dist.all_gather_into_tensor(full, pkg.adaptive_gemm(a_rows, b)), 2, 10)
    out["tf32_then_allgather_ms"] = ms

    fused_impl = impl if impl in ("prefetch_smem", "prefetch_reg") else "prefetch_reg"
    gathered, why = None, ""
    try:
        gathered = sharded.GatheredOutput(C5_M, C5_N, plan)
    except Exception as exc:  # noqa: BLE001
        why = f"{type(exc).__name__}: {exc}"[:200]
    if not sharded.all_ranks_ok(gathered is not None):
        out["fused_error"] = why or "symmetric allocation failed on another rank"
        return out
    failure = [None]

    def guarded(fn):
        """A step of the fused path; after a failure nothing more is enqueued on this rank (the
        others' bounded barriers give up and report instead of spinning)."""
        def run(i):
            if failure[0] is None:
                try:
                    fn(i)
                    gathered.barrier()
                except Exception as exc:  # noqa: BLE001
                    failure[0] = f"{type(exc).__name__}: {exc}"[:200]
        return run

    fp32_fused = guarded(lambda i: sharded.sharded_gemm_gather(a_col, b, gathered, impl=fused_impl))
    tf32_fused = guarded(lambda i: sharded.sharded_adaptive_gemm_gather(a_rows, b, gathered))
    same = []
    for fused_fn, collective in ((fp32_fused, lambda: pkg.gemm(a_col, b, impl=fused_impl)),
                                 (tf32_fused, lambda: pkg.adaptive_gemm(a_rows, b))):
        dist.all_gather_into_tensor(full, collective())
        fused_fn(0)
        torch.cuda.synchronize()
        same.append(bool(torch.equal(gathered.full, full)))
        if not sharded.all_ranks_ok(failure[0] is None):
            break
        gathered.barrier()      # nobody overwrites a copy that a peer is still comparing
    ok = sharded.all_ranks_ok(failure[0] is None and all(same) and len(same) == 2)
    out["fused_bit_identical"] = ok
    if ok:
        ms, _ = timed(fp32_fused, 1, 3)
        out["fp32_fused_ms"] = ms
        ms, _ = timed(tf32_fused, 2, 10)
        out["tf32_fused_ms"] = ms
        try:
            gathered.check()
        except RuntimeError as exc:
            failure[0] = str(exc)[:200]
    if failure[0] is not None:
        out["fused_error"] = failure[0]
    out["fused_impl"] = fused_impl
    return out


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--sgemm-impl", default="prefetch_reg")
    parser.add_argument("--no-extras", action="store_true")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    torch.set_num_threads(max(1, host_threads() // max(1, world)))   # the parity gates run on the CPU
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    dist = None
    if distributed:
        import torch.distributed as dist  # noqa: F811

        from cuda_ai_kernels import sharded

        sharded.init_distributed("nccl", timeout_s=600.0, device=dev)

    import cuda_ai_kernels as pkg
    from cuda_ai_kernels import _C  # noqa: F401 - no extension, no benchmark
    from oracle import oracle

    peaks = load_peaks()
    impl = args.sgemm_impl
    launches_per_step = 2 if impl == "split_k" else 1  # split_k clears its output with a memset node first

    # This rank's shard: rows [rank*M, (rank+1)*M) of a (world*M) x K matrix A, full B.
    a_cpu, b_cpu = oracle.ladder_inputs(M, N, K, seed=rank)
    if distributed:
        _, b_cpu = oracle.ladder_inputs(M, N, K, seed=0)  # B is replicated
    a_storage = a_cpu.t()  # contiguous [K, M]
    a_sets = [a_storage.to(dev).t(), a_storage.flip(1).contiguous().to(dev).t()]
    b_sets = [b_cpu.to(dev), b_cpu.flip(1).contiguous().to(dev)]

    def step(i):
        return pkg.gemm(a_sets[i & 1], b_sets[i & 1], impl=impl)

    # Correctness gate before any timing, as the reference's harness does.
    check = step(0)
    expected = oracle.gemm_fp64(a_cpu[:256], b_cpu)
    err = (check[:256].cpu() - expected).abs().max().item()
    tol = oracle.sgemm_abs_tolerance(a_cpu, b_cpu)
    if not err <= tol:
        raise SystemExit(f"gemm[{impl}] failed its parity gate: max abs error {err:.3e} > {tol:.3e}")
    del check

    for i in range(args.warmup):
        step(i)
    if distributed:
        dist.barrier()
    with ClockSampler(local_rank) as clocks:
        elapsed_ms = event_time_ms(step, args.steps)
    if distributed:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        elapsed_ms = float(t.item())
    flops_per_step = 2.0 * M * N * K * world
    value = flops_per_step * args.steps / elapsed_ms / 1e9
    per_gpu_tflops = value / world

    # End to end through the operator API from pinned host memory. Every step copies its operands
    # from the host and reads its C back; the legs run on separate streams with two device slots, so
    # the upload of step i + 1 and the download of step i - 1 overlap the GEMM of step i (PCIe is
    # full duplex); nothing is skipped, reused or left on the device. With several ranks a rank
    # uploads its own rows of A and K / world rows of B; an all-gather over NVLink (NCCL) completes
    # B on every GPU, so every byte of B crosses PCIe once instead of once per rank.
    k_rows = K // world
    a_host = a_cpu.t().contiguous().pin_memory()   # storage [K, M]
    b_host = b_cpu[rank * k_rows:(rank + 1) * k_rows].contiguous().pin_memory()   # this rank's rows of B (all of it alone)
    c_host = [torch.empty(M, N).pin_memory() for _ in range(2)]
    a_stage = [torch.empty(K, M, device=dev) for _ in range(2)]
    b_part = [torch.empty(k_rows, N, device=dev) for _ in range(2)]
    b_stage = [torch.empty(K, N, device=dev) for _ in range(2)] if distributed else b_part
    up, gather, compute, down = (torch.cuda.Stream(dev) for _ in range(4))
    slot_free = [torch.cuda.Event() for _ in range(2)]     # GEMM that read the slot has finished
    host_free = [torch.cuda.Event() for _ in range(2)]     # download into the host slot has finished

    def e2e_step(i):
        slot = i & 1
        with torch.cuda.stream(up):
            up.wait_event(slot_free[slot])
            a_stage[slot].copy_(a_host, non_blocking=True)
            b_part[slot].copy_(b_host, non_blocking=True)
            ready = up.record_event()
        if distributed:
            with torch.cuda.stream(gather):
                gather.wait_event(ready)
                dist.all_gather_into_tensor(b_stage[slot], b_part[slot])
                ready = gather.record_event()
        with torch.cuda.stream(compute):
            compute.wait_event(ready)
            c_dev = pkg.gemm(a_stage[slot].t(), b_stage[slot], impl=impl)
            slot_free[slot].record(compute)
            computed = compute.record_event()
        with torch.cuda.stream(down):
            down.wait_event(computed)
            down.wait_event(host_free[slot])
            c_host[slot].copy_(c_dev, non_blocking=True)
            c_dev.record_stream(down)
            host_free[slot].record(down)

    streams = (up, gather, compute, down)

    def e2e_run(steps: int) -> float:
        """Milliseconds from the first upload to the last download of `steps` steps."""
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        main_stream = torch.cuda.current_stream()
        begin.record(main_stream)
        for stream in streams:
            stream.wait_event(begin)
        for i in range(steps):
            e2e_step(i)
        for stream in streams:
            main_stream.wait_stream(stream)
        end.record(main_stream)
        torch.cuda.synchronize()
        return begin.elapsed_time(end)

    # Enough steps that filling and draining the pipeline (one upload, one GEMM and one download
    # that overlap nothing) weigh little: 40 steps take about 0.1 s.
    # The host link is shared with whatever else runs on the box (one run in a dozen was seen at half
    # its usual rate for a fraction of a second), so the 40-step region is timed five times and the
    # median is reported, with all five beside it.
    # With several ranks the first hundred or so steps run slower (four ranks: 9.0, 6.3, 4.4, 3.8,
    # 3.7 ms per step over five repeats after a four-step warm-up; one rank shows no such ramp), so the
    # warm-up there is two untimed repeats.
    e2e_steps = max(args.steps, 40)
    if distributed:
        for _ in range(2):
            dist.barrier()
            e2e_run(e2e_steps)
    else:
        e2e_run(4)
    e2e_samples = []
    for _ in range(5):
        if distributed:
            dist.barrier()
        ms = e2e_run(e2e_steps)
        if distributed:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        e2e_samples.append(ms)
    e2e_ms = statistics.median(e2e_samples)
    e2e_value = flops_per_step * e2e_steps / e2e_ms / 1e9
    e2e_err = max((c[:256] - expected).abs().max().item() for c in c_host)
    if not e2e_err <= tol:
        raise SystemExit(f"end-to-end result failed its parity gate: {e2e_err:.3e} > {tol:.3e}")
    h2d_bytes = (world * M * K + K * N) * 4        # every rank its rows of A; B once in total
    d2h_bytes = world * M * N * 4

    also: dict = {}
    also.update(measure_host_link(dev, world, dist))
    also["e2e_b_upload"] = "K/world rows of B per rank over PCIe, all-gather over NVLink" if distributed else "full B per step"
    del a_stage, b_part, b_stage, c_host

    if distributed:
        from cuda_ai_kernels import sharded

        # Optional collective, timed on its own: gather the row shards of C on every rank.
        c_shard = step(0)
        gathered = torch.empty(world * M, N, device=dev)
        for _ in range(3):
            dist.all_gather_into_tensor(gathered, c_shard)
        dist.barrier()
        gather_ms = event_time_ms(lambda i: dist.all_gather_into_tensor(gathered, c_shard), 10) / 10
        t = torch.tensor([gather_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        recv_bytes = (world - 1) * M * N * 4
        also["allgather_c_ms"] = float(t.item())
        also["allgather_c_recv_gbs_per_rank"] = recv_bytes / float(t.item()) / 1e6
        del gathered, c_shard
        # The same gather fused into the GEMM: the kernel's epilogue stores every tile into every
        # rank's copy of C (peer stores over NVLink), one device-side barrier per step. Reported
        # beside "GEMM, then the collective"; never part of `value`. A box where the symmetric
        # allocation cannot be set up reports why instead of a number. Only the two pipeline
        # entries that store each tile once can fan out; any other --sgemm-impl uses prefetch_reg here.
        fused_impl = impl if impl in ("prefetch_smem", "prefetch_reg") else "prefetch_reg"
        also["gemm_fused_allgather_impl"] = fused_impl
        out, setup_error = None, ""
        try:
            out = sharded.GatheredOutput(world * M, N, [(r * M, M) for r in range(world)])
        except Exception as exc:  # noqa: BLE001
            setup_error = f"{type(exc).__name__}: {exc}"[:200]
        # Every rank goes on only if every rank has its buffer: no rank may wait alone.
        if not sharded.all_ranks_ok(out is not None):
            also["gemm_fused_allgather_error"] = setup_error or "symmetric allocation failed on another rank"
        else:
            failure = [None]

            def fused(i):
                # After a failure this rank enqueues nothing more; the other ranks' barriers are
                # bounded, give up and report through the status word instead of spinning.
                if failure[0] is None:
                    try:
                        sharded.sharded_gemm_gather(a_sets[i & 1], b_sets[i & 1], out, impl=fused_impl)
                        out.barrier()
                    except Exception as exc:  # noqa: BLE001
                        failure[0] = f"{type(exc).__name__}: {exc}"[:200]

            def sequential(i):
                dist.all_gather_into_tensor(seq_out, pkg.gemm(a_sets[i & 1], b_sets[i & 1], impl=fused_impl))

            seq_out = torch.empty(world * M, N, device=dev)
            for name, fn in (("gemm_then_allgather_ms", sequential), ("gemm_fused_allgather_ms", fused)):
                for i in range(3):
                    fn(i)
                if not sharded.all_ranks_ok(failure[0] is None):
                    break
                dist.barrier()
                t = torch.tensor([event_time_ms(fn, 10) / 10], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                also[name] = float(t.item())
            if sharded.all_ranks_ok(failure[0] is None):
                fused(0), sequential(0)
                torch.cuda.synchronize()
                same = torch.tensor([int(torch.equal(out.full, seq_out))], device=dev)
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
                also["gemm_fused_allgather_bit_identical"] = bool(same.item())
                try:
                    out.check()
                except RuntimeError as exc:
                    failure[0] = str(exc)[:200]
            if not sharded.all_ranks_ok(failure[0] is None):
                also["gemm_fused_allgather_error"] = failure[0] or "another rank failed"
            del seq_out, out

    del a_sets, b_sets
    torch.cuda.empty_cache()
    if not args.no_extras:
        also["c5"] = measure_c5(pkg, dev, rank, world, dist, impl, local_rank)
        for key in ("fp32_ms", "tf32_ms", "fp32_tflops_total", "tf32_tflops_total"):
            if key in also["c5"]:
                also[f"c5_{key}"] = also["c5"][key]
        torch.cuda.empty_cache()

    cpu_baseline = None
    if rank == 0 and world == 1:
        torch.set_num_threads(host_threads())
        cpu_baseline = cpu_baseline_block(a_cpu, b_cpu, repeats=3)
        if not args.no_extras:
            also["cpu_rowops"] = cpu_rowop_seconds()
            also.update(measure_extras(pkg, peaks, local_rank, warmup=args.warmup))
            torch.cuda.empty_cache()
            also["upstream_kernels_rebuilt"] = rebuilt_reference_figures()

    if rank == 0:
        clk = clocks.summary()
        sm_max = peaks.get("sm_max_mhz", 1965.0)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        fma_peak = 2.0 * FP32_LANES_PER_SM * sms * sm_max * 1e6 / 1e12
        roofline = {"bound": "fp32_fma", "achieved": per_gpu_tflops, "peak": fma_peak, "unit": "TFLOP/s",
                    "frac": per_gpu_tflops / fma_peak,
                    "peak_source": f"2 flop x {FP32_LANES_PER_SM} lanes x {sms} SMs x {sm_max:.0f} MHz (max SM clock)",
                    "traffic": NCU_TRAFFIC_BYTES["sgemm_4096"]}
        if clk.get("sm_mhz"):
            roofline["frac_at_observed_clock"] = per_gpu_tflops / (fma_peak * clk["sm_mhz"] / sm_max)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": per_gpu_tflops / PUBLISHED_A800_SPLIT_K_TFLOPS, "dtype": "f32",
            "data": "synthetic",
            "config": make_config(world, impl),
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "repeats": len(e2e_samples),
                    "ms_per_step_each_repeat": [round(ms / e2e_steps, 4) for ms in e2e_samples]},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clk,
            "also": also,
        }
        print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
