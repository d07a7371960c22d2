"""Benchmark of the hot path on B200. Prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--sgemm-impl NAME] [--no-extras]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (N = 1): FP32 SIMT GEMM, M = N = K = 4096, A column-major,
B and C row-major, N(0,1) inputs from seed 0 - the configuration the reference
publishes its numbers on. One step is one `cuda_ai_kernels.gemm` call.

  value     TFLOP/s (2*M*N*K / device time) with inputs resident in HBM, CUDA
            events around exactly K steps on the launching stream; two input
            sets are rotated so that a step never finds its operands in L2.
  e2e       the same metric through the operator API from pinned HOST buffers:
            host->device copies of A and B and the device->host read of C are
            inside the timed region of every step; upload, GEMM and download of
            neighbouring steps overlap on three streams.
  roofline  the dominant kernel against the FP32 FMA peak; `also` carries the
            TF32 tensor-core GEMM (tensor roofline) and the two row operators
            (HBM roofline) measured in the same run, next to cuBLAS.
  cpu_baseline  the reference's CPU-capable path - its FP64 torch matmul oracle -
            timed on this host's cores (rank 0, N = 1).

N > 1 (one rank per GPU under torchrun): the GEMM is sharded along M - every
rank owns 4096 rows of A and a full B, C stays sharded, no data-path collective
(weak scaling). An all-gather of C over NCCL is timed separately and reported
under `also`.

`--impl reference` times the reference's own CPU implementation of the path
(the FP64 oracle expression) on the host cores, one full 4096^3 product per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
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
METRIC = "fp32_simt_gemm_4096_tflops"
UNIT = "TFLOP/s"
FP32_LANES_PER_SM = 128
# The reference's published figure for this metric: split_k at 4096^3 on an
# A800 80GB PCIe, 17.206 TFLOP/s (its README.md:17). Other hardware; per GPU.
PUBLISHED_A800_SPLIT_K_TFLOPS = 17.206
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the
# committed Nsight Compute captures of exactly these workloads (profiles/*.md).
# bench.py cannot run ncu on itself; the figures are carried here so that the
# roofline objects can set traffic beside the algorithmic bytes.
NCU_TRAFFIC_BYTES = {
    "sgemm_4096": 334.2e6 + 54.9e6,      # profiles/sgemm_pipeline_4096.md (algorithmic: 201 MB of operands + output)
    "tf32_4096": 372.6e6 + 50.7e6,       # profiles/tf32_umma_4096.md (CTA-pair kernel)
    "rmsnorm_16384x4096": 268.5e6 + 213.0e6,   # profiles/rowops_c4.md (writes partly still in L2 at kernel end)
    "softmax_32768x1024": 134.2e6 + 78.2e6,
}


def load_peaks() -> dict:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        peaks["source"] = "measured"
        return peaks
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "sm_max_mhz": 1965.0,
            "source": "fallback"}


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
        if self._handle is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

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


def event_time_ms(fn, steps: int, stream=None) -> float:
    """Device time of `steps` calls of fn(i), CUDA events on the current stream."""
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for i in range(steps):
        fn(i)
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end)


def cpu_oracle_seconds(a_cpu, b_cpu, repeats: int) -> float:
    from oracle import oracle

    oracle.gemm_fp64(a_cpu, b_cpu)  # warm-up
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.gemm_fp64(a_cpu, b_cpu)
        best = min(best, time.perf_counter() - t0)
    return best


def run_reference(args, rank: int) -> None:
    """The reference's CPU path (its FP64 torch oracle) on the host cores."""
    if rank != 0:
        return
    from oracle import oracle

    a_cpu, b_cpu = oracle.ladder_inputs(M, N, K, seed=0)
    for _ in range(args.warmup):
        oracle.gemm_fp64(a_cpu, b_cpu)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemm_fp64(a_cpu, b_cpu)
    elapsed = time.perf_counter() - t0
    tflops = 2.0 * M * N * K * args.steps / elapsed / 1e12
    cores = torch.get_num_threads()
    sample = f"{args.steps} full {M}x{N}x{K} FP64 products, (A.double() @ B.double()).float(), column-major A"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"fp32_gemm_{M}x{N}x{K}_colmajorA", "host_cores": os.cpu_count()},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def measure_extras(pkg, peaks: dict, steps: int, warmup: int) -> dict:
    """TF32 GEMM, row operators and library baselines, same process, same GPU."""
    from oracle import oracle

    out: dict = {}
    dev = "cuda"

    def timed(fn, flush=None):
        for i in range(warmup):
            fn(i)
        return event_time_ms(fn, steps) / steps

    # cuBLAS strict-FP32 SGEMM through the operator API, same inputs as the headline.
    a_sets = [torch.randn(K, M, device=dev).t() for _ in range(2)]
    b_sets = [torch.randn(K, N, device=dev) for _ in range(2)]
    flops = 2.0 * M * N * K
    for name in ("cublas", "prefetch_smem", "prefetch_reg", "split_k", "thread_tile_8x8", "warp_tile"):
        ms = timed(lambda i, name=name: pkg.gemm(a_sets[i & 1], b_sets[i & 1], impl=name))
        out[f"sgemm_{name}_tflops"] = flops / ms / 1e9
    del a_sets, b_sets
    # The other two FP32 benchmark shapes: 1024^3 and 1024 x 4096 x 4096, where tiles do not fill
    # whole rounds of SMs and the stream-K entry (output cleared inside the timed call) matters.
    for (m_, n_, k_) in ((1024, 1024, 1024), (1024, 4096, 4096)):
        a_small = [torch.randn(k_, m_, device=dev).t() for _ in range(2)]
        b_small = [torch.randn(k_, n_, device=dev) for _ in range(2)]
        for name in ("cublas", "prefetch_reg", "split_k"):
            ms = timed(lambda i, name=name: pkg.gemm(a_small[i & 1], b_small[i & 1], impl=name))
            out[f"sgemm_{name}_{m_}x{n_}x{k_}_tflops"] = 2.0 * m_ * n_ * k_ / ms / 1e9
        del a_small, b_small

    # TF32 tcgen05 GEMM with fused epilogue, D = relu(A@B + 0.5*C), and cuBLAS TF32.
    tf32_peak = peaks["bf16_tflops"] / 2.0
    for size in (4096, 8192):
        a = [torch.randn(size, size, device=dev) for _ in range(2)]
        b = [torch.randn(size, size, device=dev) for _ in range(2)]
        c = torch.randn(size, size, device=dev)
        f = 2.0 * size ** 3
        ms = timed(lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1], c=c, alpha=1.0, beta=0.5, epilogue="relu"))
        out[f"tf32_relu_{size}_tflops"] = f / ms / 1e9
        ms = timed(lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1], c=c, alpha=1.0, beta=0.5, epilogue="linear"))
        out[f"tf32_linear_{size}_tflops"] = f / ms / 1e9
        ms = timed(lambda i: torch.relu_(pkg.adaptive_gemm(a[i & 1], b[i & 1], c=c, alpha=1.0, beta=0.5,
                                                           kernel="cublas")))
        out[f"tf32_cublas_unfused_relu_{size}_tflops"] = f / ms / 1e9
        del a, b, c
    out["tf32_roofline"] = {"bound": "tensor", "achieved": out["tf32_relu_4096_tflops"], "peak": tf32_peak,
                            "unit": "TFLOP/s", "frac": out["tf32_relu_4096_tflops"] / tf32_peak,
                            "peak_source": f"{peaks['source']} bf16 burst / 2",
                            "traffic": NCU_TRAFFIC_BYTES["tf32_4096"]}

    # TF32 registry entries for the shapes the tile kernels fit badly, each beside cuBLAS TF32
    # (microseconds per call, alpha = 1, beta = 0): 1024^3 (benchmark configuration), decode-like
    # rows (FP32 stream / split-K cluster), misaligned operands (warp-specialised loader).
    from cuda_ai_kernels import _C

    for label, (m_, n_, k_) in (("1024", (1024, 1024, 1024)), ("1x4096x4096", (1, 4096, 4096)),
                                ("16x4096x4096", (16, 4096, 4096)), ("1024x1024x8192", (1024, 1024, 8192)),
                                ("4095x4093x4091", (4095, 4093, 4091))):
        a = [torch.randn(m_, k_, device=dev) for _ in range(2)]
        b = [torch.randn(k_, n_, device=dev) for _ in range(2)]
        ms = timed(lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1]))
        out[f"tf32_{label}_us"] = ms * 1e3
        out[f"tf32_{label}_kernel"] = _C.adaptive_gemm_last_kernel()
        ms = timed(lambda i: pkg.adaptive_gemm(a[i & 1], b[i & 1], kernel="cublas"))
        out[f"tf32_{label}_cublas_us"] = ms * 1e3
        del a, b

    # Row operators: bytes = one read of x + one write of y (+ weight once).
    rows, hidden = 16384, 4096
    xs = [torch.randn(rows, hidden, device=dev) for _ in range(2)]
    w = torch.rand(hidden, device=dev) + 0.5
    ms = timed(lambda i: pkg.rmsnorm(xs[i & 1], w, 1e-6))
    rms_bytes = 2.0 * rows * hidden * 4 + hidden * 4
    out["rmsnorm_16384x4096_gbs"] = rms_bytes / ms / 1e6
    ms = timed(lambda i: oracle_free_torch_rmsnorm(xs[i & 1], w))
    out["rmsnorm_torch_gbs"] = rms_bytes / ms / 1e6
    del xs
    rows, cols = 32768, 1024
    ls = [2 * torch.randn(rows, cols, device=dev) for _ in range(3)]   # 3 x 128 MiB rotate through L2
    ms = timed(lambda i: pkg.softmax(ls[i % 3]))
    sm_bytes = 2.0 * rows * cols * 4
    out["softmax_32768x1024_gbs"] = sm_bytes / ms / 1e6
    ms = timed(lambda i: torch.softmax(ls[i % 3], dim=1))
    out["softmax_torch_gbs"] = sm_bytes / ms / 1e6
    del ls
    for key in ("rmsnorm_16384x4096_gbs", "softmax_32768x1024_gbs"):
        out[key.replace("_gbs", "_roofline")] = {
            "bound": "hbm", "achieved": out[key], "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": out[key] / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth",
            "traffic": NCU_TRAFFIC_BYTES[key.replace("_gbs", "")]}
    return out


def oracle_free_torch_rmsnorm(x, w, eps: float = 1e-6):
    """Eager PyTorch RMSNorm on the GPU, as the reference's benchmark times it
    (benchmarks/bench_rmsnorm.py:27-29)."""
    return x * torch.rsqrt(torch.mean(x * x, dim=-1, keepdim=True) + eps) * w


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
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import cuda_ai_kernels as pkg
    from cuda_ai_kernels import _C  # noqa: F401 - no extension, no benchmark
    from oracle import oracle

    peaks = load_peaks()
    dev = torch.device("cuda", local_rank)
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

    # End to end through the operator API from pinned host memory. Every step
    # copies its A and B from the host and reads its C back. The three legs run
    # on three streams with two device slots, so the upload of step i + 1 and
    # the download of step i - 1 overlap the GEMM of step i (PCIe is full
    # duplex); nothing is skipped, reused or left on the device.
    a_host = a_cpu.t().contiguous().pin_memory()   # storage [K, M]
    b_host = b_cpu.contiguous().pin_memory()
    c_host = [torch.empty(M, N).pin_memory() for _ in range(2)]
    a_stage = [torch.empty(K, M, device=dev) for _ in range(2)]
    b_stage = [torch.empty(K, N, device=dev) for _ in range(2)]
    up, compute, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    slot_free = [torch.cuda.Event() for _ in range(2)]     # GEMM that read the slot has finished
    host_free = [torch.cuda.Event() for _ in range(2)]     # download into the host slot has finished

    def e2e_step(i):
        slot = i & 1
        with torch.cuda.stream(up):
            up.wait_event(slot_free[slot])
            a_stage[slot].copy_(a_host, non_blocking=True)
            b_stage[slot].copy_(b_host, non_blocking=True)
            uploaded = up.record_event()
        with torch.cuda.stream(compute):
            compute.wait_event(uploaded)
            c_dev = pkg.gemm(a_stage[slot].t(), b_stage[slot], impl=impl)
            slot_free[slot].record(compute)
            computed = compute.record_event()
        with torch.cuda.stream(down):
            down.wait_event(computed)
            down.wait_event(host_free[slot])
            c_host[slot].copy_(c_dev, non_blocking=True)
            c_dev.record_stream(down)
            host_free[slot].record(down)

    def e2e_run(steps: int) -> float:
        """Milliseconds from the first upload to the last download of `steps` steps."""
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        main = torch.cuda.current_stream()
        begin.record(main)
        for stream in (up, compute, down):
            stream.wait_event(begin)
        for i in range(steps):
            e2e_step(i)
        for stream in (up, compute, down):
            main.wait_stream(stream)
        end.record(main)
        torch.cuda.synchronize()
        return begin.elapsed_time(end)

    # Enough steps that filling and draining the three-stage pipeline (one upload, one GEMM and one
    # download that overlap nothing) weigh little: 40 steps take about 0.1 s.
    e2e_steps = max(args.steps, 40)
    e2e_run(4)
    if distributed:
        dist.barrier()
    e2e_ms = e2e_run(e2e_steps)
    if distributed:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = flops_per_step * e2e_steps / e2e_ms / 1e9
    e2e_err = max((c[:256] - expected).abs().max().item() for c in c_host)
    if not e2e_err <= tol:
        raise SystemExit(f"end-to-end result failed its parity gate: {e2e_err:.3e} > {tol:.3e}")

    also: dict = {}
    if distributed:
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
        # allocation cannot be set up reports why instead of a number.
        from cuda_ai_kernels import sharded

        out, setup_error = None, ""
        try:
            out = sharded.GatheredOutput(world * M, N, [(r * M, M) for r in range(world)])
        except Exception as exc:  # noqa: BLE001
            setup_error = f"{type(exc).__name__}: {exc}"[:200]
        # Every rank goes on only if every rank has its buffer: no rank may wait alone in a collective.
        ready = torch.tensor([int(out is not None)], device=dev)
        dist.all_reduce(ready, op=dist.ReduceOp.MIN)
        if not bool(ready.item()):
            also["gemm_fused_allgather_error"] = setup_error or "symmetric allocation failed on another rank"
        else:

            def fused(i):
                sharded.sharded_gemm_gather(a_sets[i & 1], b_sets[i & 1], out, impl=impl)
                out.barrier()

            def sequential(i):
                dist.all_gather_into_tensor(seq_out, step(i))

            seq_out = torch.empty(world * M, N, device=dev)
            for name, fn in (("gemm_then_allgather_ms", sequential), ("gemm_fused_allgather_ms", fused)):
                for i in range(3):
                    fn(i)
                dist.barrier()
                t = torch.tensor([event_time_ms(fn, 10) / 10], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                also[name] = float(t.item())
            fused(0), sequential(0)
            torch.cuda.synchronize()
            same = torch.tensor([int(torch.equal(out.full, seq_out))], device=dev)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            also["gemm_fused_allgather_bit_identical"] = bool(same.item())
            out.barrier()
            del seq_out, out

    cpu_baseline = None
    if rank == 0 and world == 1:
        cores = torch.get_num_threads()
        seconds = cpu_oracle_seconds(a_cpu, b_cpu, repeats=3)
        cpu_baseline = {"value": 2.0 * M * N * K / seconds / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"full {M}x{N}x{K} FP64 torch matmul oracle, best of 3 after 1 warm-up, "
                                  f"{seconds:.3f} s; host has {os.cpu_count()} logical CPUs"}
        if not args.no_extras:
            del a_sets, b_sets, a_stage, b_stage, c_host
            torch.cuda.empty_cache()
            also.update(measure_extras(pkg, peaks, steps=max(5, min(args.steps, 20)), warmup=args.warmup))

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
            "config": {"workload": f"fp32_gemm_{M}x{N}x{K}_colmajorA_per_gpu", "impl": impl,
                       "sharding": "rows of A per rank, B replicated, C sharded" if distributed else "single GPU",
                       "global_m": M * world,
                       "l2": "two input sets alternate (A+B 256 MB > 126 MB L2), no flush kernel"},
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": (M * K + K * N) * 4 * world,
                    "d2h_bytes_per_step": M * N * 4 * world, "steps": e2e_steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clk,
            "also": also,
        }
        print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
