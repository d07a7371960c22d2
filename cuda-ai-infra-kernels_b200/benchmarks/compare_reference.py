"""Side-by-side timing: this package's kernels vs the reference's own sm_80-era
kernels recompiled for the box, cuBLAS, and PyTorch eager row ops.

    python cuda-ai-infra-kernels_b200/benchmarks/compare_reference.py [--out FILE.json] [--quick]

`--quick` keeps the benchmark configurations only (split_k and prefetch_reg at
4096^3, adaptive auto ReLU at 4096^3 and 8192^3, the two row operators);
`--arm reference --quick` is what the repository's `bench.py` runs in a child
process to put the rebuilt upstream kernels beside its own numbers.

Both packages are called `cuda_ai_kernels`, so each arm runs in its own child
process with its own `sys.path`:
  ours       <repo>/cuda-ai-infra-kernels_b200/python
  reference  <repo>/baseline/_ref   (the reference's package with its `_C`
             built for sm_100; not part of the repository, skipped when absent)

Method, as in the reference's harness (benchmarks/bench_gemm_all.py:46-77):
CUDA-graph capture of 10 calls, warm-up 10, 50 timed replays, median and mean;
GEMM throughput = 2*M*N*K / time; row-op bandwidth = (one read + one write) / time.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
ARMS = {
    "ours": REPO / "cuda-ai-infra-kernels_b200" / "python",
    "reference": REPO / "baseline" / "_ref",
}
LADDER = ["naive", "block_tile", "block_tile_float4_16x16", "block_tile_float4_16x32", "block_tile_float4_32x32",
          "thread_tile_4x4", "thread_tile_4x8", "thread_tile_8x8", "thread_tile_8x8_warp4x8", "warp_tile",
          "prefetch_smem", "prefetch_reg", "split_k", "cublas"]
GEMM_SHAPES = [(1024, 1024, 1024), (1024, 4096, 4096), (4096, 4096, 4096)]
ADAPTIVE_SIZES = [1024, 4096, 8192]


def graph_time_ms(torch, fn, warmup=10, repeat=50, calls=10):
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for _ in range(calls):
            fn()
    samples = []
    with torch.cuda.stream(stream):
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        for _ in range(repeat):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
            samples.append(begin.elapsed_time(end) / calls)
    torch.cuda.current_stream().wait_stream(stream)
    return {"median_ms": statistics.median(samples), "mean_ms": statistics.fmean(samples), "min_ms": min(samples)}


def event_time_ms(torch, fn, warmup=10, repeat=50):
    """Plain event timing for kernels that ignore the current stream (the
    reference's row operators launch on the legacy default stream and cannot be
    captured on a side stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(repeat):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        fn()
        end.record()
        end.synchronize()
        samples.append(begin.elapsed_time(end))
    return {"median_ms": statistics.median(samples), "mean_ms": statistics.fmean(samples), "min_ms": min(samples)}


def run_arm(arm: str, quick: bool = False) -> dict:
    sys.path.insert(0, str(ARMS[arm]))
    import torch
    import cuda_ai_kernels as pkg
    from cuda_ai_kernels import _C

    results = {"arm": arm, "module": _C.__file__, "gpu": torch.cuda.get_device_name(0), "gemm": [], "adaptive": [],
               "rows": []}
    torch.manual_seed(0)
    # Quick mode: 3 warm-up calls, 5 calls per graph, 10 replays (the full run: 10 / 10 / 50).
    timing = dict(warmup=3, repeat=10, calls=5) if quick else {}
    gemm_shapes = [(4096, 4096, 4096)] if quick else GEMM_SHAPES
    ladder = ["prefetch_reg", "split_k", "cublas"] if quick else LADDER
    adaptive_sizes = [4096, 8192] if quick else ADAPTIVE_SIZES
    for m, n, k in gemm_shapes:
        a = torch.randn(k, m, device="cuda").t()
        b = torch.randn(k, n, device="cuda")
        expected = (a.double() @ b.double()).float()
        for impl in ladder:
            out = pkg.gemm(a, b, impl=impl)
            err = (out - expected).abs().max().item()
            t = graph_time_ms(torch, lambda: pkg.gemm(a, b, impl=impl), **timing)
            results["gemm"].append({"shape": [m, n, k], "impl": impl, "max_abs_error": err,
                                    "tflops_median": 2.0 * m * n * k / t["median_ms"] / 1e9, **t})
        del a, b, expected
    for size in adaptive_sizes:
        a = torch.randn(size, size, device="cuda")
        b = torch.randn(size, size, device="cuda")
        c = torch.randn(size, size, device="cuda")
        flops = 2.0 * size ** 3
        cases = {
            "auto_relu": lambda: pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, epilogue="relu"),
            "auto_linear": lambda: pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, epilogue="linear"),
            "cublas_plus_torch_relu": lambda: torch.relu_(pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5,
                                                                           kernel="cublas")),
            "cublas_linear": lambda: pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, kernel="cublas"),
        }
        if quick:
            cases = {"auto_relu": cases["auto_relu"]}
        for name, fn in cases.items():
            t = graph_time_ms(torch, fn, **timing)
            results["adaptive"].append({"size": size, "case": name, "tflops_median": flops / t["median_ms"] / 1e9, **t})
        del a, b, c
    x = torch.randn(16384, 4096, device="cuda")
    w = torch.rand(4096, device="cuda") + 0.5
    logits = 2 * torch.randn(32768, 1024, device="cuda")
    row_cases = {
        "rmsnorm_naive": (lambda: pkg.rmsnorm(x, w, 1e-6, impl="naive"), 2.0 * x.numel() * 4 + 4096 * 4),
        "rmsnorm_cache_x": (lambda: pkg.rmsnorm(x, w, 1e-6, impl="cache_x"), 2.0 * x.numel() * 4 + 4096 * 4),
        "rmsnorm_torch_eager": (lambda: x * torch.rsqrt(torch.mean(x * x, dim=-1, keepdim=True) + 1e-6) * w,
                                2.0 * x.numel() * 4 + 4096 * 4),
        "softmax_naive": (lambda: pkg.softmax(logits), 2.0 * logits.numel() * 4),
        "softmax_torch": (lambda: torch.softmax(logits, dim=1), 2.0 * logits.numel() * 4),
    }
    for name, (fn, nbytes) in row_cases.items():
        t = event_time_ms(torch, fn, **({'warmup': 3, 'repeat': 10} if quick else {}))
        results["rows"].append({"case": name, "algorithmic_bytes": nbytes, "gbs_median": nbytes / t["median_ms"] / 1e6,
                                **t})
    return results


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--arm", choices=list(ARMS))
    parser.add_argument("--out")
    parser.add_argument("--quick", action="store_true")
    args = parser.parse_args()
    if args.arm:
        print("RESULT " + json.dumps(run_arm(args.arm, args.quick)))
        return
    merged = {}
    for arm, path in ARMS.items():
        if not (path / "cuda_ai_kernels").is_dir():
            merged[arm] = {"unavailable": f"{path} has no cuda_ai_kernels package"}
            continue
        proc = subprocess.run([sys.executable, __file__, "--arm", arm, *(["--quick"] if args.quick else [])],
                              capture_output=True, text=True)
        line = next((l for l in proc.stdout.splitlines() if l.startswith("RESULT ")), None)
        merged[arm] = json.loads(line[7:]) if line else {"unavailable": (proc.stderr or proc.stdout)[-800:]}
    if args.out:
        Path(args.out).write_text(json.dumps(merged, indent=1))

    def table(section, key, label, value):
        rows = {}
        for arm, data in merged.items():
            for item in data.get(section, []):
                rows.setdefault(key(item), {})[arm] = item[value]
        print(f"\n{label}")
        for k, v in rows.items():
            ours, ref = v.get("ours"), v.get("reference")
            ratio = f"{ours / ref:6.2f}x" if ours and ref else "   n/a"
            print(f"  {str(k):48s} ours {ours or float('nan'):10.2f}   reference {ref or float('nan'):10.2f}   {ratio}")

    table("gemm", lambda i: (tuple(i["shape"]), i["impl"]), "FP32 GEMM, TFLOP/s (median, graph timing)", "tflops_median")
    table("adaptive", lambda i: (i["size"], i["case"]), "TF32 adaptive GEMM, TFLOP/s", "tflops_median")
    table("rows", lambda i: i["case"], "Row operators, GB/s (algorithmic bytes)", "gbs_median")


if __name__ == "__main__":
    main()
