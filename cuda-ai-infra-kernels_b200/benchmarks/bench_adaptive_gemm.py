"""TF32 adaptive GEMM benchmark: registry kernels vs the cuBLAS baseline.

    python cuda-ai-infra-kernels_b200/benchmarks/bench_adaptive_gemm.py \
        [--sizes 1024,4096,8192 | --shape MxNxK[,MxNxK...]] [--kernel all|auto|fast|...[,...]] [--epilogue linear|relu] \
        [--alpha 1.0] [--beta 0.5] [--timing graph|event] [--warmup 10] [--repeat 50] [--idle SECONDS] [--output FILE] [--profile]

Follows the reference's benchmarks/bench_adaptive_gemm.py: each kernel is
checked first (here against the FP64 result computed on the device: relative
Frobenius error <= 5e-3, plus the reference's atol = rtol = 3e-2 scaled by
sqrt(K) for long reductions), then timed. With `--epilogue relu` the cuBLAS
baseline is cuBLAS + a separate `torch.relu_` (`fused_relu: false`), as in the
reference (:14-54); `cublaslt` is cuBLASLt with the ReLU (and bias) fused into its
epilogue, the fair competitor of the fused kernels. `--kernel auto,cublaslt` with a list of shapes
gives the sweep of automatic dispatch against the library; `--idle 0.6` lets the GPU idle before each
timed kernel, so that a short problem is not timed at the clock the power cap left behind after a
long one (about 1400 MHz, which slows the kernels here by up to a third and cuBLASLt's by less). `--profile` runs one NVTX-ranged call per kernel and saves
nothing. Throughput = 2*M*N*K / median time; the tensor roofline uses half the
measured BF16 peak of MEASURED_PEAKS.json when that file is present.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "python"))

from cuda_ai_kernels import adaptive_gemm  # noqa: E402
from cuda_ai_kernels.benchmark import cuda_event_benchmark, cuda_graph_benchmark, now_tag, save_json  # noqa: E402
from cuda_ai_kernels.env import collect_env  # noqa: E402

# "skinny*" runs only M <= 16 and is reported as skipped elsewhere.
LINEAR_KERNELS = ["auto", "skinny", "swap", "splitk", "pair_splitk", "pair_mid", "pair", "width32", "width96", "width160", "medium", "width224", "wide", "narrow", "fast", "fallback", "fast_mwarp", "fallback_mwarp",
                  "fast_stage3", "fast_stage2", "cublas", "cublaslt"]
RELU_KERNELS = ["auto", "skinny_relu", "swap_relu", "splitk_relu", "pair_splitk_relu", "pair_mid_relu", "pair_relu", "width32_relu", "width96_relu", "width160_relu", "medium_relu", "width224_relu", "wide_relu", "narrow_relu", "fast_relu", "fallback_relu", "cublas",
                "cublaslt"]
GELU_KERNELS = ["auto", "skinny_gelu", "swap_gelu", "splitk_gelu", "pair_splitk_gelu", "pair_mid_gelu", "pair_gelu", "width32_gelu", "width96_gelu", "width160_gelu", "medium_gelu", "width224_gelu", "wide_gelu", "narrow_gelu", "fast_gelu", "fallback_gelu"]
REL_FROBENIUS = 5e-3


def tf32_peak_tflops() -> tuple[float, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text())["bf16_tflops"] / 2.0, "measured BF16 burst / 2"
    return 1100.0, "nominal dense TF32"


def make_runner(kernel: str, epilogue: str, a, b, c, alpha: float, beta: float):
    """Callable for one benchmark arm and whether its ReLU is fused."""
    if kernel == "cublas" and epilogue == "relu":
        # The library baseline has no fused activation: GEMM, then an in-place ReLU.
        return (lambda: torch.relu_(adaptive_gemm(a, b, c=c, alpha=alpha, beta=beta, kernel="cublas"))), False
    return (lambda: adaptive_gemm(a, b, c=c, alpha=alpha, beta=beta, epilogue=epilogue, kernel=kernel)), epilogue == "relu"


def check(actual, expected, k: int) -> dict:
    diff = (actual.double() - expected).abs()
    rel_frob = float((actual.double() - expected).norm() / expected.norm())
    atol = 3e-2 * max(1.0, (k / 64) ** 0.5 / 2)
    ok = rel_frob <= REL_FROBENIUS and bool((diff <= atol + 3e-2 * expected.abs()).all()) and bool(torch.isfinite(actual).all())
    return {"reference": "FP64 on device", "rel_frobenius": rel_frob, "atol": atol, "rtol": 3e-2,
            "max_absolute_error": float(diff.max()), "passed": ok}


def benchmark_problem(m: int, n: int, k: int, args) -> dict:
    a = torch.randn(m, k, device="cuda")
    b = torch.randn(k, n, device="cuda")
    c = torch.randn(m, n, device="cuda") if args.beta != 0 else None
    expected = args.alpha * (a.double() @ b.double())
    if c is not None:
        expected = expected + args.beta * c.double()
    if args.epilogue == "relu":
        expected = expected.relu()
    elif args.epilogue == "gelu":
        expected = torch.nn.functional.gelu(expected)
    by_epilogue = {"linear": LINEAR_KERNELS, "relu": RELU_KERNELS, "gelu": GELU_KERNELS}
    names = by_epilogue[args.epilogue] if args.kernel == "all" else args.kernel.split(",")
    timer = cuda_graph_benchmark if args.timing == "graph" else cuda_event_benchmark
    peak, peak_source = tf32_peak_tflops()
    flops = 2.0 * m * n * k
    rows = []
    for name in names:
        run, fused = make_runner(name, args.epilogue, a, b, c, args.alpha, args.beta)
        try:
            out = run()
        except RuntimeError as exc:  # a forced kernel that cannot run this problem is reported, not fatal
            rows.append({"kernel": name, "skipped": str(exc).splitlines()[0]})
            continue
        from cuda_ai_kernels import _C

        chosen = _C.adaptive_gemm_last_kernel()
        correctness = check(out, expected, k)
        if not correctness["passed"]:
            raise RuntimeError(f"{name} ({chosen}) failed validation at {m}x{n}x{k}: {correctness}")
        if args.profile:
            torch.cuda.nvtx.range_push("adaptive_gemm_profile")
            run()
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
            rows.append({"kernel": name, "registry_name": chosen, "correctness": correctness})
            continue
        if args.idle > 0:
            torch.cuda.synchronize()
            time.sleep(args.idle)
        stats = timer(run, warmup=args.warmup, repeat=args.repeat)
        rows.append({"kernel": name, "registry_name": chosen, "fused_relu": fused, "correctness": correctness,
                     "stats": stats, "tflops_mean": flops / stats["mean_ms"] / 1e9,
                     "tflops_median": flops / stats["p50_ms"] / 1e9,
                     "tflops_min_latency": flops / stats["min_ms"] / 1e9,
                     "roofline": {"bound": "tensor", "peak_tflops": peak, "peak_source": peak_source,
                                  "frac": flops / stats["p50_ms"] / 1e9 / peak}})
    base = next((r for r in rows if r["kernel"] == "cublas" and "stats" in r), None)
    fused_base = next((r for r in rows if r["kernel"] == "cublaslt" and "stats" in r), None)
    for r in rows:
        if "stats" in r:
            r["speedup_vs_cublas"] = base["stats"]["p50_ms"] / r["stats"]["p50_ms"] if base else None
            r["speedup_vs_cublaslt"] = fused_base["stats"]["p50_ms"] / r["stats"]["p50_ms"] if fused_base else None
    return {"m": m, "n": n, "k": k, "alpha": args.alpha, "beta": args.beta, "epilogue": args.epilogue, "results": rows}


def main(argv=None) -> dict:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--sizes", default="1024,4096,8192")
    parser.add_argument("--shape", default="")
    parser.add_argument("--kernel", default="all")
    parser.add_argument("--epilogue", choices=["linear", "relu", "gelu"], default="relu")
    parser.add_argument("--alpha", type=float, default=1.0)
    parser.add_argument("--beta", type=float, default=0.5)
    parser.add_argument("--timing", choices=["graph", "event"], default="graph")
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--repeat", type=int, default=50)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--idle", type=float, default=0.0)
    parser.add_argument("--output", default="")
    parser.add_argument("--profile", action="store_true")
    args = parser.parse_args(argv)
    if args.kernel == "cublas" and args.epilogue == "relu" and args.profile:
        parser.error("--profile with the unfused cuBLAS + ReLU baseline would capture two kernels; pick a fused kernel")
    if not torch.cuda.is_available():
        raise SystemExit("bench_adaptive_gemm.py needs a CUDA device")
    torch.manual_seed(args.seed)
    if args.shape:
        problems = [tuple(int(v) for v in shape.split("x")) for shape in args.shape.lower().split(",")]
    else:
        problems = [(int(s),) * 3 for s in args.sizes.split(",")]
    payload = {"kernel": "adaptive_gemm", "dtype": "float32 in / TF32 multiply / FP32 accumulate", "timing": args.timing,
               "warmup": args.warmup, "repeat": args.repeat, "seed": args.seed, "device": torch.cuda.get_device_name(),
               "env": collect_env(), "problems": []}
    for m, n, k in problems:
        problem = benchmark_problem(m, n, k, args)
        payload["problems"].append(problem)
        if args.profile:
            continue
        print(f"\n{m}x{n}x{k} epilogue={args.epilogue} alpha={args.alpha} beta={args.beta}")
        for r in problem["results"]:
            if "skipped" in r:
                print(f"  {r['kernel']:16} skipped: {r['skipped'][:70]}")
                continue
            vs, vs_lt = r["speedup_vs_cublas"], r["speedup_vs_cublaslt"]
            print(f"  {r['kernel']:16} {r['registry_name']:28} {r['stats']['p50_ms']:9.4f} ms {r['tflops_median']:8.1f} TFLOP/s "
                  f"{100 * r['roofline']['frac']:5.1f}% of peak  vs cuBLAS {(f'{vs:.2f}x' if vs else 'n/a')}  "
                  f"vs cuBLASLt fused {(f'{vs_lt:.2f}x' if vs_lt else 'n/a')}  rel_frob {r['correctness']['rel_frobenius']:.1e}")
    if not args.profile:
        out = args.output or f"results/raw/adaptive_gemm_{now_tag()}.json"
        save_json(out, payload)
        print(f"\nsaved {out}")
    return payload


if __name__ == "__main__":
    main()
