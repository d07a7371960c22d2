"""Full FP32 GEMM ladder benchmark: validate every stage, then time every stage.

    python cuda-ai-infra-kernels_b200/benchmarks/bench_gemm_all.py \
        [--shapes 1024x1024x1024,4096x4096x4096] [--timing graph|event] [--warmup 10] [--repeat 50] \
        [--seed 0] [--impls a,b,...] [--output results/raw/gemm_all.json] [--profile]

Same protocol and JSON layout as the reference's benchmarks/bench_gemm_all.py
(:80-175), with roofline fields added:
  * inputs once per shape: A = randn(k, m).t() (column-major view), B = randn(k, n);
    the very same tensor objects go to every stage;
  * the FP64 product on the same device is the reference; ALL stages must pass
    assert_close(atol = rtol = 1e-3) before ANY stage is timed - a wrong kernel
    blocks the run instead of producing a number;
  * timing: CUDA graph of 10 calls replayed `repeat` times (headline) or plain
    events; mean, median, min and max are reported, TFLOP/s from the median
    (the reference's published table uses the median);
  * per result: stage, impl, tile multiples, max abs error, stats, TFLOP/s,
    speed-up over cuBLAS and over naive, fraction of the FP32 FMA roofline.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "python"))

from cuda_ai_kernels import gemm  # noqa: E402
from cuda_ai_kernels.benchmark import cuda_event_benchmark, cuda_graph_benchmark, now_tag, save_json  # noqa: E402
from cuda_ai_kernels.env import collect_env  # noqa: E402
from cuda_ai_kernels.gemm_stages import GEMM_STAGES  # noqa: E402

ATOL = RTOL = 1e-3
FP32_LANES_PER_SM = 128


def parse_shapes(text: str) -> list[tuple[int, int, int]]:
    """'MxNxK[,MxNxK...]' -> [(m, n, k), ...]; every size a positive integer."""
    shapes = []
    for item in text.split(","):
        parts = item.lower().strip().split("x")
        if len(parts) != 3:
            raise argparse.ArgumentTypeError(f"shape '{item}' is not MxNxK")
        try:
            m, n, k = (int(p) for p in parts)
        except ValueError as exc:
            raise argparse.ArgumentTypeError(f"shape '{item}' has a non-integer size") from exc
        if min(m, n, k) <= 0:
            raise argparse.ArgumentTypeError(f"shape '{item}' must be positive")
        shapes.append((m, n, k))
    return shapes


def make_inputs(m: int, n: int, k: int, device: str = "cuda"):
    a = torch.randn(k, m, device=device, dtype=torch.float32).t()
    b = torch.randn(k, n, device=device, dtype=torch.float32)
    return a, b


def stages_for(m: int, n: int, k: int, only: set[str] | None):
    """Ladder entries whose tile multiples divide the shape (others are listed as skipped)."""
    runnable, skipped = [], []
    for stage, impl, tile in GEMM_STAGES:
        if only and impl not in only:
            continue
        bm, bn, bk = tile
        (runnable if m % bm == 0 and n % bn == 0 and k % bk == 0 else skipped).append((stage, impl, tile))
    return runnable, skipped


def fma_peak_tflops(device=None) -> float:
    props = torch.cuda.get_device_properties(device or torch.cuda.current_device())
    clock_hz = props.clock_rate * 1e3 if hasattr(props, "clock_rate") else 1.965e9
    return 2.0 * FP32_LANES_PER_SM * props.multi_processor_count * clock_hz / 1e12


def benchmark_shape(m: int, n: int, k: int, args, run=gemm, timer=None) -> dict:
    a, b = make_inputs(m, n, k)
    expected = (a.double() @ b.double()).float()
    runnable, skipped = stages_for(m, n, k, set(args.impls.split(",")) if args.impls else None)

    # Phase 1: correctness of every stage, on the same tensor objects.
    errors = {}
    for stage, impl, _ in runnable:
        try:
            actual = run(a, b, impl=impl)
            torch.cuda.synchronize()
            torch.testing.assert_close(actual, expected, atol=ATOL, rtol=RTOL)
        except Exception as exc:  # attribute the failure to the stage and stop before timing anything
            raise RuntimeError(f"stage {stage} ({impl}) failed validation at {m}x{n}x{k}: {exc}") from exc
        errors[impl] = (actual - expected).abs().max().item()
        del actual

    if args.profile:
        return {"m": m, "n": n, "k": k, "validated": [impl for _, impl, _ in runnable]}

    # Phase 2: timing.
    if timer is None:
        timer = cuda_graph_benchmark if args.timing == "graph" else cuda_event_benchmark
    flops = 2.0 * m * n * k
    peak = fma_peak_tflops()
    results = []
    for stage, impl, tile in runnable:
        stats = timer(lambda impl=impl: run(a, b, impl=impl), warmup=args.warmup, repeat=args.repeat)
        tflops = flops / stats["p50_ms"] / 1e9
        results.append({
            "stage": stage, "impl": impl, "tile_multiples": list(tile), "correct": True,
            "max_absolute_error": errors[impl], "stats": stats, "tflops": tflops,
            "tflops_mean": flops / stats["mean_ms"] / 1e9,
            "roofline": {"bound": "fp32_fma", "peak_tflops": peak, "achieved_tflops": tflops, "frac": tflops / peak,
                         "algorithmic_flops": flops},
        })
    by_impl = {r["impl"]: r for r in results}
    for r in results:
        for base in ("cublas", "naive"):
            ref = by_impl.get(base)
            r[f"speedup_over_{base}"] = ref["stats"]["p50_ms"] / r["stats"]["p50_ms"] if ref else None
    return {"m": m, "n": n, "k": k, "a_stride": list(a.stride()), "b_stride": list(b.stride()),
            "results": results, "skipped": [impl for _, impl, _ in skipped]}


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--shapes", type=parse_shapes, default=parse_shapes("1024x1024x1024,1024x4096x4096,4096x4096x4096"))
    parser.add_argument("--timing", choices=["graph", "event"], default="graph")
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--repeat", type=int, default=50)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--impls", default="", help="comma-separated subset of ladder names (default: all)")
    parser.add_argument("--output", default="")
    parser.add_argument("--profile", action="store_true", help="validate only (for use under ncu); nothing is saved")
    return parser


def main(argv=None) -> dict:
    args = build_parser().parse_args(argv)
    if args.warmup < 0 or args.repeat <= 0:
        raise SystemExit("--warmup must be >= 0 and --repeat > 0")
    if not torch.cuda.is_available():
        raise SystemExit("bench_gemm_all.py needs a CUDA device")
    torch.manual_seed(args.seed)
    payload = {
        "kernel": "gemm_all", "dtype": "float32",
        "layout": {"a": "column-major [M,K] (strides 1,M)", "b": "row-major [K,N]", "c": "row-major [M,N]"},
        "cublas_compute": "CUBLAS_COMPUTE_32F_PEDANTIC", "reference": "(a.double() @ b.double()).float() on the device",
        "timing": args.timing,
        "timing_note": "CUDA graph of 10 calls per replay" if args.timing == "graph" else "CUDA events per call",
        "warmup": args.warmup, "repeat": args.repeat, "seed": args.seed,
        "device": torch.cuda.get_device_name(), "env": collect_env(), "shapes": [],
    }
    for m, n, k in args.shapes:
        shape = benchmark_shape(m, n, k, args)
        payload["shapes"].append(shape)
        if args.profile:
            continue
        print(f"\n{m}x{n}x{k}  (median of {args.repeat}, {args.timing} timing)")
        print(f"  {'stage':>5} {'impl':28} {'ms':>9} {'TFLOP/s':>9} {'vs cuBLAS':>10} {'of FMA peak':>12} {'max|err|':>10}")
        for r in shape["results"]:
            vs = r["speedup_over_cublas"]
            print(f"  {r['stage']:>5} {r['impl']:28} {r['stats']['p50_ms']:9.4f} {r['tflops']:9.2f} "
                  f"{(f'{100 * vs:.1f}%' if vs else 'n/a'):>10} {100 * r['roofline']['frac']:11.1f}% "
                  f"{r['max_absolute_error']:10.2e}")
    if not args.profile:
        out = args.output or f"results/raw/gemm_all_{now_tag()}.json"
        save_json(out, payload)
        print(f"\nsaved {out}")
    return payload


if __name__ == "__main__":
    main()
