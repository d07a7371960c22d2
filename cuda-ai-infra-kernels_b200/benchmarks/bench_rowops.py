"""RMSNorm / softmax benchmark against the HBM roofline.

    python cuda-ai-infra-kernels_b200/benchmarks/bench_rowops.py [--op rmsnorm|softmax|both] \
        [--rmsnorm-shapes 16384x4096,...] [--softmax-shapes 32768x1024,...] [--warmup 10] [--repeat 50] [--output FILE]

Counterpart of the reference's benchmarks/bench_rmsnorm.py and bench_softmax.py.
Bandwidth is reported twice: with the ALGORITHMIC bytes (one read of x, one
write of y, plus the weight vector - what a single-pass kernel must move) and
with the reference's convention of three passes over the tensor
(bench_rmsnorm.py:33, bench_softmax.py:30), so that old and new tables can be
compared. Inputs rotate through enough buffers to exceed L2 between calls.
PyTorch eager runs beside each operator.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "python"))

from cuda_ai_kernels import rmsnorm, softmax  # noqa: E402
from cuda_ai_kernels.benchmark import cuda_event_benchmark, now_tag, save_json  # noqa: E402
from cuda_ai_kernels.env import collect_env  # noqa: E402
from cuda_ai_kernels.testing import rmsnorm_reference  # noqa: E402

L2_BYTES = 126e6


def hbm_peak_gbs() -> tuple[float, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text())["hbm_gbs"], "measured copy bandwidth"
    return 8000.0, "nominal HBM3e"


def parse_2d(text: str):
    return [tuple(int(v) for v in item.lower().split("x")) for item in text.split(",") if item]


def rotating(make, nbytes: int):
    """Enough independent inputs that consecutive calls cannot hit in L2."""
    count = max(2, int(2 * L2_BYTES // max(nbytes, 1)) + 1)
    return [make() for _ in range(min(count, 16))]


def bench_one(name, shape, fn_ours, fn_torch, inputs, algorithmic, args, peak, peak_source, check):
    rows, cols = shape
    out = fn_ours(inputs[0])
    ref = check(inputs[0])
    rel = float((out.double() - ref).abs().max() / ref.abs().max())
    if not rel <= 1e-5:
        raise RuntimeError(f"{name} {rows}x{cols} failed validation: relative error {rel:.2e}")
    result = {"op": name, "rows": rows, "cols": cols, "relative_error": rel, "algorithmic_bytes": algorithmic,
              "reference_convention_bytes": 3.0 * rows * cols * 4, "arms": {}}
    for arm, fn in (("ours", fn_ours), ("torch_eager", fn_torch)):
        state = {"i": 0}

        def step():
            state["i"] += 1
            return fn(inputs[state["i"] % len(inputs)])

        stats = cuda_event_benchmark(step, warmup=args.warmup, repeat=args.repeat)
        gbs = algorithmic / stats["p50_ms"] / 1e6
        result["arms"][arm] = {"stats": stats, "gbs_algorithmic": gbs,
                               "gbs_reference_convention": 3.0 * rows * cols * 4 / stats["p50_ms"] / 1e6,
                               "roofline": {"bound": "hbm", "peak_gbs": peak, "peak_source": peak_source,
                                            "frac": gbs / peak}}
    o, t = result["arms"]["ours"], result["arms"]["torch_eager"]
    print(f"  {name:8} {rows}x{cols}: ours {o['gbs_algorithmic']:8.1f} GB/s ({100 * o['roofline']['frac']:.1f}% of {peak_source}), "
          f"torch eager {t['gbs_algorithmic']:8.1f} GB/s, rel err {rel:.1e}")
    return result


def main(argv=None) -> dict:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--op", choices=["rmsnorm", "softmax", "both"], default="both")
    parser.add_argument("--rmsnorm-shapes", default="16384x4096,4096x8192,1024x16384,65536x1024")
    parser.add_argument("--softmax-shapes", default="32768x1024,16384x4096,4096x32768,131072x256")
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--repeat", type=int, default=50)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--output", default="")
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("bench_rowops.py needs a CUDA device")
    torch.manual_seed(args.seed)
    peak, peak_source = hbm_peak_gbs()
    payload = {"kernel": "rowops", "dtype": "float32", "timing": "event", "warmup": args.warmup, "repeat": args.repeat,
               "device": torch.cuda.get_device_name(), "env": collect_env(), "results": []}
    if args.op in ("rmsnorm", "both"):
        for rows, cols in parse_2d(args.rmsnorm_shapes):
            w = torch.rand(cols, device="cuda") + 0.5
            xs = rotating(lambda: torch.randn(rows, cols, device="cuda"), rows * cols * 4)
            payload["results"].append(bench_one(
                "rmsnorm", (rows, cols), lambda x: rmsnorm(x, w, 1e-6), lambda x: rmsnorm_reference(x, w, 1e-6), xs,
                2.0 * rows * cols * 4 + cols * 4, args, peak, peak_source,
                lambda x: rmsnorm_reference(x.double(), w.double(), 1e-6)))
            del xs
    if args.op in ("softmax", "both"):
        for rows, cols in parse_2d(args.softmax_shapes):
            xs = rotating(lambda: 2 * torch.randn(rows, cols, device="cuda"), rows * cols * 4)
            payload["results"].append(bench_one(
                "softmax", (rows, cols), softmax, lambda x: torch.softmax(x, dim=1), xs, 2.0 * rows * cols * 4, args,
                peak, peak_source, lambda x: torch.softmax(x.double(), dim=1)))
            del xs
    out = args.output or f"results/raw/rowops_{now_tag()}.json"
    save_json(out, payload)
    print(f"saved {out}")
    return payload


if __name__ == "__main__":
    main()
