"""Runs the three operator benchmarks over the YAML shape lists in shapes/.

    python cuda-ai-infra-kernels_b200/benchmarks/run_all.py [--out-dir results/raw]

Counterpart of the reference's benchmarks/run_all.py (:25-66): one JSON file per
operator family, named with a time tag.
"""
from __future__ import annotations

import argparse
from pathlib import Path

import yaml

import bench_adaptive_gemm
import bench_gemm_all
import bench_rowops
from cuda_ai_kernels.benchmark import now_tag

SHAPES = Path(__file__).resolve().parent / "shapes"


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--out-dir", default="results/raw")
    args = parser.parse_args(argv)
    tag = now_tag()
    out = Path(args.out_dir)

    gemm = yaml.safe_load((SHAPES / "gemm.yaml").read_text())
    shapes = ",".join(f"{s['m']}x{s['n']}x{s['k']}" for s in gemm["shapes"])
    bench_gemm_all.main(["--shapes", shapes, "--output", str(out / f"gemm_all_{tag}.json")])

    adaptive = yaml.safe_load((SHAPES / "adaptive_gemm.yaml").read_text())
    bench_adaptive_gemm.main(["--sizes", ",".join(str(s) for s in adaptive["sizes"]), "--epilogue", adaptive["epilogue"],
                              "--alpha", str(adaptive["alpha"]), "--beta", str(adaptive["beta"]),
                              "--output", str(out / f"adaptive_gemm_{tag}.json")])

    rows = yaml.safe_load((SHAPES / "rowops.yaml").read_text())
    bench_rowops.main(["--rmsnorm-shapes", ",".join(rows["rmsnorm"]), "--softmax-shapes", ",".join(rows["softmax"]),
                       "--output", str(out / f"rowops_{tag}.json")])


if __name__ == "__main__":
    main()
