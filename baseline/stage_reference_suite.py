"""Stages the upstream project's own test-suite next to its rebuilt extension.

    python baseline/stage_reference_suite.py --reference /path/to/cuda-ai-infra-kernels

Copies the upstream checkout's ``tests/`` and ``benchmarks/`` (three of its test
files load benchmark scripts by path) into ``baseline/_ref/suite/``. That folder
is ignored by git - the upstream files are not part of this repository - and
``tests/test_reference_suite_gpu.py`` runs them, unchanged, against this
repository's ``cuda_ai_kernels`` package when the folder is present.

The upstream extension rebuilt for sm_100 lives beside it in
``baseline/_ref/cuda_ai_kernels`` and was produced from a scratch copy of the
checkout (its source tree is read-only and ``third_party/cutlass`` is an empty
submodule there):

    cp -r <checkout> /tmp/refbuild && rmdir /tmp/refbuild/third_party/cutlass
    ln -s <site-packages>/flashinfer/data/cutlass /tmp/refbuild/third_party/cutlass
    cd /tmp/refbuild && TORCH_CUDA_ARCH_LIST=10.0 MAX_JOBS=8 python setup.py build_ext --inplace
    cp -r /tmp/refbuild/python/cuda_ai_kernels <repo>/baseline/_ref/
"""
from __future__ import annotations

import argparse
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent


def stage(reference: Path, target: Path) -> int:
    count = 0
    for name in ("tests", "benchmarks"):
        src = reference / name
        if not src.is_dir():
            raise SystemExit(f"{src} is missing: not an upstream checkout")
        dst = target / name
        if dst.exists():
            shutil.rmtree(dst)
        shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", ".pytest_cache"))
        count += sum(1 for p in dst.rglob("*") if p.is_file())
    return count


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--reference", type=Path, required=True, help="upstream checkout")
    parser.add_argument("--target", type=Path, default=HERE / "_ref" / "suite")
    args = parser.parse_args()
    args.target.mkdir(parents=True, exist_ok=True)
    print(f"staged {stage(args.reference, args.target)} files under {args.target}")
