"""Builds the two native artefacts of this package, in tree.

1. ``lib/libb200_kernels.so`` - the torch-free CUDA library behind the C ABI of
   ``include/b200_kernels.h``: every ``csrc/kernels/*.cu`` compiled by nvcc for
   ``sm_100a`` (the ``a`` suffix is required by tcgen05 and the packed FP32
   FMA) and linked with the static CUDA runtime.
2. ``python/cuda_ai_kernels/_C*.so`` - the pybind11 module with the PyTorch
   launchers (``csrc/torch/*.cpp``), compiled by g++ only (no device code) and
   linked against libtorch, cuBLAS and (1).

Both steps cross-compile on a machine without a GPU. Object files are cached in
``build/`` and rebuilt when a source or header is newer.

``--debug-bounds`` additionally builds ``lib/libb200_kernels_debug.so``: the same
sources with ``-DB200_DEBUG_BOUNDS``, in which the kernels' stores and unpredicated
loads are wrapped in index checks that record a bit in the device status word and
skip the access (nothing traps). It stands in for a memory checker on shared GPUs;
``tests/test_debug_bounds_gpu.py`` runs the exact small cases against it.

Usage: ``python build.py [--force] [--kernels-only] [--debug-bounds] [--verbose]``
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
REPO = PKG.parent
KERNEL_DIR = PKG / "csrc" / "kernels"
TORCH_DIR = PKG / "csrc" / "torch"
OBJ_DIR = PKG / "build"
LIB_DIR = PKG / "lib"
KERNEL_LIB = LIB_DIR / "libb200_kernels.so"
DEBUG_LIB = LIB_DIR / "libb200_kernels_debug.so"
PY_PKG = PKG / "python" / "cuda_ai_kernels"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    f"-I{REPO / 'include'}",
]


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths if p.exists()), default=0.0)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(cmd[:4])} ...")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr, flush=True)


def extension_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PY_PKG / f"_C{suffix}"


def build_kernels(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    target = DEBUG_LIB if debug_bounds else KERNEL_LIB
    prefix = "dbg_" if debug_bounds else ""
    extra = ["-DB200_DEBUG_BOUNDS"] if debug_bounds else []
    sources = sorted(KERNEL_DIR.glob("*.cu"))
    headers = list(KERNEL_DIR.glob("*.h")) + list(KERNEL_DIR.glob("*.cuh")) + [REPO / "include" / "b200_kernels.h"]
    header_time = _newest(headers)
    jobs = []
    objects = []
    for src in sources:
        obj = OBJ_DIR / (prefix + src.stem + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            jobs.append([NVCC, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or not target.exists():
        _run([NVCC, "-shared", "-o", str(target), *map(str, objects), "-cudart", "static"], verbose)
    return target


def build_extension(force: bool = False, verbose: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    out = extension_path()
    sources = sorted(TORCH_DIR.glob("*.cpp"))
    headers = list(TORCH_DIR.glob("*.h")) + [REPO / "include" / "b200_kernels.h"]
    header_time = _newest(headers)
    torch_lib = Path(torch.__file__).parent / "lib"
    # cuBLAS and the CUDA runtime must be the copies PyTorch itself loads (pip
    # wheels ship them under site-packages/nvidia); fall back to the toolkit.
    nvidia_root = Path(torch.__file__).parent.parent / "nvidia"
    cublas_dir = nvidia_root / "cublas" / "lib"
    cudart_dir = nvidia_root / "cuda_runtime" / "lib"
    if not (cublas_dir / "libcublas.so.12").exists():
        cublas_dir = CUDA_HOME / "lib64"
    if not (cudart_dir / "libcudart.so.12").exists():
        cudart_dir = CUDA_HOME / "lib64"
    includes = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], str(CUDA_HOME / "include"),
                str(REPO / "include"), str(TORCH_DIR)]
    cxx_flags = ["-std=c++17", "-O2", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                 f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-Wno-deprecated-declarations"]
    cxx_flags += [f"-isystem{p}" for p in includes]
    OBJ_DIR.mkdir(exist_ok=True)
    jobs, objects = [], []
    for src in sources:
        obj = OBJ_DIR / ("torch_" + src.stem + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            jobs.append(["g++", *cxx_flags, "-c", str(src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or not out.exists() or out.stat().st_mtime < KERNEL_LIB.stat().st_mtime:
        link = ["g++", "-shared", "-o", str(out), *map(str, objects),
                f"-L{LIB_DIR}", "-lb200_kernels", "-Wl,-rpath,$ORIGIN/../../lib",
                f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
                f"-Wl,-rpath,{torch_lib}",
                f"-L{cublas_dir}", "-l:libcublas.so.12", "-l:libcublasLt.so.12", f"-Wl,-rpath,{cublas_dir}",
                f"-L{cudart_dir}", "-l:libcudart.so.12", f"-Wl,-rpath,{cudart_dir}"]
        _run(link, verbose)
    return out


def build_all(force: bool = False, verbose: bool = False, kernels_only: bool = False, debug_bounds: bool = False) -> None:
    build_kernels(force, verbose)
    if debug_bounds:
        build_kernels(force, verbose, debug_bounds=True)
    if not kernels_only:
        build_extension(force, verbose)


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--kernels-only", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--debug-bounds", action="store_true")
    args = parser.parse_args()
    build_all(args.force, args.verbose, args.kernels_only, args.debug_bounds)
    print(f"built {KERNEL_LIB}")
    if not args.kernels_only:
        print(f"built {extension_path()}")
