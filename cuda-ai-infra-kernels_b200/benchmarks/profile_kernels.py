"""Launches each hot-path kernel a few times at its benchmark shape, for ncu.

    python cuda-ai-infra-kernels_b200/benchmarks/profile_kernels.py [sgemm] [tf32] [tf32_pair] [rows] [tf32_other] [tf32_mid] [--small]

Meant to be wrapped by Nsight Compute: ONE kernel per capture, two or three
launches, the small case, e.g.

    ncu --set full --clock-control none -k regex:sgemm_pipeline -c 3 -o prof \
        python cuda-ai-infra-kernels_b200/benchmarks/profile_kernels.py sgemm --small

(on a shared GPU a multi-pass capture must end by itself within a minute or two:
anything beyond a plain launch list is taken with `--small`, one `-k` pattern
and `-c 2` or `-c 3`). The role of the reference's profiling/profile_*.sh
wrappers. `--small` halves the GEMM edge (2048: operands 3 x 16 MiB) so that a
multi-pass capture stays short; the row-operator shapes (256 MiB and 128 MiB per
tensor) are already small enough. `tf32` goes through automatic dispatch (CTA pairs at
4096, 128 x 256 tiles at 2048); `tf32_pair` forces the CTA-pair kernel at either size. `tf32_mid` runs the mid-sized shapes where one
round of tiles decides (1536^3 through the 128 x 128 TMA tile kernel,
1024 x 1024 x 8192 through automatic dispatch). `tf32_other`
runs the registry entries for awkward shapes: the warp-specialised loader on
misaligned operands (2047 x 2049 x 2051), the operand-swapped kernel
(16 x 4096 x 4096), the split-K cluster kernel (64 x 4096 x 4096) and the FP32
stream kernel (4 x 4096 x 16384, B = 268 MB).
"""
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "python"))
import cuda_ai_kernels as pkg  # noqa: E402


def main(argv):
    small = "--small" in argv
    which = [a for a in argv if not a.startswith("--")] or ["sgemm", "tf32", "rows"]
    edge = 2048 if small else 4096
    dev = "cuda"
    if "sgemm" in which:
        a = torch.randn(edge, edge, device=dev).t()
        b = torch.randn(edge, edge, device=dev)
        for impl in ("prefetch_reg", "prefetch_reg", "split_k", "prefetch_smem"):
            pkg.gemm(a, b, impl=impl)
    if "tf32" in which:
        a = torch.randn(edge, edge, device=dev)
        b = torch.randn(edge, edge, device=dev)
        c = torch.randn(edge, edge, device=dev)
        for _ in range(2):
            pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, epilogue="relu")
    if "tf32_pair" in which:
        a = torch.randn(edge, edge, device=dev)
        b = torch.randn(edge, edge, device=dev)
        c = torch.randn(edge, edge, device=dev)
        for _ in range(3):
            pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, epilogue="relu", kernel="pair_relu")
    if "tf32_mid" in which:
        a = torch.randn(1536, 1536, device=dev)
        b = torch.randn(1536, 1536, device=dev)
        c = torch.randn(1536, 1536, device=dev)
        for _ in range(3):
            pkg.adaptive_gemm(a, b, c=c, alpha=1.0, beta=0.5, epilogue="relu", kernel="fast_relu")
        a = torch.randn(1024, 8192, device=dev)
        b = torch.randn(8192, 1024, device=dev)
        for _ in range(3):
            pkg.adaptive_gemm(a, b)
    if "tf32_other" in which:
        for (m, n, k) in ((2047, 2049, 2051), (16, 4096, 4096), (64, 4096, 4096), (4, 4096, 16384)):
            a = torch.randn(m, k, device=dev)
            b = torch.randn(k, n, device=dev)
            for _ in range(2):
                pkg.adaptive_gemm(a, b)
    if "rows" in which:
        x = torch.randn(16384, 4096, device=dev)
        w = torch.rand(4096, device=dev) + 0.5
        for _ in range(2):
            pkg.rmsnorm(x, w, 1e-6)
        logits = torch.randn(32768, 1024, device=dev)
        for _ in range(2):
            pkg.softmax(logits)
    torch.cuda.synchronize()
    print("profiled:", " ".join(which))


if __name__ == "__main__":
    main(sys.argv[1:])
