"""CPU oracle for the GEMM / row-operator hot path. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module: it exists so that tests,
the smoke check and the CPU-baseline leg of the benchmark have an independent
statement of what the GPU kernels must compute. Every function restates, with
PyTorch CPU tensor arithmetic in FP64, the expression the reference project
uses as its own oracle; the citation next to each function is the reference
file and line it follows. The module is pinned against golden vectors that were
produced by running the reference's own Python code (see
``tests/golden/make_golden.py``): parity is pinned, not assumed.

The input generators make the seeded synthetic tensors of the five benchmark
configurations on the CPU, so that the very same bits feed the oracle and the
GPU (CPU and CUDA random streams differ).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

# --------------------------------------------------------------------- oracles


def gemm_fp64(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """FP64 product rounded once to FP32.

    Reference: ``(a.double() @ b.double()).float()`` in tests/test_gemm.py:79,
    tests/test_gemm_split_k.py:27, benchmarks/bench_gemm_all.py:82. Layout does
    not matter to the oracle: a column-major view is just a strided tensor.
    """
    return (a.detach().cpu().double() @ b.detach().cpu().double()).float()


def adaptive_gemm_fp64(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, alpha: float = 1.0,
                       beta: float = 0.0, epilogue: str = "linear", bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(alpha * A @ B + beta * C [+ bias])`` in FP64, cast to FP32.

    Reference: tests/test_adaptive_gemm.py:221-224 (ReLU applied after scaling
    and source add) and benchmarks/bench_adaptive_gemm.py:38-46. alpha and beta
    are rounded to FP32 first because the operator receives them as floats
    (csrc/adaptive_gemm/adaptive_gemm.cu:163-164). With beta == 0 the source is
    not read at all, so a NaN-filled C must not propagate
    (tests/test_adaptive_gemm.py:247-254).

    ``gelu`` and the ``bias*`` epilogues are named by the reference
    (adaptive_gemm.cu:39-59) but refused by it at run time, so it holds no
    expression or vector for them. They are stated here with the meaning of the
    CUTLASS functors its kernel_config.h:41-46 aliases: the bias is a length-N
    vector added to every row before the activation, GELU is the exact
    erf-based form ``0.5 z (1 + erf(z / sqrt 2))``.
    """
    kinds = {"linear": ("linear", False), "relu": ("relu", False), "gelu": ("gelu", False),
             "bias": ("linear", True), "bias_relu": ("relu", True), "bias_gelu": ("gelu", True)}
    if epilogue not in kinds:
        raise ValueError(f"unsupported epilogue: {epilogue}")
    activation, wants_bias = kinds[epilogue]
    if wants_bias != (bias is not None):
        raise ValueError("bias tensor and epilogue do not agree")
    alpha32 = float(torch.tensor(alpha, dtype=torch.float32))
    beta32 = float(torch.tensor(beta, dtype=torch.float32))
    out = alpha32 * (a.detach().cpu().double() @ b.detach().cpu().double())
    if beta32 != 0.0:
        if c is None:
            raise ValueError("C is required when beta is non-zero")
        out = out + beta32 * c.detach().cpu().double()
    if bias is not None:
        out = out + bias.detach().cpu().double()[None, :]
    if activation == "relu":
        out = torch.relu(out)
    elif activation == "gelu":
        out = 0.5 * out * (1.0 + torch.erf(out / math.sqrt(2.0)))
    return out.float()


def rmsnorm_fp64(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x*x, -1) + eps) * weight`` in FP64, cast to FP32.

    Reference: python/cuda_ai_kernels/testing.py:17-19 (``rmsnorm_reference``);
    tests/test_rmsnorm.py:19-21 states the same value as ``(x / sqrt(.)) * w``.
    """
    x64 = x.detach().cpu().double()
    w64 = weight.detach().cpu().double()
    inv_rms = torch.rsqrt(torch.mean(x64 * x64, dim=-1, keepdim=True) + eps)
    return (x64 * inv_rms * w64).float()


def softmax_fp64(x: torch.Tensor) -> torch.Tensor:
    """Softmax over the last dimension in FP64, cast to FP32.

    Reference: ``torch.softmax(x, dim=1)`` in tests/test_softmax.py:17 and
    benchmarks/bench_softmax.py:25-26.
    """
    return torch.softmax(x.detach().cpu().double(), dim=-1).float()


# ------------------------------------------------------------------ tolerances


def sgemm_abs_tolerance(a: torch.Tensor, b: torch.Tensor) -> float:
    """FP32 SIMT bound: max|C - ref| <= 1e-4 * sqrt(K) * max|A| * max|B|."""
    k = a.shape[1]
    return 1e-4 * math.sqrt(k) * float(a.abs().max()) * float(b.abs().max())


TF32_REL_FROBENIUS = 5e-3  # ||D - ref||_F / ||ref||_F for the TF32 path
ROWOP_REL = 1e-5           # max|y - ref| / max|ref| for RMSNorm and softmax


def rel_frobenius(actual: torch.Tensor, expected: torch.Tensor) -> float:
    e = expected.detach().cpu().double()
    d = actual.detach().cpu().double() - e
    return float(d.norm() / e.norm().clamp_min(1e-300))


def rel_max(actual: torch.Tensor, expected: torch.Tensor) -> float:
    e = expected.detach().cpu().double()
    d = (actual.detach().cpu().double() - e).abs().max()
    return float(d / e.abs().max().clamp_min(1e-300))


# ------------------------------------------------------------ seeded workloads


def _generator(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def ladder_inputs(m: int, n: int, k: int, seed: int = 0):
    """A as a column-major [M,K] view of N(0,1) storage [K,M], B row-major [K,N].

    Recipe of benchmarks/bench_gemm_all.py:40-43 (``randn(k, m).t()``).
    """
    g = _generator(seed)
    a_storage = torch.randn(k, m, generator=g, dtype=torch.float32)
    b = torch.randn(k, n, generator=g, dtype=torch.float32)
    return a_storage.t(), b


def adaptive_inputs(m: int, n: int, k: int, seed: int = 0):
    """Row-major A [M,K], B [K,N], C [M,N], all N(0,1) float32."""
    g = _generator(seed)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(k, n, generator=g, dtype=torch.float32)
    c = torch.randn(m, n, generator=g, dtype=torch.float32)
    return a, b, c


def rmsnorm_inputs(rows: int, hidden: int, seed: int = 0):
    """x ~ N(0,1), weight ~ U(0.5, 1.5)."""
    g = _generator(seed)
    x = torch.randn(rows, hidden, generator=g, dtype=torch.float32)
    w = torch.rand(hidden, generator=g, dtype=torch.float32) + 0.5
    return x, w


def softmax_inputs(rows: int, cols: int, seed: int = 0):
    """logits ~ N(0, 2^2) with 1% of entries set to +8 to exercise max-subtraction."""
    g = _generator(seed)
    x = 2.0 * torch.randn(rows, cols, generator=g, dtype=torch.float32)
    mask = torch.rand(rows, cols, generator=g) < 0.01
    x[mask] = 8.0
    return x


def to_device_preserving_strides(t: torch.Tensor, device) -> torch.Tensor:
    """Copies a column-major view to the device without changing its strides."""
    if t.dim() == 2 and t.stride(0) == 1 and t.stride(1) == t.size(0) and not t.is_contiguous():
        return t.t().contiguous().to(device).t()
    return t.to(device)
