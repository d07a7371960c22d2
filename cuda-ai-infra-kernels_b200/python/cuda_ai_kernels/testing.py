"""Comparison helpers used by tests and benchmarks.

``rmsnorm_reference`` and ``assert_close`` have the signatures of
python/cuda_ai_kernels/testing.py:9-19 in the reference.
"""
import torch


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is required for this project")


def assert_close(name: str, actual: torch.Tensor, expected: torch.Tensor, atol: float = 1e-4,
                 rtol: float = 1e-4) -> None:
    torch.testing.assert_close(actual, expected, atol=atol, rtol=rtol)
    diff = (actual - expected).abs()
    max_abs = diff.max().item() if diff.numel() else 0.0
    max_rel = (diff / expected.abs().clamp_min(1e-12)).max().item() if diff.numel() else 0.0
    print(f"{name}: max_abs_error={max_abs:.6e}, max_rel_error={max_rel:.6e}")


def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    scale = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * scale * weight
