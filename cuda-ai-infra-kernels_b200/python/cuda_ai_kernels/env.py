"""Environment record attached to benchmark output (python/cuda_ai_kernels/env.py:8-18)."""
from __future__ import annotations

import platform

import torch


def collect_env() -> dict[str, str | int | None]:
    has_gpu = torch.cuda.is_available()
    device = torch.cuda.current_device() if has_gpu else None
    return {
        "python": platform.python_version(),
        "platform": platform.platform(),
        "torch": torch.__version__,
        "cuda_runtime": torch.version.cuda,
        "cuda_available": str(has_gpu),
        "gpu": torch.cuda.get_device_name(device) if has_gpu else None,
        "capability": ".".join(str(v) for v in torch.cuda.get_device_capability(device)) if has_gpu else None,
    }
