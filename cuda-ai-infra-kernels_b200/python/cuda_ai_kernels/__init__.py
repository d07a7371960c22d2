"""cuda_ai_kernels - operator API backed by hand-written sm_100a kernels.

The six public operators are the ones the reference package exports
(python/cuda_ai_kernels/__init__.py:1-44). They are resolved lazily so that
importing the package does not load the native module; the first call does, and
fails loudly if the module or the CUDA library behind it is missing - there is
no Python or CPU fallback.
"""

__all__ = [
    "adaptive_gemm",
    "attention_decode",
    "gemm",
    "rmsnorm",
    "rope",
    "softmax",
]


def __getattr__(name):
    # PEP 562: forward the public operator names to ops.py on first use.
    if name in __all__:
        from . import ops

        return getattr(ops, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + __all__)
