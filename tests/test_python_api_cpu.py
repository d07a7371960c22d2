"""Python operator wrappers exercised on CPU against a stub native module:
name tables, error types, and the rule that ladder GEMMs hand the caller's very
tensors to the native layer (no copy, no transpose, no fallback)."""
import importlib
import sys
import types

import pytest
import torch


@pytest.fixture()
def stub_ops(monkeypatch):
    calls = []

    def recorder(name):
        def fn(*args):
            calls.append((name, args))
            return name
        return fn

    names = ["gemm_cublas", "gemm_naive", "gemm_block_tile", "gemm_thread_tile", "gemm_block_tile_float4_16x16",
             "gemm_block_tile_float4_16x32", "gemm_block_tile_float4_32x32", "gemm_thread_tile_4x4",
             "gemm_thread_tile_4x8", "gemm_thread_tile_8x8", "gemm_thread_tile_8x8_warp4x8", "gemm_warp_tile",
             "gemm_tensor_core", "gemm_prefetch_smem", "gemm_prefetch_reg", "gemm_split_k", "gemm_cutlass",
             "rmsnorm_naive", "rmsnorm_cache_x", "softmax_naive", "rope_forward", "attention_decode_forward",
             "adaptive_gemm"]
    stub = types.ModuleType("cuda_ai_kernels._C")
    for name in names:
        setattr(stub, name, recorder(name))
    import cuda_ai_kernels

    monkeypatch.setitem(sys.modules, "cuda_ai_kernels._C", stub)
    monkeypatch.setattr(cuda_ai_kernels, "_C", stub, raising=False)
    sys.modules.pop("cuda_ai_kernels.ops", None)
    ops = importlib.import_module("cuda_ai_kernels.ops")
    yield ops, calls
    sys.modules.pop("cuda_ai_kernels.ops", None)


def test_package_exports_the_reference_surface():
    import cuda_ai_kernels

    assert cuda_ai_kernels.__all__ == ["adaptive_gemm", "attention_decode", "gemm", "rmsnorm", "rope", "softmax"]
    with pytest.raises(AttributeError):
        cuda_ai_kernels.not_an_operator


def test_stage_table():
    from cuda_ai_kernels.gemm_stages import COLUMN_MAJOR_IMPLS, GEMM_STAGE_IMPLS, GEMM_STAGES

    assert len(GEMM_STAGES) == 14 and GEMM_STAGE_IMPLS[0] == "naive" and GEMM_STAGE_IMPLS[-1] == "cublas"
    assert [s for s, _, _ in GEMM_STAGES] == sorted(s for s, _, _ in GEMM_STAGES)
    assert "thread_tile" in COLUMN_MAJOR_IMPLS and "tensor_core" not in COLUMN_MAJOR_IMPLS
    assert dict((n, t) for _, n, t in GEMM_STAGES)["split_k"] == (128, 128, 16)


def test_ladder_impls_receive_the_callers_tensors_untouched(stub_ops):
    ops, calls = stub_ops
    from cuda_ai_kernels.gemm_stages import COLUMN_MAJOR_IMPLS

    a = torch.randn(8, 16).t()            # column-major view, not contiguous
    b = torch.randn(8, 4)
    for impl in sorted(COLUMN_MAJOR_IMPLS):
        calls.clear()
        ops.gemm(a, b, impl=impl)
        (name, args), = calls
        assert args[0] is a and args[1] is b, impl


def test_row_major_side_entries_get_contiguous_copies(stub_ops):
    ops, calls = stub_ops
    a = torch.randn(8, 16).t()
    b = torch.randn(8, 4)
    for impl in ("tensor_core", "cutlass"):
        calls.clear()
        ops.gemm(a, b, impl=impl)
        (name, args), = calls
        assert args[0] is not a and args[0].is_contiguous() and torch.equal(args[0], a)


def test_every_gemm_name_routes_to_its_native_function(stub_ops):
    ops, _ = stub_ops
    a, b = torch.zeros(4, 4), torch.zeros(4, 4)
    expected = {"thread_tile": "gemm_thread_tile", "tensor_core": "gemm_tensor_core", "cutlass": "gemm_cutlass",
                "prefetch_smem": "gemm_prefetch_smem", "prefetch_reg": "gemm_prefetch_reg",
                "split_k": "gemm_split_k", "cublas": "gemm_cublas"}
    for impl in ops._GEMM_IMPLS:
        assert ops.gemm(a, b, impl=impl) == expected.get(impl, f"gemm_{impl}")
    assert len(ops._GEMM_IMPLS) == 17


def test_unknown_names_raise_value_error(stub_ops):
    ops, _ = stub_ops
    x = torch.zeros(2, 4)
    with pytest.raises(ValueError, match="unknown GEMM impl: nope"):
        ops.gemm(x, x, impl="nope")
    with pytest.raises(ValueError, match="unknown RMSNorm impl"):
        ops.rmsnorm(x, torch.zeros(4), impl="nope")
    with pytest.raises(ValueError, match="unknown softmax impl"):
        ops.softmax(x, impl="nope")


def test_row_ops_and_adaptive_forward_defaults(stub_ops):
    ops, calls = stub_ops
    x = torch.randn(4, 6)[:, ::2]          # non-contiguous
    w = torch.randn(3)
    ops.rmsnorm(x, w)
    name, args = calls[-1]
    assert name == "rmsnorm_naive" and args[0].is_contiguous() and args[2] == 1e-6
    ops.rmsnorm(x, w, eps=1e-8, impl="cache_x")
    assert calls[-1][0] == "rmsnorm_cache_x" and calls[-1][1][2] == 1e-8
    ops.softmax(x)
    assert calls[-1][0] == "softmax_naive" and calls[-1][1][0].is_contiguous()
    ops.adaptive_gemm(x, x.t())
    name, args = calls[-1]
    assert name == "adaptive_gemm" and args[2] is None and args[3] is None
    assert args[4:] == (1.0, 0.0, "linear", "auto")
    c = torch.randn(4, 4)
    ops.adaptive_gemm(x, x.t(), c=c, alpha=0.5, beta=2.0, epilogue="relu", kernel="fast_relu")
    assert calls[-1][1][2] is c and calls[-1][1][4:] == (0.5, 2.0, "relu", "fast_relu")


def test_native_module_rejects_cpu_tensors_before_touching_a_gpu():
    # The real extension, on a machine without a GPU: argument validation runs
    # first, so the error is about the tensors, not about CUDA being absent.
    from cuda_ai_kernels import _C

    x = torch.zeros(128, 128)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        _C.gemm_prefetch_reg(x.t(), x)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        _C.adaptive_gemm(x, x)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        _C.rmsnorm_naive(x, torch.zeros(128), 1e-6)
    with pytest.raises(RuntimeError, match="2D"):
        _C.gemm_split_k(torch.zeros(2, 2, 2), x)
    with pytest.raises(RuntimeError, match="positive"):
        _C.gemm_prefetch_smem(torch.zeros(0, 128).t(), torch.zeros(0, 128))
