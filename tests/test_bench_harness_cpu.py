"""The ladder benchmark's protocol, checked on CPU with stand-in operators (as
the reference checks its own harness, tests/test_bench_gemm_all.py): shape
parsing, every stage validated before any timing, a wrong stage blocks the run
and is named, the same tensor objects reach every stage."""
import argparse
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

from conftest import PACKAGE


@pytest.fixture()
def harness(monkeypatch):
    # The module imports cuda_ai_kernels.gemm at import time; that needs the
    # native module, which loads fine without a GPU.
    spec = importlib.util.spec_from_file_location("bench_gemm_all_under_test", PACKAGE / "benchmarks" / "bench_gemm_all.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    monkeypatch.setattr(module, "make_inputs", lambda m, n, k, device="cpu": (torch.randn(k, m).t(), torch.randn(k, n)))
    monkeypatch.setattr(module, "fma_peak_tflops", lambda device=None: 74.45)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    return module


def args(**over):
    base = dict(impls="", profile=False, timing="graph", warmup=1, repeat=2)
    base.update(over)
    return argparse.Namespace(**base)


def fake_timer(log):
    def timer(fn, warmup, repeat):
        fn()
        log.append("timed")
        return {"mean_ms": 2.0, "p50_ms": 1.0, "min_ms": 0.5, "max_ms": 3.0}
    return timer


def test_parse_shapes(harness):
    assert harness.parse_shapes("128x256x64, 4096X4096x4096") == [(128, 256, 64), (4096, 4096, 4096)]
    for bad in ("128x256", "ax1x1", "0x1x1", "1x-2x3"):
        with pytest.raises(argparse.ArgumentTypeError):
            harness.parse_shapes(bad)


def test_all_stages_are_validated_before_any_is_timed_and_share_inputs(harness):
    log, seen = [], []

    def run(a, b, impl):
        log.append(impl)
        seen.append((a, b))
        return (a.double() @ b.double()).float()

    out = harness.benchmark_shape(128, 128, 16, args(), run=run, timer=fake_timer(log))
    impls = [r["impl"] for r in out["results"]]
    assert len(impls) == 14 and impls[0] == "naive" and impls[-1] == "cublas"
    first_timed = log.index("timed")
    assert log[:first_timed - 1] == impls          # phase 1: one validation call per stage, ladder order
    assert log.count("timed") == 14
    assert all(a is seen[0][0] and b is seen[0][1] for a, b in seen)
    for r in out["results"]:
        assert r["correct"] and r["tflops"] == pytest.approx(2 * 128 * 128 * 16 / 1.0 / 1e9)
        assert r["speedup_over_cublas"] == 1.0 and r["speedup_over_naive"] == 1.0
        assert r["roofline"]["bound"] == "fp32_fma" and 0 < r["roofline"]["frac"] < 1
    assert out["a_stride"] == [1, 128] and out["skipped"] == []


def test_a_wrong_stage_blocks_timing_and_is_named(harness):
    log = []

    def run(a, b, impl):
        out = (a.double() @ b.double()).float()
        return out + 1 if impl == "warp_tile" else out

    with pytest.raises(RuntimeError, match=r"stage 5 \(warp_tile\) failed validation at 128x128x16"):
        harness.benchmark_shape(128, 128, 16, args(), run=run, timer=fake_timer(log))
    assert log == []


def test_shapes_that_do_not_fit_a_stage_are_skipped_not_failed(harness):
    out = harness.benchmark_shape(32, 32, 8, args(), run=lambda a, b, impl: (a.double() @ b.double()).float(),
                                  timer=fake_timer([]))
    ran = {r["impl"] for r in out["results"]}
    assert "block_tile_float4_32x32" in ran and "naive" in ran and "cublas" in ran
    assert "prefetch_reg" in out["skipped"] and "split_k" in out["skipped"]


def test_impl_filter_and_profile_mode(harness):
    calls = []
    out = harness.benchmark_shape(128, 128, 16, args(impls="split_k,cublas", profile=True),
                                  run=lambda a, b, impl: calls.append(impl) or (a.double() @ b.double()).float())
    assert calls == ["split_k", "cublas"] and out["validated"] == ["split_k", "cublas"]


def test_cli_refuses_without_a_gpu_or_with_bad_counts(harness):
    with pytest.raises(SystemExit):
        harness.main(["--repeat", "0"])
    if not torch.cuda.is_available():
        with pytest.raises(SystemExit, match="CUDA device"):
            harness.main([])


# --------------------------------------------------- adaptive GEMM benchmark

@pytest.fixture()
def adaptive_harness(monkeypatch):
    spec = importlib.util.spec_from_file_location("bench_adaptive_under_test",
                                                  PACKAGE / "benchmarks" / "bench_adaptive_gemm.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    calls = []

    def fake_adaptive_gemm(a, b, c=None, alpha=1.0, beta=0.0, epilogue="linear", kernel="auto"):
        calls.append({"epilogue": epilogue, "kernel": kernel, "alpha": alpha, "beta": beta})
        out = alpha * (a @ b) + (beta * c if c is not None else 0)
        return out.relu() if epilogue == "relu" else out

    monkeypatch.setattr(module, "adaptive_gemm", fake_adaptive_gemm)
    return module, calls


def test_relu_baseline_is_cublas_plus_a_separate_relu(adaptive_harness):
    module, calls = adaptive_harness
    a, b, c = torch.randn(8, 8), torch.randn(8, 8), torch.randn(8, 8)
    run, fused = module.make_runner("cublas", "relu", a, b, c, 1.0, 0.5)
    out = run()
    assert fused is False and calls[-1] == {"epilogue": "linear", "kernel": "cublas", "alpha": 1.0, "beta": 0.5}
    assert torch.equal(out, (a @ b + 0.5 * c).relu())
    run, fused = module.make_runner("fast_relu", "relu", a, b, c, 1.0, 0.5)
    run()
    assert fused is True and calls[-1]["epilogue"] == "relu" and calls[-1]["kernel"] == "fast_relu"
    run, fused = module.make_runner("cublas", "linear", a, b, None, 2.0, 0.0)
    run()
    assert fused is False and calls[-1] == {"epilogue": "linear", "kernel": "cublas", "alpha": 2.0, "beta": 0.0}


def test_adaptive_check_scales_the_absolute_gate_with_k(adaptive_harness):
    module, _ = adaptive_harness
    expected = torch.randn(16, 16, dtype=torch.float64)
    good = module.check((expected + 1e-4).float(), expected, k=64)
    assert good["passed"] and good["atol"] == pytest.approx(3e-2)
    assert module.check(expected.float(), expected, k=8192)["atol"] == pytest.approx(3e-2 * (128 ** 0.5) / 2)
    bad = module.check((expected * 1.05).float(), expected, k=64)
    assert not bad["passed"] and bad["rel_frobenius"] > 5e-3
    nan = expected.float().clone()
    nan[0, 0] = float("nan")
    assert not module.check(nan, expected, k=64)["passed"]


def test_kernel_lists_cover_the_registry_aliases(adaptive_harness, abi):
    import ctypes

    from conftest import KernelMeta

    module, _ = adaptive_harness
    aliases = {0: set(), 1: set(), 2: set()}
    for i in range(abi.b200_tf32_registry_size()):
        meta = KernelMeta()
        abi.b200_tf32_registry_entry(i, ctypes.byref(meta))
        aliases[meta.epilogue].add(meta.alias.decode())
    assert aliases[0] <= set(module.LINEAR_KERNELS) and aliases[1] <= set(module.RELU_KERNELS)
    assert aliases[2] <= set(module.GELU_KERNELS)
