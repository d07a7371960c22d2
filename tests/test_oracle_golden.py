"""Pins oracle/oracle.py against vectors produced by the reference's own Python
code (tests/golden/make_golden.py). CPU only."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle

GOLDEN = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")


def t(name):
    return torch.from_numpy(GOLDEN[name])


@pytest.mark.parametrize("tag", ["gemm_a", "gemm_b"])
def test_gemm_oracle_matches_reference_expression(tag):
    a = t(f"{tag}_a_storage").t()  # column-major view, as the ladder receives it
    b = t(f"{tag}_b")
    assert a.stride(0) == 1
    torch.testing.assert_close(oracle.gemm_fp64(a, b), t(f"{tag}_expected"), atol=0, rtol=0)


@pytest.mark.parametrize("tag,alpha,beta", [("p75_p25", 0.75, 0.25), ("m50_1", -0.5, 1.0), ("1_p5", 1.0, 0.5)])
@pytest.mark.parametrize("epilogue", ["linear", "relu"])
def test_adaptive_oracle_matches_reference_expression(tag, alpha, beta, epilogue):
    actual = oracle.adaptive_gemm_fp64(t("adaptive_a"), t("adaptive_b"), t("adaptive_c"), alpha, beta, epilogue)
    torch.testing.assert_close(actual, t(f"adaptive_{epilogue}_{tag}"), atol=0, rtol=0)


def test_adaptive_oracle_exact_relu_after_scaling():
    eye = torch.eye(4)
    b = torch.tensor([[-2.0, -1.0, 1.0, 2.0]]).repeat(4, 1)
    c = torch.tensor([[-2.0, -2.0, 2.0, 2.0]]).repeat(4, 1)
    actual = oracle.adaptive_gemm_fp64(eye, b, c, alpha=-1.0, beta=1.0, epilogue="relu")
    torch.testing.assert_close(actual, t("adaptive_exact_expected"), atol=0, rtol=0)


def test_adaptive_oracle_ignores_nan_source_when_beta_is_zero():
    eye = torch.eye(4)
    b = torch.tensor([[-2.0, -1.0, 1.0, 2.0]]).repeat(4, 1)
    nan_c = torch.full((4, 4), float("nan"))
    actual = oracle.adaptive_gemm_fp64(eye, b, nan_c, beta=0.0, epilogue="relu")
    torch.testing.assert_close(actual, b.relu(), atol=0, rtol=0)


def test_adaptive_oracle_bias_and_gelu_agree_with_torch_functional():
    # No reference vectors exist for these epilogues (the reference refuses them);
    # the oracle is cross-checked against PyTorch's own FP64 GELU instead.
    a, b, c = t("adaptive_a"), t("adaptive_b"), t("adaptive_c")
    bias = torch.linspace(-1, 1, b.shape[1])
    z = 0.75 * (a.double() @ b.double()) + 0.25 * c.double()
    torch.testing.assert_close(oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, "gelu"),
                               torch.nn.functional.gelu(z).float(), atol=0, rtol=1e-6)
    zb = z + bias.double()
    torch.testing.assert_close(oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, "bias", bias), zb.float(), atol=0, rtol=0)
    torch.testing.assert_close(oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, "bias_relu", bias), zb.relu().float(),
                               atol=0, rtol=0)
    torch.testing.assert_close(oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, "bias_gelu", bias),
                               torch.nn.functional.gelu(zb).float(), atol=0, rtol=1e-6)
    with pytest.raises(ValueError):
        oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.0, "bias")           # bias epilogue without a bias
    with pytest.raises(ValueError):
        oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.0, "relu", bias)     # bias without a bias epilogue


def test_rmsnorm_oracle_matches_reference_module_and_inline_form():
    x, w = t("rmsnorm_x"), t("rmsnorm_w")
    # Both forms are the same value up to the last FP64 bit; after the cast to
    # FP32 at most one ulp of the result can differ.
    torch.testing.assert_close(oracle.rmsnorm_fp64(x, w, 1e-6), t("rmsnorm_module_eps1e-6"), atol=0, rtol=0)
    torch.testing.assert_close(oracle.rmsnorm_fp64(x, w, 1e-8), t("rmsnorm_inline_eps1e-8"), atol=0, rtol=2e-7)


def test_softmax_oracle_matches_torch_softmax():
    torch.testing.assert_close(oracle.softmax_fp64(t("softmax_x")), t("softmax_expected"), atol=0, rtol=0)


def test_closed_forms():
    for k, total in GOLDEN["closed_sum_k_squares"]:
        values = torch.arange(1, int(k) + 1, dtype=torch.float32)
        a = values.unsqueeze(0).expand(8, -1)       # every row holds 1..k
        b = values.unsqueeze(1).expand(-1, 8)
        assert torch.all(oracle.gemm_fp64(a, b) == total)
    for k, total in GOLDEN["closed_sum_1_to_k"]:
        values = torch.arange(1, int(k) + 1, dtype=torch.float32)
        a = values.unsqueeze(0).expand(8, -1)
        assert torch.all(oracle.gemm_fp64(a, torch.ones(int(k), 8)) == total)
    m, n, k = (int(v) for v in GOLDEN["closed_k_row_col_shape"])
    rows = torch.arange(1, m + 1, dtype=torch.float32)
    cols = torch.arange(1, n + 1, dtype=torch.float32)
    a = rows.expand(k, m).contiguous().t()
    b = cols.expand(k, n).contiguous()
    torch.testing.assert_close(oracle.gemm_fp64(a, b), k * rows[:, None] * cols[None, :], atol=0, rtol=0)


def test_seeded_workloads_are_reproducible_and_shaped():
    a, b = oracle.ladder_inputs(128, 256, 64)
    assert a.shape == (128, 64) and a.stride() == (1, 128) and b.shape == (64, 256) and b.is_contiguous()
    a2, b2 = oracle.ladder_inputs(128, 256, 64)
    assert torch.equal(a, a2) and torch.equal(b, b2)
    x, w = oracle.rmsnorm_inputs(8, 4096)
    assert 0.5 <= float(w.min()) and float(w.max()) <= 1.5 and x.shape == (8, 4096)
    logits = oracle.softmax_inputs(64, 1024)
    spikes = (logits == 8.0).float().mean().item()
    assert 0.003 < spikes < 0.03
    assert abs(float(logits[logits != 8.0].std()) - 2.0) < 0.1


def test_tolerance_formulas():
    a, b = oracle.ladder_inputs(128, 128, 1024)
    tol = oracle.sgemm_abs_tolerance(a, b)
    assert tol == pytest.approx(1e-4 * 32 * float(a.abs().max()) * float(b.abs().max()))
    ref = torch.ones(4, 4)
    assert oracle.rel_frobenius(ref * 1.001, ref) == pytest.approx(1e-3, rel=1e-3)
    assert oracle.rel_max(ref + 1e-3, ref) == pytest.approx(1e-3, rel=1e-3)
