"""Generates tests/golden/reference_vectors.npz by running the reference's OWN
Python code. Run once on a machine that has the reference checkout; the output
is committed and is what pins oracle/oracle.py.

    python tests/golden/make_golden.py /path/to/cuda-ai-infra-kernels

What is executed from the reference:
  * python/cuda_ai_kernels/testing.py: ``rmsnorm_reference`` (imported),
  * the oracle expressions of its test-suite, evaluated verbatim on the inputs
    its tests build: ``(a.double() @ b.double()).float()`` (tests/test_gemm.py:79),
    ``torch.relu(alpha * (a @ b) + beta * c)`` (tests/test_adaptive_gemm.py:221-224),
    ``(x / torch.sqrt(mean(x*x) + eps)) * weight`` (tests/test_rmsnorm.py:19-21),
    ``torch.softmax(x, dim=1)`` (tests/test_softmax.py:17),
  * the closed-form exact cases of its tests (k*row*col, sum 1..k, sum k^2,
    per-tile constants, the ReLU-after-alpha/beta vector).
Inputs are stored next to the outputs so that the check does not depend on the
random generator staying stable across PyTorch versions.
"""
import sys
from pathlib import Path

import numpy as np
import torch


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "python"))
    from cuda_ai_kernels.testing import rmsnorm_reference  # the reference's module

    out = {}
    torch.set_num_threads(1)

    # FP32 ladder: seed 7, A = randn(k, m).t() (tests/test_gemm.py:75-79).
    for tag, (m, n, k) in {"gemm_a": (32, 48, 24), "gemm_b": (16, 16, 64)}.items():
        torch.manual_seed(7)
        a = torch.randn(k, m).t()
        b = torch.randn(k, n)
        out[f"{tag}_a_storage"] = a.t().contiguous().numpy()
        out[f"{tag}_b"] = b.numpy()
        out[f"{tag}_expected"] = (a.double() @ b.double()).float().numpy()

    # Adaptive epilogue: seed 0 (tests/test_adaptive_gemm.py:207-224), FP64 here.
    torch.manual_seed(0)
    m, n, k = 33, 65, 17
    a, b, c = torch.randn(m, k), torch.randn(k, n), torch.randn(m, n)
    out["adaptive_a"], out["adaptive_b"], out["adaptive_c"] = a.numpy(), b.numpy(), c.numpy()
    for tag, (alpha, beta) in {"p75_p25": (0.75, 0.25), "m50_1": (-0.5, 1.0), "1_p5": (1.0, 0.5)}.items():
        expected = alpha * (a.double() @ b.double()) + beta * c.double()
        out[f"adaptive_linear_{tag}"] = expected.float().numpy()
        out[f"adaptive_relu_{tag}"] = torch.relu(expected).float().numpy()
    # Exact ReLU-after-alpha/beta vector (tests/test_adaptive_gemm.py:239-244).
    eye = torch.eye(4)
    b4 = torch.tensor([[-2.0, -1.0, 1.0, 2.0]]).repeat(4, 1)
    c4 = torch.tensor([[-2.0, -2.0, 2.0, 2.0]]).repeat(4, 1)
    out["adaptive_exact_expected"] = torch.relu(-1.0 * (eye @ b4) + 1.0 * c4).numpy()

    # RMSNorm: seed 0, weight ~ N(0,1), eps 1e-8 (tests/test_rmsnorm.py:10-21).
    torch.manual_seed(0)
    x = torch.randn(4, 768)
    w = torch.randn(768)
    out["rmsnorm_x"], out["rmsnorm_w"] = x.numpy(), w.numpy()
    out["rmsnorm_module_eps1e-6"] = rmsnorm_reference(x.double(), w.double(), 1e-6).float().numpy()
    mean_square = torch.mean(x.double() * x.double(), dim=1, keepdim=True)
    out["rmsnorm_inline_eps1e-8"] = ((x.double() / torch.sqrt(mean_square + 1e-8)) * w.double()).float().numpy()

    # Softmax: seed 0 (tests/test_softmax.py:9-17).
    torch.manual_seed(0)
    x = torch.randn(4, 128)
    out["softmax_x"] = x.numpy()
    out["softmax_expected"] = torch.softmax(x.double(), dim=1).float().numpy()

    # Closed forms used as exact (atol = 0) checks by the reference tests.
    out["closed_k_row_col_shape"] = np.array([256, 384, 24])           # tests/test_gemm.py:56-67
    out["closed_tile_constants_expected"] = np.array([120.0])          # tests/test_gemm_prefetch_smem.py:38-46
    out["closed_sum_k_squares"] = np.array([[k, k * (k + 1) * (2 * k + 1) / 6] for k in (8, 16, 24, 40)])
    out["closed_sum_1_to_k"] = np.array([[k, k * (k + 1) / 2] for k in (16, 32, 48, 64)])

    target = Path(__file__).with_name("reference_vectors.npz")
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
