"""Parity of the RMSNorm and softmax kernels with the CPU oracle, through the
C ABI. Tolerance: max|y - ref| / max|ref| <= 1e-5 (north star) plus the
reference suite's atol = 1e-5; every row-length path is covered (warp, block,
staged through shared memory by the copy engine, cluster / DSMEM, streaming, unaligned)."""
import pytest
import torch

from conftest import current_stream_ptr
from oracle import oracle

pytestmark = pytest.mark.gpu

# (rows, cols): warp path (<= 1024), block path (256 / 512 threads, <= 4096 /
# 8192), rows staged in shared memory (8196 .. 50176), cluster paths (8 CTAs,
# <= 65536 / 262144), streaming path, lengths that are not a multiple of four,
# single row / single column.
SHAPES = [(16, 128), (16, 768), (32, 1024), (33, 516), (8, 2048), (8, 4096), (5, 8192), (7, 8196), (4, 12288), (3, 16384),
          (3, 28672), (3, 28676), (3, 32768), (3, 33000), (300, 20000), (3, 50176), (2, 50180), (2, 65536), (2, 70000), (2, 140000), (1, 262144),
          (1, 300000), (5, 1001), (7, 3), (1, 1), (300, 4), (0, 16)]


def rmsnorm(abi, x, w, eps, impl=0):
    y = torch.full_like(x, float("nan"))
    status = abi.b200_rmsnorm(impl, x.data_ptr(), w.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], eps,
                              current_stream_ptr())
    assert status == 0, abi.b200_status_string(status)
    return y


def softmax(abi, x):
    y = torch.full_like(x, float("nan"))
    status = abi.b200_softmax(0, x.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], current_stream_ptr())
    assert status == 0, abi.b200_status_string(status)
    return y


def check(actual, expected):
    if expected.numel() == 0:
        return
    assert oracle.rel_max(actual, expected) <= oracle.ROWOP_REL
    torch.testing.assert_close(actual.cpu(), expected, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("eps", [1e-6, 1e-8])
def test_rmsnorm_matches_oracle(abi, shape, eps):
    x, w = oracle.rmsnorm_inputs(*shape)
    check(rmsnorm(abi, x.cuda(), w.cuda(), eps), oracle.rmsnorm_fp64(x, w, eps))


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[1] <= 4096])
def test_rmsnorm_cache_x_entry(abi, shape):
    x, w = oracle.rmsnorm_inputs(*shape, seed=1)
    check(rmsnorm(abi, x.cuda(), w.cuda(), 1e-6, impl=1), oracle.rmsnorm_fp64(x, w, 1e-6))


def test_rmsnorm_cache_x_keeps_its_row_length_limit(abi):
    x = torch.zeros(2, 8192, device="cuda")
    w = torch.zeros(8192, device="cuda")
    assert abi.b200_rmsnorm(1, x.data_ptr(), w.data_ptr(), x.data_ptr(), 2, 8192, 1e-6, current_stream_ptr()) == 3


def test_rmsnorm_with_normal_weights_as_in_the_reference_suite(abi):
    torch.manual_seed(0)
    for shape in [(16, 768), (32, 1024), (8, 4096)]:
        x, w = torch.randn(shape), torch.randn(shape[1])
        y = rmsnorm(abi, x.cuda(), w.cuda(), 1e-8)
        assert torch.allclose(y.cpu(), oracle.rmsnorm_fp64(x, w, 1e-8), atol=1e-5)


def test_rmsnorm_unaligned_base_pointer(abi):
    x, w = oracle.rmsnorm_inputs(6, 1024)
    x_dev = torch.empty(6 * 1024 + 1, device="cuda")[1:].view(6, 1024).copy_(x)
    check(rmsnorm(abi, x_dev, w.cuda(), 1e-6), oracle.rmsnorm_fp64(x, w, 1e-6))


@pytest.mark.parametrize("shape", SHAPES)
def test_softmax_matches_oracle(abi, shape):
    x = oracle.softmax_inputs(*shape)
    y = softmax(abi, x.cuda())
    check(y, oracle.softmax_fp64(x))
    if x.numel():
        torch.testing.assert_close(y.sum(dim=1).cpu(), torch.ones(shape[0]), atol=1e-5, rtol=0)


def test_softmax_is_shift_invariant_and_survives_large_logits(abi):
    x = oracle.softmax_inputs(64, 1024)
    base = softmax(abi, x.cuda())
    shifted = softmax(abi, (x + 64.0).cuda())   # exact shift for these magnitudes
    torch.testing.assert_close(shifted, base, atol=1e-6, rtol=1e-5)
    huge = torch.full((4, 2048), 3.0e4, device="cuda")
    huge[:, 7] = 3.0e4 + 20
    y = softmax(abi, huge)
    assert torch.isfinite(y).all() and bool((y[:, 7] > 0.99).all())


def test_baseline_config_rmsnorm_16384x4096(abi):
    x, w = oracle.rmsnorm_inputs(16384, 4096)
    y = rmsnorm(abi, x.cuda(), w.cuda(), 1e-6)
    check(y, oracle.rmsnorm_fp64(x, w, 1e-6))
    # Property: with unit weights every output row has mean square 1 / (1 + eps / ms).
    ones = torch.ones(4096, device="cuda")
    y1 = rmsnorm(abi, x.cuda(), ones, 1e-6)
    torch.testing.assert_close((y1.double() ** 2).mean(dim=1), torch.ones(16384, dtype=torch.float64, device="cuda"),
                               atol=1e-5, rtol=0)


def test_baseline_config_softmax_32768x1024(abi):
    x = oracle.softmax_inputs(32768, 1024)
    y = softmax(abi, x.cuda())
    check(y, oracle.softmax_fp64(x))
    torch.testing.assert_close(y.double().sum(dim=1), torch.ones(32768, dtype=torch.float64, device="cuda"),
                               atol=1e-5, rtol=0)
    assert bool((y > 0).all()) and bool((y <= 1).all())


@pytest.mark.parametrize("shape", [(64, 1024), (16, 4096), (6, 16384), (3, 40000), (9, 1001)])
def test_calls_in_a_row_read_what_the_last_one_wrote(abi, shape):
    # The row kernels are launched under programmatic stream serialization (a kernel is scheduled
    # while the one before it drains and waits for it before its first load): RMSNorm, softmax of
    # its output, RMSNorm of that, with nothing between them in the stream.
    x, w = oracle.rmsnorm_inputs(*shape, seed=3)
    x_dev, w_dev = x.cuda(), w.cuda()
    y = [torch.full_like(x_dev, float("nan")) for _ in range(3)]
    torch.cuda.synchronize()
    stream = current_stream_ptr()
    assert abi.b200_rmsnorm(0, x_dev.data_ptr(), w_dev.data_ptr(), y[0].data_ptr(), shape[0], shape[1], 1e-6, stream) == 0
    assert abi.b200_softmax(0, y[0].data_ptr(), y[1].data_ptr(), shape[0], shape[1], stream) == 0
    assert abi.b200_rmsnorm(0, y[1].data_ptr(), w_dev.data_ptr(), y[2].data_ptr(), shape[0], shape[1], 1e-6, stream) == 0
    step1 = oracle.rmsnorm_fp64(x, w, 1e-6)
    check(y[0], step1)
    step2 = oracle.softmax_fp64(y[0].cpu())
    check(y[1], step2)
    check(y[2], oracle.rmsnorm_fp64(y[1].cpu(), w, 1e-6))
