"""Parity of the FP32 SIMT GEMM ladder with the CPU oracle, through the C ABI
(ctypes on libb200_kernels.so) and through the Python operator API.

Tolerances: the north-star bound max|C - ref| <= 1e-4 * sqrt(K) * max|A| * max|B|
and the reference suite's own atol = rtol = 1e-3 against the FP64 oracle; exact
(atol = 0) for integer-valued inputs, where any summation order is exact."""
import ctypes

import pytest
import torch

from conftest import assert_device_clean, current_stream_ptr
from oracle import oracle

pytestmark = pytest.mark.gpu

LADDER = ["naive", "block_tile", "block_tile_float4_16x16", "block_tile_float4_16x32", "block_tile_float4_32x32",
          "thread_tile_4x4", "thread_tile_4x8", "thread_tile_8x8", "thread_tile_8x8_warp4x8", "warp_tile",
          "prefetch_smem", "prefetch_reg", "split_k"]
PIPELINE = ["prefetch_smem", "prefetch_reg", "split_k"]
TILE_128 = LADDER[5:]


def abi_sgemm(abi, name, a, b):
    """C[M,N] through b200_sgemm; `a` is a column-major [M,K] view on the GPU."""
    assert a.stride(0) == 1 and b.is_contiguous()
    m, k = a.shape
    n = b.shape[1]
    c = torch.full((m, n), float("nan"), device=a.device)
    impl = abi.b200_sgemm_impl_from_name(name.encode())
    status = abi.b200_sgemm(impl, a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, current_stream_ptr())
    assert status == 0, abi.b200_status_string(status)
    return c


def device_inputs(m, n, k, seed=7):
    a, b = oracle.ladder_inputs(m, n, k, seed)
    return a, b, oracle.to_device_preserving_strides(a, "cuda"), b.cuda()


def check_against_oracle(actual, a_cpu, b_cpu):
    expected = oracle.gemm_fp64(a_cpu, b_cpu)
    tol = oracle.sgemm_abs_tolerance(a_cpu, b_cpu)
    err = (actual.cpu() - expected).abs().max().item()
    assert err <= tol, f"max abs error {err:.3e} exceeds 1e-4*sqrt(K)*max|A|*max|B| = {tol:.3e}"
    torch.testing.assert_close(actual.cpu(), expected, atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("impl", LADDER)
@pytest.mark.parametrize("shape", [(128, 128, 16), (128, 256, 48), (256, 128, 64), (384, 256, 80)])
def test_ladder_matches_oracle(abi, impl, shape):
    a_cpu, b_cpu, a, b = device_inputs(*shape)
    check_against_oracle(abi_sgemm(abi, impl, a, b), a_cpu, b_cpu)
    assert_device_clean(abi)


@pytest.mark.parametrize("impl", LADDER)
def test_minimum_tile_is_exact(abi, impl):
    idx = abi.b200_sgemm_impl_from_name(impl.encode())
    bm, bn, bk, vec = (ctypes.c_int() for _ in range(4))
    abi.b200_sgemm_tile(idx, bm, bn, bk, vec)
    m, n, k = bm.value, bn.value, bk.value
    a_storage = (torch.arange(m * k, dtype=torch.float32).view(k, m) % 7).cuda()
    b = (torch.arange(k * n, dtype=torch.float32).view(k, n) % 5).cuda()
    expected = oracle.gemm_fp64(a_storage.t(), b)
    torch.testing.assert_close(abi_sgemm(abi, impl, a_storage.t(), b).cpu(), expected, atol=0, rtol=0)


@pytest.mark.parametrize("impl", TILE_128)
def test_output_coordinates_are_exact(abi, impl):
    # Distinct row and column factors expose swapped or duplicated thread, warp
    # and CTA tiles, including CTA boundaries in both dimensions.
    m, n, k = 256, 384, 48
    rows = torch.arange(1, m + 1, device="cuda", dtype=torch.float32)
    cols = torch.arange(1, n + 1, device="cuda", dtype=torch.float32)
    a = rows.expand(k, m).contiguous().t()
    b = cols.expand(k, n).contiguous()
    expected = k * rows[:, None] * cols[None, :]
    torch.testing.assert_close(abi_sgemm(abi, impl, a, b), expected, atol=0, rtol=0)


@pytest.mark.parametrize("impl", PIPELINE)
@pytest.mark.parametrize("k", [16, 32, 48, 80, 144, 2048])
def test_every_k_row_is_used_exactly_once(abi, impl, k):
    # Row k of A holds k + 1 and so does row k of B: the product is the sum of
    # squares, which changes if a pipeline stage is dropped, repeated or if rows
    # past a K slice leak in.
    values = torch.arange(1, k + 1, device="cuda", dtype=torch.float32) % 13 + 1
    a = values.unsqueeze(1).expand(k, 128).contiguous().t()
    b = values.unsqueeze(1).expand(k, 256).contiguous()
    expected = torch.full((128, 256), float((values.double() ** 2).sum()), device="cuda")
    torch.testing.assert_close(abi_sgemm(abi, impl, a, b), expected, atol=0, rtol=0)


@pytest.mark.parametrize("impl", LADDER[1:10])
@pytest.mark.parametrize("k", [8, 24, 32, 40, 56, 72, 264])
def test_staged_ladder_uses_every_k_row_once(abi, impl, k):
    # The shared-memory stages hold 8 (register tiles) or 32 (one output per thread) rows of K per
    # slab, double-buffered; K ends inside a slab for most of these. Same construction as above:
    # exact on small integers, wrong if a slab is dropped, repeated or read past K.
    values = torch.arange(1, k + 1, device="cuda", dtype=torch.float32) % 13 + 1
    a = values.unsqueeze(1).expand(k, 128).contiguous().t()
    b = values.unsqueeze(1).expand(k, 256).contiguous()
    expected = torch.full((128, 256), float((values.double() ** 2).sum()), device="cuda")
    torch.testing.assert_close(abi_sgemm(abi, impl, a, b), expected, atol=0, rtol=0)
    assert_device_clean(abi)


@pytest.mark.parametrize("impl", ["prefetch_smem", "prefetch_reg"])
@pytest.mark.parametrize("k", [8, 24, 40])
def test_k_tails_shorter_than_a_stage(abi, impl, k):
    a_cpu, b_cpu, a, b = device_inputs(128, 128, k)
    check_against_oracle(abi_sgemm(abi, impl, a, b), a_cpu, b_cpu)


@pytest.mark.parametrize("impl", PIPELINE)
@pytest.mark.parametrize("shape", [(256, 128, 1024), (640, 256, 304), (2048, 1152, 512)])
def test_pipeline_kernels_on_multi_tile_shapes(abi, impl, shape):
    # More tiles than one wave of persistent CTAs needs, ragged K stages.
    a_cpu, b_cpu, a, b = device_inputs(*shape)
    check_against_oracle(abi_sgemm(abi, impl, a, b), a_cpu, b_cpu)
    assert_device_clean(abi)


@pytest.mark.parametrize("impl", LADDER)
def test_baseline_config_1024_cubed(abi, impl):
    a_cpu, b_cpu = oracle.ladder_inputs(1024, 1024, 1024, seed=0)
    a, b = oracle.to_device_preserving_strides(a_cpu, "cuda"), b_cpu.cuda()
    check_against_oracle(abi_sgemm(abi, impl, a, b), a_cpu, b_cpu)


@pytest.mark.parametrize("impl", PIPELINE)
@pytest.mark.parametrize("shape", [(4096, 4096, 4096), (1024, 4096, 4096)])
def test_baseline_config_full_size(abi, impl, shape):
    a_cpu, b_cpu = oracle.ladder_inputs(*shape, seed=0)
    a, b = oracle.to_device_preserving_strides(a_cpu, "cuda"), b_cpu.cuda()
    actual = abi_sgemm(abi, impl, a, b)
    check_against_oracle(actual, a_cpu, b_cpu)
    # Size-independent property: linearity in A. (2A)B == 2(AB) bit for bit,
    # because scaling by two is exact in binary floating point.
    doubled = abi_sgemm(abi, impl, (a.t() * 2).t(), b)
    if impl != "split_k":   # atomics make the reduction order, hence the last bit, run-dependent
        assert torch.equal(doubled, actual * 2)
    else:
        torch.testing.assert_close(doubled, actual * 2, atol=2 * oracle.sgemm_abs_tolerance(a_cpu, b_cpu), rtol=0)
    assert_device_clean(abi)


def test_split_k_clears_recycled_output(abi):
    a = torch.ones(32, 128, device="cuda").t()
    b = torch.ones(32, 256, device="cuda")
    impl = abi.b200_sgemm_impl_from_name(b"split_k")
    c = torch.full((128, 256), 12345.0, device="cuda")
    for value in (2.0, 0.0, 3.0):
        a.fill_(value)
        assert abi.b200_sgemm(impl, a.data_ptr(), b.data_ptr(), c.data_ptr(), 128, 256, 32, current_stream_ptr()) == 0
        torch.testing.assert_close(c, torch.full_like(c, value * 32), atol=0, rtol=0)


def test_abi_rejects_without_launching(abi):
    a = torch.zeros(16, 128, device="cuda").t()
    b = torch.zeros(16, 128, device="cuda")
    c = torch.zeros(128, 128, device="cuda")
    impl = abi.b200_sgemm_impl_from_name(b"prefetch_reg")
    args = (a.data_ptr(), b.data_ptr(), c.data_ptr())
    assert abi.b200_sgemm(impl, *args, 127, 128, 16, current_stream_ptr()) == 2
    assert abi.b200_sgemm(impl, *args, 128, 128, 0, current_stream_ptr()) == 4
    assert abi.b200_sgemm(impl, a.data_ptr() + 4, b.data_ptr(), c.data_ptr(), 128, 128, 8, current_stream_ptr()) == 1
    # A misaligned output: every vectorised entry stores C with 128-bit accesses, so it is refused
    # before any launch; the two scalar entries accept it.
    big = torch.zeros(128 * 128 + 4, device="cuda")
    shifted_c = big.data_ptr() + 4
    for name in LADDER:
        idx = abi.b200_sgemm_impl_from_name(name.encode())
        status = abi.b200_sgemm(idx, a.data_ptr(), b.data_ptr(), shifted_c, 128, 128, 16, current_stream_ptr())
        assert status == (0 if name in ("naive", "block_tile") else 1), name
    peers = (ctypes.c_void_p * 1)(c.data_ptr())
    assert abi.b200_sgemm_gather(impl, a.data_ptr(), b.data_ptr(), shifted_c, peers, 1, 128, 128, 16,
                                 current_stream_ptr()) == 1
    assert_device_clean(abi)


# Few tiles and a long K: prefetch_smem / prefetch_reg run clusters of 4 or 2 CTAs per tile that
# share the K range and add their partial tiles through distributed shared memory.
CLUSTER_SPLIT_SHAPES = [(256, 384, 1024),    # 6 tiles, 16 K blocks: clusters of 4
                        (128, 128, 200),     # 1 tile, 4 K blocks with a ragged last one: clusters of 2
                        (128, 128, 4096),    # 1 tile, 64 K blocks
                        (1024, 1024, 512),   # 64 tiles, 8 K blocks: clusters of 2
                        (640, 768, 1104)]    # 30 tiles, 18 K blocks (uneven shares, ragged K): clusters of 4


@pytest.mark.parametrize("impl", ["prefetch_smem", "prefetch_reg"])
@pytest.mark.parametrize("shape", CLUSTER_SPLIT_SHAPES)
def test_cluster_split_is_exact_on_integers_and_matches_the_oracle(abi, impl, shape):
    m, n, k = shape
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randint(-3, 4, (k, m), generator=g).float().cuda().t()      # column-major A
    b = torch.randint(-3, 4, (k, n), generator=g).float().cuda()
    out = abi_sgemm(abi, impl, a, b)
    torch.testing.assert_close(out.cpu(), oracle.gemm_fp64(a, b), atol=0, rtol=0)
    a_cpu, b_cpu, a_dev, b_dev = device_inputs(m, n, k, seed=k)
    first = abi_sgemm(abi, impl, a_dev, b_dev)
    check_against_oracle(first, a_cpu, b_cpu)
    assert torch.equal(abi_sgemm(abi, impl, a_dev, b_dev), first)          # partial tiles are added in rank order
    assert_device_clean(abi)


@pytest.mark.parametrize("name", PIPELINE)
@pytest.mark.parametrize("n", [128, 512, 19 * 1024])
def test_calls_in_a_row_read_what_the_last_one_wrote(abi, name, n):
    # The pipeline kernel is launched under programmatic stream serialization (it may become resident
    # while the kernel before it still runs and waits for it before touching global memory): three
    # calls with nothing between them, C of one the B of the next. A in {-1, 0, 1}, K = 128: exact.
    m = k = 128
    g = torch.Generator().manual_seed(n)
    a = torch.randint(-1, 2, (m, k), generator=g).float()
    b = torch.randint(-2, 3, (k, n), generator=g).float()
    a_dev = oracle.to_device_preserving_strides(a.t().contiguous().t(), "cuda")   # column-major [M, K]
    outs = [b.cuda()] + [torch.full((m, n), float("nan"), device="cuda") for _ in range(3)]
    impl = abi.b200_sgemm_impl_from_name(name.encode())
    torch.cuda.synchronize()
    for i in range(3):
        assert abi.b200_sgemm(impl, a_dev.data_ptr(), outs[i].data_ptr(), outs[i + 1].data_ptr(), m, n, k, current_stream_ptr()) == 0
    expected = b.double()
    for i in range(3):
        expected = a.double() @ expected
    torch.testing.assert_close(outs[3].cpu().double(), expected, atol=0, rtol=0)
    assert_device_clean(abi)
