"""Parity of the tcgen05 TF32 GEMM + fused epilogue with the CPU oracle, through
the C ABI. Tolerances: relative Frobenius error <= 5e-3 (north star) and the
reference suite's atol = rtol = 3e-2; exact for inputs that TF32 represents
exactly (small integers), which is what checks the shared-memory descriptors,
the swizzled layouts and the TMEM addressing element by element."""
import ctypes

import pytest
import torch

from conftest import GemmProblem, KernelMeta, assert_device_clean, current_stream_ptr
from oracle import oracle

pytestmark = pytest.mark.gpu

LINEAR, RELU, GELU = 0, 1, 2
EPILOGUE_NAME = {LINEAR: "linear", RELU: "relu", GELU: "gelu"}


def registry(abi):
    out = []
    for i in range(abi.b200_tf32_registry_size()):
        meta = KernelMeta()
        abi.b200_tf32_registry_entry(i, ctypes.byref(meta))
        out.append((meta.id, meta.alias.decode(), meta.epilogue, meta.alignment_a))
    return out


def run(abi, kernel_id, a, b, c=None, alpha=1.0, beta=0.0, epilogue=LINEAR, dispatch=False, bias=None):
    m, k = a.shape
    n = b.shape[1]
    d = torch.full((m, n), float("nan"), device=a.device)
    q = GemmProblem(m, n, k, a.data_ptr(), b.data_ptr(), c.data_ptr() if c is not None else None, d.data_ptr(),
                    a.stride(0), b.stride(0), c.stride(0) if c is not None else n, d.stride(0), alpha, beta, epilogue,
                    bias.data_ptr() if bias is not None else None)
    if dispatch:
        chosen = ctypes.c_int(-1)
        status = abi.b200_tf32_gemm_dispatch(kernel_id, ctypes.byref(q), ctypes.byref(chosen), current_stream_ptr())
        return status, d, chosen.value
    status = abi.b200_tf32_gemm_launch(kernel_id, ctypes.byref(q), current_stream_ptr())
    return status, d, kernel_id


def check(actual, expected, k=64):
    assert oracle.rel_frobenius(actual, expected) <= oracle.TF32_REL_FROBENIUS
    # Element-wise gate of the reference suite (3e-2, chosen there for K <= 64).
    # tcgen05 truncates FP32 operands to TF32, so the absolute error of a sum
    # grows like sqrt(K); the absolute part of the gate is scaled accordingly.
    atol = 3e-2 * max(1.0, (k / 64) ** 0.5 / 2)
    torch.testing.assert_close(actual.cpu(), expected, atol=atol, rtol=3e-2)


def entries(align=None, epilogue=None, skinny=False):
    """Registry entries as (id, alias, epilogue, alignment of A); the tensor-core ones unless `skinny`."""
    import conftest

    lib = conftest.load_abi()
    return [e for e in registry(lib) if (align is None or e[3] == align) and (epilogue is None or e[2] == epilogue)
            and e[1].startswith("skinny") == skinny]


@pytest.mark.parametrize("entry", entries(), ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [(128, 128, 32), (128, 256, 64), (256, 512, 96), (384, 320, 160)])
def test_integer_inputs_are_reproduced_exactly(abi, entry, shape):
    # Values in [-4, 4] are exact in TF32 and every partial sum is exact in
    # FP32, so any element that comes from the wrong (m, k) or (k, n) shows.
    kernel_id, _, epilogue, _ = entry
    m, n, k = shape
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randint(-4, 5, (m, k), generator=g).float()
    b = torch.randint(-4, 5, (k, n), generator=g).float()
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), epilogue=epilogue)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, epilogue=EPILOGUE_NAME[epilogue])
    # The accumulator is exact; only the erf of the GELU entries is rounded.
    tol = 1e-5 if epilogue == GELU else 0
    torch.testing.assert_close(d.cpu(), expected, atol=tol, rtol=tol)
    assert_device_clean(abi)


@pytest.mark.parametrize("entry", entries(), ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [(128, 128, 64), (33, 68, 20), (200, 264, 1000), (1024, 1024, 1024)])
def test_aligned_shapes_match_oracle(abi, entry, shape):
    kernel_id, _, epilogue, _ = entry
    a, b, c = oracle.adaptive_inputs(*shape)
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), alpha=1.0, beta=0.5, epilogue=epilogue)
    assert status == 0, abi.b200_status_string(status)
    check(d, oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, EPILOGUE_NAME[epilogue]), k=shape[2])
    assert_device_clean(abi)


@pytest.mark.parametrize("entry", entries(align=1), ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [(33, 65, 17), (1, 1, 1), (33, 65, 20), (33, 68, 17), (130, 259, 70), (5, 300, 33)])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (0.75, 0.25), (-0.5, 1.0), (0.0, -1.0)])
def test_generic_loader_takes_any_shape(abi, entry, shape, alpha, beta):
    kernel_id, _, epilogue, _ = entry
    a, b, c = oracle.adaptive_inputs(*shape)
    c_dev = c.cuda() if beta else None
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c_dev, alpha, beta, epilogue)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, alpha, beta, EPILOGUE_NAME[epilogue])
    torch.testing.assert_close(d.cpu(), expected, atol=3e-2, rtol=3e-2)
    if epilogue == RELU:
        assert bool((d >= 0).all())
    assert_device_clean(abi)


@pytest.mark.parametrize("entry", entries(align=4), ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [(33, 65, 20), (33, 68, 17)])
def test_tma_entries_refuse_misaligned_shapes(abi, entry, shape):
    a, b, _ = oracle.adaptive_inputs(*shape)
    status, _, _ = run(abi, entry[0], a.cuda(), b.cuda(), epilogue=entry[2])
    assert status == 1  # misaligned operand


def test_misaligned_pointer_falls_through_to_the_generic_loader(abi):
    a, b, _ = oracle.adaptive_inputs(128, 128, 64)
    a_dev = torch.empty(128 * 64 + 1, device="cuda")[1:].view(128, 64).copy_(a)
    status, d, chosen = run(abi, 0, a_dev, b.cuda(), dispatch=True)
    assert status == 0 and chosen == 3
    check(d, oracle.adaptive_gemm_fp64(a, b))


@pytest.mark.parametrize("kernel", [0, 8, 9])
def test_relu_is_applied_after_scale_and_source_add(abi, kernel):
    a = torch.eye(4, device="cuda")
    b = torch.tensor([[-2.0, -1.0, 1.0, 2.0]], device="cuda").repeat(4, 1)
    c = torch.tensor([[-2.0, -2.0, 2.0, 2.0]], device="cuda").repeat(4, 1)
    status, d, _ = run(abi, kernel, a, b, c, alpha=-1.0, beta=1.0, epilogue=RELU, dispatch=True)
    assert status == 0
    expected = torch.tensor([[0.0, 0.0, 1.0, 0.0]], device="cuda").repeat(4, 1)
    torch.testing.assert_close(d, expected, atol=0, rtol=0)


@pytest.mark.parametrize("kernel", [0, 8, 9])
def test_beta_zero_never_reads_the_source(abi, kernel):
    a = torch.eye(4, device="cuda")
    b = torch.tensor([[-2.0, -1.0, 1.0, 2.0]], device="cuda").repeat(4, 1)
    c = torch.full((4, 4), float("nan"), device="cuda")
    status, d, _ = run(abi, kernel, a, b, c, beta=0.0, epilogue=RELU, dispatch=True)
    assert status == 0
    torch.testing.assert_close(d, b.relu(), atol=0, rtol=0)


def test_auto_dispatch_order(abi):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    # Mid-sized aligned problem: no shape gate fires, the reference order decides.
    m = 128 * ((sms + 1) // 2 + 1)          # too many 128-wide tiles for "narrow", too few 256 x 256 for "pair"
    a, b, _ = oracle.adaptive_inputs(m, 128, 64)
    assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] == 2               # fast
    assert run(abi, 0, a.cuda(), b.cuda(), epilogue=RELU, dispatch=True)[2] == 8  # fast_relu
    # Small problems: 128-wide tiles would idle most SMs -> the narrowest width that runs in one round.
    a, b, _ = oracle.adaptive_inputs(256, 256, 64)
    assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] == 57              # width32
    assert run(abi, 0, a.cuda(), b.cuda(), epilogue=RELU, dispatch=True)[2] == 58
    a, b, _ = oracle.adaptive_inputs(128 * 8, 64 * (sms // 8), 64)             # 32-wide tiles would need two rounds
    assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] == 18              # narrow
    assert run(abi, 0, a.cuda(), b.cuda(), epilogue=RELU, dispatch=True)[2] == 19
    # Large problem: 256 x 256 CTA pairs fill at least one round of pairs.
    a, b, _ = oracle.adaptive_inputs(256 * 8, 256 * ((sms // 2 + 7) // 8), 64)
    assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] == 20              # pair
    assert run(abi, 0, a.cuda(), b.cuda(), epilogue=RELU, dispatch=True)[2] == 21
    # In between: the narrowest tile width (a multiple of 32 columns) whose tiles run in one round.
    a, b, _ = oracle.adaptive_inputs(128 * 8, 256 * (sms // 8), 64)            # only 128 x 256 tiles do
    assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] == 16              # wide
    assert run(abi, 0, a.cuda(), b.cuda(), epilogue=RELU, dispatch=True)[2] == 17
    for width, linear_id in ((224, 54), (192, 45), (160, 51), (96, 48)):
        n = width * (sms // 8)                                                  # 8 x (sms // 8) tiles of that width
        a, b, _ = oracle.adaptive_inputs(128 * 8, n, 64)
        assert 8 * -(-n // (width - 32)) > sms                                  # one width narrower needs a second round
        assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] == linear_id
        assert run(abi, 0, a.cuda(), b.cuda(), epilogue=RELU, dispatch=True)[2] == linear_id + 1
    a, b, _ = oracle.adaptive_inputs(33, 65, 17)
    assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] == 3               # fallback
    assert run(abi, 0, a.cuda(), b.cuda(), epilogue=RELU, dispatch=True)[2] == 9  # fallback_relu


def test_strided_operands(abi):
    # Leading dimensions larger than the logical width (sub-matrices of wider buffers).
    big_a = torch.randn(256, 192, device="cuda")
    big_b = torch.randn(192, 512, device="cuda")
    big_c = torch.randn(256, 640, device="cuda")
    a, b, c = big_a[:, :128], big_b[:128, :384], big_c[:, :384]
    status, d, chosen = run(abi, 0, a, b, c, alpha=0.5, beta=2.0, dispatch=True)
    assert status == 0 and chosen in (2, 18, 57)
    check(d, oracle.adaptive_gemm_fp64(a, b, c, 0.5, 2.0))


@pytest.mark.parametrize("epilogue", [LINEAR, RELU])
def test_baseline_config_8192_sampled_rows(abi, epilogue):
    # D = relu(1.0 * A @ B + 0.5 * C) at M = N = K = 8192. The FP64 oracle is
    # evaluated on 96 sampled rows (and therefore every column and the whole K
    # range); a row of a GEMM depends on nothing outside that row of A and C.
    n = 8192
    g = torch.Generator().manual_seed(0)
    a = torch.randn(n, n, generator=g)
    b = torch.randn(n, n, generator=g)
    c = torch.randn(n, n, generator=g)
    status, d, chosen = run(abi, 0, a.cuda(), b.cuda(), c.cuda(), 1.0, 0.5, epilogue, dispatch=True)
    assert status == 0
    rows = torch.randperm(n, generator=g)[:96]
    expected = oracle.adaptive_gemm_fp64(a[rows], b, c[rows], 1.0, 0.5, EPILOGUE_NAME[epilogue])
    check(d[rows.cuda()], expected, k=n)
    # Size-independent property: with beta = 0 the ReLU output is the positive
    # part of the linear output, element for element.
    if epilogue == RELU:
        lin = run(abi, 0, a.cuda(), b.cuda(), c.cuda(), 1.0, 0.5, LINEAR, dispatch=True)[1]
        assert torch.equal(d, lin.clamp_min(0))
    assert_device_clean(abi)


# ------------------------------------------------ bias and GELU epilogues
# Declared by the reference, refused by it at run time; no reference vectors
# exist, the oracle states them (bias added before the activation, erf GELU).

@pytest.mark.parametrize("entry", entries(), ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [(128, 128, 64), (300, 520, 100)])
def test_bias_is_added_before_the_activation(abi, entry, shape):
    kernel_id, _, epilogue, align = entry
    m, n, k = shape
    if align == 1:
        m, n, k = m + 1, n + 3, k + 1          # the generic loader's territory
    a, b, c = oracle.adaptive_inputs(m, n, k)
    bias = torch.linspace(-2, 2, n)
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), 0.5, 0.25, epilogue, bias=bias.cuda())
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, 0.5, 0.25, "bias" if epilogue == LINEAR else "bias_" + EPILOGUE_NAME[epilogue],
                                         bias)
    check(d, expected, k=k)
    assert_device_clean(abi)


def test_exact_bias_and_gelu_values(abi):
    # Identity A: the accumulator is B exactly; bias and GELU act on known values.
    a = torch.eye(4, device="cuda")
    b = torch.tensor([[-2.0, -1.0, 0.0, 2.0]], device="cuda").repeat(4, 1)
    bias = torch.tensor([1.0, 1.0, -3.0, 0.5], device="cuda")
    status, d, _ = run(abi, 0, a, b, epilogue=RELU, dispatch=True, bias=bias)
    assert status == 0
    torch.testing.assert_close(d, torch.tensor([[0.0, 0.0, 0.0, 2.5]], device="cuda").repeat(4, 1), atol=0, rtol=0)
    status, d, chosen = run(abi, 0, a, b, epilogue=GELU, dispatch=True)
    assert status == 0 and chosen == 29   # four rows: the skinny entry under automatic dispatch
    expected = torch.nn.functional.gelu(b.double()).float()
    torch.testing.assert_close(d, expected, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("size", [1024, 4096])
def test_gelu_auto_dispatch_at_benchmark_sizes(abi, size):
    a, b, c = oracle.adaptive_inputs(size, size, size)
    rows = torch.arange(0, size, max(1, size // 64))
    bias = torch.randn(size)
    status, d, chosen = run(abi, 0, a.cuda(), b.cuda(), c.cuda(), 1.0, 0.5, GELU, dispatch=True, bias=bias.cuda())
    assert status == 0 and chosen in (22, 23, 24, 25, 32)   # narrow or pair entries at these sizes
    expected = oracle.adaptive_gemm_fp64(a[rows], b, c[rows], 1.0, 0.5, "bias_gelu", bias)
    check(d[rows.cuda()], expected, k=size)


def test_misaligned_bias_pointer_uses_scalar_epilogue(abi):
    a, b, c = oracle.adaptive_inputs(128, 128, 64)
    bias = torch.randn(128)
    bias_dev = torch.empty(129, device="cuda")[1:].copy_(bias)
    status, d, chosen = run(abi, 0, a.cuda(), b.cuda(), c.cuda(), 1.0, 1.0, LINEAR, dispatch=True, bias=bias_dev)
    assert status == 0
    check(d, oracle.adaptive_gemm_fp64(a, b, c, 1.0, 1.0, "bias", bias))


# ----------------------------------------------------------------- skinny rows
# M <= 16: FP32 FMA stream over B with K split over warps and a cluster. FP32
# arithmetic, so besides the TF32 gates the result has to be FP32-accurate.


@pytest.mark.parametrize("entry", entries(skinny=True), ids=lambda e: e[1])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(4096, 4096), (132, 100), (4, 7), (260, 1000), (1024, 8)])
def test_skinny_rows_match_oracle(abi, entry, m, n, k):
    kernel_id, _, epilogue, _ = entry
    a, b, c = oracle.adaptive_inputs(m, n, k, seed=m)
    bias = torch.linspace(-1.0, 1.0, n)
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), alpha=0.75, beta=0.25, epilogue=epilogue,
                       bias=bias.cuda())
    assert status == 0, abi.b200_status_string(status)
    name = "bias" if epilogue == LINEAR else "bias_" + EPILOGUE_NAME[epilogue]
    expected = oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, name, bias=bias)
    check(d, expected, k=k)
    tol = oracle.sgemm_abs_tolerance(a, b)   # the FP32 ladder's bound
    assert float((d.cpu() - expected).abs().max()) <= tol
    assert_device_clean(abi)


@pytest.mark.parametrize("m", [1, 7, 16])
def test_skinny_rows_reproduce_integers_exactly(abi, m):
    g = torch.Generator().manual_seed(m)
    a = torch.randint(-4, 5, (m, 777), generator=g).float()
    b = torch.randint(-4, 5, (777, 520), generator=g).float()
    status, d, _ = run(abi, 27, a.cuda(), b.cuda())
    assert status == 0
    torch.testing.assert_close(d.cpu(), oracle.adaptive_gemm_fp64(a, b), atol=0, rtol=0)


def test_skinny_dispatch_and_refusals(abi):
    a, b, _ = oracle.adaptive_inputs(4, 4096, 4096)
    for epilogue, expected_id in ((LINEAR, 27), (RELU, 28), (GELU, 29)):
        status, _, chosen = run(abi, 0, a.cuda(), b.cuda(), epilogue=epilogue, dispatch=True)
        assert status == 0 and chosen == expected_id
    # From five rows on automatic dispatch prefers the tensor-core entries: operands swapped up to 16 rows.
    a5, b5, _ = oracle.adaptive_inputs(16, 4096, 4096)
    assert run(abi, 0, a5.cuda(), b5.cuda(), dispatch=True)[2] == 36
    a6, b6, _ = oracle.adaptive_inputs(17, 4096, 4096)
    assert run(abi, 0, a6.cuda(), b6.cuda(), dispatch=True)[2] == 30
    # More than 16 rows: a forced call is refused.
    a17, b17, _ = oracle.adaptive_inputs(17, 256, 64)
    assert run(abi, 27, a17.cuda(), b17.cuda())[0] == 2          # invalid problem
    assert run(abi, 0, a17.cuda(), b17.cuda(), dispatch=True)[2] not in (27, 28, 29)
    # Columns that are not whole float4 groups, or a misaligned B: refused, dispatch moves on.
    a1, b1, _ = oracle.adaptive_inputs(4, 66, 32)
    assert run(abi, 27, a1.cuda(), b1.cuda())[0] in (1, 2)
    status, d, chosen = run(abi, 0, a1.cuda(), b1.cuda(), dispatch=True)
    assert status == 0 and chosen == 3
    check(d, oracle.adaptive_gemm_fp64(a1, b1))
    b_off = torch.empty(64 * 128 + 1, device="cuda")[1:].view(64, 128)
    a2, b2, _ = oracle.adaptive_inputs(4, 128, 64)
    b_off.copy_(b2)
    assert run(abi, 27, a2.cuda(), b_off)[0] == 1                # misaligned operand
    # A may sit anywhere: only B is read with 128-bit loads.
    a_off = torch.empty(4 * 64 + 1, device="cuda")[1:].view(4, 64).copy_(a2)
    status, d, _ = run(abi, 27, a_off, b2.cuda())
    assert status == 0
    check(d, oracle.adaptive_gemm_fp64(a2, b2))
    assert_device_clean(abi)


def test_skinny_beta_zero_never_reads_the_source(abi):
    a, b, _ = oracle.adaptive_inputs(8, 512, 256)
    poison = torch.full((8, 512), float("nan"), device="cuda")
    status, d, _ = run(abi, 27, a.cuda(), b.cuda(), poison, alpha=1.0, beta=0.0)
    assert status == 0
    check(d, oracle.adaptive_gemm_fp64(a, b), k=256)


# --------------------------------------------------------------- split-K cluster
# One 128 x 128 tile per cluster of 1/2/4/8 CTAs; partial tiles are exchanged
# through distributed shared memory and added in rank order.


@pytest.mark.parametrize("entry", [e for e in entries() if e[1].startswith("splitk")], ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [
    (16, 4096, 4096),    # decode-like: 32 tiles x 8 ranks
    (64, 128, 288),      # 9 K blocks over 4 ranks: the last rank has an empty range
    (100, 200, 200),     # 7 K blocks over 2 ranks, ragged rows, columns and K
    (512, 512, 2048),    # 16 tiles x 8 ranks
    (1024, 1024, 1024),  # 64 tiles x 4 ranks
    (130, 132, 4100),    # tile edges inside a cluster's column shares
])
def test_split_k_cluster_matches_oracle(abi, entry, shape):
    kernel_id, _, epilogue, _ = entry
    a, b, c = oracle.adaptive_inputs(*shape, seed=shape[0])
    bias = torch.linspace(-1.0, 1.0, shape[1])
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), alpha=0.75, beta=0.25, epilogue=epilogue,
                       bias=bias.cuda())
    assert status == 0, abi.b200_status_string(status)
    name = "bias" if epilogue == LINEAR else "bias_" + EPILOGUE_NAME[epilogue]
    check(d, oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, name, bias=bias), k=shape[2])
    assert_device_clean(abi)


def test_split_k_cluster_is_deterministic_and_exact_on_integers(abi):
    g = torch.Generator().manual_seed(5)
    a = torch.randint(-4, 5, (48, 1024), generator=g).float()
    b = torch.randint(-4, 5, (1024, 384), generator=g).float()
    first = run(abi, 30, a.cuda(), b.cuda())[1]
    torch.testing.assert_close(first.cpu(), oracle.adaptive_gemm_fp64(a, b), atol=0, rtol=0)
    a2, b2, _ = oracle.adaptive_inputs(48, 384, 1024)
    runs = [run(abi, 30, a2.cuda(), b2.cuda())[1] for _ in range(3)]
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])


def test_split_k_auto_dispatch(abi):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    a, b, _ = oracle.adaptive_inputs(64, 1024, 2048)       # 8 tiles, 64 K blocks
    for epilogue, expected_id in ((LINEAR, 30), (RELU, 31), (GELU, 32)):
        status, _, chosen = run(abi, 0, a.cuda(), b.cuda(), epilogue=epilogue, dispatch=True)
        assert status == 0 and chosen == expected_id
    # Enough tiles for every SM: no split.
    a, b, _ = oracle.adaptive_inputs(128 * 8, 128 * ((sms + 7) // 8), 256)
    assert run(abi, 0, a.cuda(), b.cuda(), dispatch=True)[2] not in (30, 31, 32)


# --------------------------------------------------------- operands swapped
# D^T = B^T A^T for few rows: the MMA's 128 rows run along N, its N side holds 16 or 64 rows of A.


@pytest.mark.parametrize("entry", [e for e in entries() if e[1].startswith("swap")], ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [
    (1, 4096, 4096), (16, 4096, 4096), (13, 260, 1000), (17, 132, 100), (64, 1024, 2048), (40, 8192, 320),
    (5, 4, 8), (100, 200, 300),      # more than 64 rows: several row blocks
])
def test_swapped_operands_match_oracle(abi, entry, shape):
    kernel_id, _, epilogue, _ = entry
    a, b, c = oracle.adaptive_inputs(*shape, seed=shape[0])
    bias = torch.linspace(-1.0, 1.0, shape[1])
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), alpha=0.75, beta=0.25, epilogue=epilogue,
                       bias=bias.cuda())
    assert status == 0, abi.b200_status_string(status)
    name = "bias" if epilogue == LINEAR else "bias_" + EPILOGUE_NAME[epilogue]
    check(d, oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, name, bias=bias), k=shape[2])
    assert_device_clean(abi)


def test_swapped_operands_are_exact_on_integers_and_deterministic(abi):
    g = torch.Generator().manual_seed(11)
    for m in (3, 16, 33):
        a = torch.randint(-4, 5, (m, 1024), generator=g).float()
        b = torch.randint(-4, 5, (1024, 640), generator=g).float()
        first = run(abi, 36, a.cuda(), b.cuda())[1]
        torch.testing.assert_close(first.cpu(), oracle.adaptive_gemm_fp64(a, b), atol=0, rtol=0)
        assert torch.equal(first, run(abi, 36, a.cuda(), b.cuda())[1])


# ------------------------------------------------ CTA pairs: half tiles in the last round


@pytest.mark.parametrize("kernel,epilogue", [(20, LINEAR), (21, RELU)])
def test_pair_kernel_runs_a_short_last_round_as_half_tiles(abi, kernel, epilogue):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    pairs = sms // 2
    # pairs + 10 tiles of 256 x 256 (arranged 2 x ... would need a factorisation: use one tile row more than fits):
    tiles_n = 7
    tiles_m = (pairs + 10 + tiles_n - 1) // tiles_n        # 12 on 148 SMs: 84 tiles, 10 left over -> 20 half tiles
    assert 0 < (tiles_m * tiles_n) % pairs <= pairs // 2
    m, n, k = 256 * tiles_m, 256 * tiles_n - 36, 100        # ragged right edge: the last half tile is partly outside
    g = torch.Generator().manual_seed(3)
    a = torch.randint(-4, 5, (m, k), generator=g).float()
    b = torch.randint(-4, 5, (k, n), generator=g).float()
    c = torch.randint(-4, 5, (m, n), generator=g).float()
    status, d, _ = run(abi, kernel, a.cuda(), b.cuda(), c.cuda(), alpha=1.0, beta=0.5, epilogue=epilogue)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, EPILOGUE_NAME[epilogue])
    torch.testing.assert_close(d.cpu(), expected, atol=0, rtol=0)      # integers: exact
    assert_device_clean(abi)


# ------------------------------------------------------------ source and destination are one buffer
# Every element's source value is read by the thread (or the warp) that later writes it, so an
# accumulation in place must give what a separate source gives: through the boxes and TMA stores of
# the tile kernels, through the split-K finishing passes (inside the matrix and at its edges).


@pytest.mark.parametrize("entry", entries(), ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [(256, 384, 192), (200, 264, 96)])
def test_source_may_be_the_destination(abi, entry, shape):
    kernel_id, alias, epilogue, align = entry
    m, n, k = (16, 256, shape[2]) if alias.startswith("swap") else shape
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randint(-4, 5, (m, k), generator=g).float()
    b = torch.randint(-4, 5, (k, n), generator=g).float()
    c = torch.randint(-4, 5, (m, n), generator=g).float()
    d = c.clone().cuda()
    a_dev, b_dev = a.cuda(), b.cuda()
    q = GemmProblem(m, n, k, a_dev.data_ptr(), b_dev.data_ptr(), d.data_ptr(), d.data_ptr(), k, n, n, n, 1.0, 0.5, epilogue, None)
    status = abi.b200_tf32_gemm_launch(kernel_id, ctypes.byref(q), current_stream_ptr())
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, EPILOGUE_NAME[epilogue])
    tol = 1e-5 if epilogue == GELU else 0
    torch.testing.assert_close(d.cpu(), expected, atol=tol, rtol=tol)
    assert_device_clean(abi)


# ------------------------------------------------ K that ends inside a pipeline stage
# Stages hold two or four 32-wide K sub-blocks; a K that ends inside the first sub-block, between
# sub-blocks or inside the last one must read the missing part as zeros.


@pytest.mark.parametrize("entry", entries(align=4), ids=lambda e: e[1])
@pytest.mark.parametrize("k", [4, 36, 64, 68, 100, 132])
def test_k_tail_inside_a_stage(abi, entry, k):
    kernel_id, alias, epilogue, _ = entry
    m, n = (16, 256) if alias.startswith("swap") else (256, 384)
    g = torch.Generator().manual_seed(k)
    a = torch.randint(-4, 5, (m, k), generator=g).float()
    b = torch.randint(-4, 5, (k, n), generator=g).float()
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), epilogue=epilogue)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, epilogue=EPILOGUE_NAME[epilogue])
    tol = 1e-5 if epilogue == GELU else 0
    torch.testing.assert_close(d.cpu(), expected, atol=tol, rtol=tol)
    assert_device_clean(abi)


# ------------------------------------------------ long K: the 128 x 128 tile's issuers take stages in turn
# Above K = 2560 the 128 x 128 tile kernel runs single-block stages that its two MMA issuers take
# alternately, padding K to an even number of 32-wide blocks that read as zeros: an odd block
# count (83), an even one, and a K that ends inside a block.


@pytest.mark.parametrize("entry", [e for e in entries(align=4) if e[1] in ("fast", "fast_relu", "fast_gelu")], ids=lambda e: e[1])
@pytest.mark.parametrize("shape", [(256, 384, 2656), (130, 200, 2600), (128, 128, 2688)])
def test_long_k_through_alternating_issuers(abi, entry, shape):
    kernel_id, _, epilogue, _ = entry
    m, n, k = shape
    g = torch.Generator().manual_seed(k + m)
    a = torch.randint(-4, 5, (m, k), generator=g).float()
    b = torch.randint(-4, 5, (k, n), generator=g).float()
    c = torch.randint(-4, 5, (m, n), generator=g).float()
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), alpha=1.0, beta=0.5, epilogue=epilogue)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, EPILOGUE_NAME[epilogue])
    tol = 1e-5 if epilogue == GELU else 0
    torch.testing.assert_close(d.cpu(), expected, atol=tol, rtol=tol)
    assert_device_clean(abi)


# ------------------------------------------------ more tiles than SMs: a CTA walks several tiles
# The persistent tile kernels hand their two accumulator buffers (each with one accumulator per MMA
# issuer) back and forth between the issuers and the epilogue warps; with more tiles than SMs some
# CTAs take a second tile, and its partial sums must not meet the first tile's.


@pytest.mark.parametrize("alias,shape", [("fast", (2048, 1280, 160)), ("fast_relu", (2048, 1280, 2720)),
                                         ("narrow", (1280, 1024, 160)), ("narrow_relu", (2560, 1024, 96)),
                                         ("wide", (2048, 2560, 96)), ("medium", (2048, 1920, 96)), ("medium_relu", (2048, 2000, 2080)),
                                         ("fast_stage3", (2048, 1280, 100))])
def test_persistent_ctas_walk_several_tiles(abi, alias, shape):
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    kernel_id = abi.b200_tf32_kernel_from_name(alias.encode())
    assert kernel_id > 0
    epilogue = RELU if alias.endswith("relu") else LINEAR
    m, n, k = shape
    tile_n = {"fast": 128, "narrow": 64, "wide": 256, "medium": 192}[alias.split("_")[0]]
    assert (m // 128) * (n // tile_n) > sms, "the shape must give some CTA a second tile"
    g = torch.Generator().manual_seed(m + k)
    a = torch.randint(-4, 5, (m, k), generator=g).float()
    b = torch.randint(-4, 5, (k, n), generator=g).float()
    c = torch.randint(-4, 5, (m, n), generator=g).float()
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), alpha=1.0, beta=0.5, epilogue=epilogue)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, EPILOGUE_NAME[epilogue])
    torch.testing.assert_close(d.cpu(), expected, atol=0, rtol=0)
    assert_device_clean(abi)


# ------------------------------------------------------- error-compensated TF32 (three products)


def run_x3(abi, a, b, c=None, alpha=1.0, beta=0.0, epilogue=LINEAR, bias=None, scratch_slack=0):
    m, k = a.shape
    n = b.shape[1]
    d = torch.full((m, n), float("nan"), device=a.device)
    q = GemmProblem(m, n, k, a.data_ptr(), b.data_ptr(), c.data_ptr() if c is not None else None, d.data_ptr(),
                    a.stride(0), b.stride(0), c.stride(0) if c is not None else n, d.stride(0), alpha, beta, epilogue,
                    bias.data_ptr() if bias is not None else None)
    need = abi.b200_tf32x3_scratch_bytes(m, n, k)
    scratch = torch.empty(need // 4 + scratch_slack, device=a.device)
    status = abi.b200_tf32x3_gemm(ctypes.byref(q), scratch.data_ptr(), need, current_stream_ptr())
    return status, d


@pytest.mark.parametrize("shape", [(256, 256, 1024), (130, 136, 300), (33, 65, 517), (1024, 1024, 1024)])
def test_compensated_tf32_has_fp32_class_accuracy(abi, shape):
    """Three TF32 products reach the accuracy bar of the FP32 SIMT ladder, which one pass misses by 100x."""
    m, n, k = shape
    a, b, c = oracle.adaptive_inputs(m, n, k, seed=11)
    status, d = run_x3(abi, a.cuda(), b.cuda(), c.cuda(), alpha=1.0, beta=0.5, epilogue=RELU)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, "relu")
    err = (d.cpu() - expected).abs().max().item()
    assert err <= oracle.sgemm_abs_tolerance(a, b), err            # 1e-4 * sqrt(K) * max|A| * max|B|
    torch.testing.assert_close(d.cpu(), expected, atol=1e-3, rtol=1e-3)
    assert oracle.rel_frobenius(d, expected) <= 2e-5
    # One pass on the same inputs, for contrast: inside the TF32 bar, far outside the FP32 one.
    _, single, _ = run(abi, 0, a.cuda(), b.cuda(), c.cuda(), 1.0, 0.5, RELU, dispatch=True)
    assert oracle.rel_frobenius(single, expected) > 20 * oracle.rel_frobenius(d, expected)
    assert_device_clean(abi)


def test_compensated_tf32_bias_integers_and_refusals(abi):
    g = torch.Generator().manual_seed(3)
    a = torch.randint(-4, 5, (200, 96), generator=g).float()
    b = torch.randint(-4, 5, (96, 264), generator=g).float()
    bias = torch.arange(264).float() - 100
    status, d = run_x3(abi, a.cuda(), b.cuda(), epilogue=LINEAR, bias=bias.cuda())
    assert status == 0
    torch.testing.assert_close(d.cpu(), oracle.adaptive_gemm_fp64(a, b, epilogue="bias", bias=bias), atol=0, rtol=0)
    # A non-finite operand poisons its row (inf times a zero correction term is NaN) and nothing else.
    a2 = a.clone()
    a2[3, 5] = float("inf")
    status, d = run_x3(abi, a2.cuda(), b.cuda())
    assert status == 0
    finite = torch.isfinite(d.cpu())
    assert not bool(finite[3].any()) and bool(finite[:3].all()) and bool(finite[4:].all())
    keep = [r for r in range(200) if r != 3]
    torch.testing.assert_close(d.cpu()[keep], oracle.adaptive_gemm_fp64(a, b)[keep], atol=0, rtol=0)
    # Scratch that is too small, missing or misaligned is refused before any launch.
    q = GemmProblem(200, 264, 96, a.cuda().data_ptr(), b.cuda().data_ptr(), None, d.data_ptr(), 96, 264, 264, 264, 1.0, 0.0,
                    LINEAR, None)
    need = abi.b200_tf32x3_scratch_bytes(200, 264, 96)
    assert need == (200 * 96 + 96 * 264) * 4
    assert abi.b200_tf32x3_scratch_bytes(3, 5, 7) == (3 * 8 + 7 * 8) * 4          # rows padded to four floats
    scratch = torch.empty(need // 4 + 4, device="cuda")
    assert abi.b200_tf32x3_gemm(ctypes.byref(q), scratch.data_ptr(), need - 4, current_stream_ptr()) == 4
    assert abi.b200_tf32x3_gemm(ctypes.byref(q), None, need, current_stream_ptr()) == 4
    assert abi.b200_tf32x3_gemm(ctypes.byref(q), scratch.data_ptr() + 4, need, current_stream_ptr()) == 4
    assert_device_clean(abi)


# ------------------------------- CTA-pair kernel: whole 256 x 256 tiles, then 256 x 128 half tiles
# A last round of tiles that would occupy at most half the pairs runs as half tiles. Their stages lie
# differently in the operand ring (four of 48 KiB across the whole tiles' three of 64 KiB, starting
# in the slot that comes free first) and their MMAs come from two threads with an accumulator each.


@pytest.mark.parametrize("size,k", [(2304, 192), (2304, 256), (2304, 320), (2304, 200), (2304, 64), (2304, 1088),
                                    (4096, 160)])
def test_pair_kernel_goes_from_whole_tiles_to_half_tiles(abi, size, k):
    # 2304: 81 tiles on 74 pairs, every pair multiplies a whole tile, fourteen of them a half tile
    # after it; K sets the ring slot the whole tile ends on (3, 4 and 5 stages of 64 floats), a ragged
    # K, a single stage and many stages. 4096: three whole tiles per pair before the half.
    # Whole numbers: every element is exact.
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    m = n = size
    tiles, pairs = (m // 256) * (n // 256), sms // 2
    if not (pairs < tiles and 2 * (tiles % pairs) <= pairs):
        pytest.skip("this part's SM count gives the shape no half tiles after whole ones")
    kernel_id = abi.b200_tf32_kernel_from_name(b"pair_relu")
    assert kernel_id > 0
    g = torch.Generator().manual_seed(k)
    a = torch.randint(-3, 4, (m, k), generator=g).float()
    b = torch.randint(-3, 4, (k, n), generator=g).float()
    c = torch.randint(-8, 9, (m, n), generator=g).float()
    status, d, _ = run(abi, kernel_id, a.cuda(), b.cuda(), c.cuda(), alpha=1.0, beta=0.5, epilogue=RELU)
    assert status == 0, abi.b200_status_string(status)
    expected = oracle.adaptive_gemm_fp64(a, b, c, 1.0, 0.5, "relu")
    torch.testing.assert_close(d.cpu(), expected, atol=0, rtol=0)
    assert_device_clean(abi)


# ------------------------------------------------ calls in a row, each reading what the last one wrote
# The tensor-core kernels are launched under programmatic stream serialization: a kernel may become
# resident while the one before it still runs, and waits for it before touching global memory. Six
# calls with nothing between them, each taking the previous output as its source C.


@pytest.mark.parametrize("alias,shape", [("narrow_relu", (256, 256, 96)), ("fast_relu", (640, 512, 160)), ("wide_relu", (512, 1024, 64)),
                                         ("medium_relu", (384, 768, 96)),
                                         ("pair_relu", (1024, 768, 128)), ("pair_mid_relu", (1024, 512, 192)),
                                         ("splitk_relu", (128, 256, 1024)), ("pair_splitk_relu", (512, 256, 1024)),
                                         ("swap_relu", (8, 512, 1024)), ("fallback_relu", (130, 132, 70))])
def test_calls_in_a_row_read_what_the_last_one_wrote(abi, alias, shape):
    kernel_id = abi.b200_tf32_kernel_from_name(alias.encode())
    assert kernel_id > 0
    m, n, k = shape
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randint(-2, 3, (m, k), generator=g).float()
    b = torch.randint(-2, 3, (k, n), generator=g).float()
    c = torch.randint(-8, 9, (m, n), generator=g).float()
    a_dev, b_dev = a.cuda(), b.cuda()
    outs = [c.cuda()] + [torch.full((m, n), float("nan"), device="cuda") for _ in range(6)]
    torch.cuda.synchronize()
    for i in range(6):   # nothing else enters the stream in between
        q = GemmProblem(m, n, k, a_dev.data_ptr(), b_dev.data_ptr(), outs[i].data_ptr(), outs[i + 1].data_ptr(), k, n, n, n,
                        1.0, 0.5, RELU, None)
        assert abi.b200_tf32_gemm_launch(kernel_id, ctypes.byref(q), current_stream_ptr()) == 0
    expected = c.double()
    product = a.double() @ b.double()
    for i in range(6):
        expected = torch.relu(product + 0.5 * expected)
    # Small whole numbers and halvings: every intermediate is exact in FP32.
    torch.testing.assert_close(outs[6].cpu().double(), expected, atol=0, rtol=0)
    assert_device_clean(abi)
