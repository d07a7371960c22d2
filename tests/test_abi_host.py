"""Host-side behaviour of libb200_kernels.so: it loads without a GPU, exports
every symbol the header declares, and its pure-host entry points (name tables,
tile table, validation, registry, compatibility test, shard planner) behave as
the reference interfaces they replace. No kernel is launched here."""
import ctypes
import re
from pathlib import Path

import pytest

from conftest import REPO, GemmProblem, KernelMeta

OK, MISALIGNED, INVALID_PROBLEM, NOT_SUPPORTED, INVALID_ARGUMENT = 0, 1, 2, 3, 4

LADDER = [
    ("naive", (16, 16, 1), 0), ("block_tile", (16, 16, 8), 0),
    ("block_tile_float4_16x16", (16, 16, 8), 1), ("block_tile_float4_16x32", (16, 32, 8), 1),
    ("block_tile_float4_32x32", (32, 32, 8), 1), ("thread_tile_4x4", (128, 128, 8), 1),
    ("thread_tile_4x8", (128, 128, 8), 1), ("thread_tile_8x8", (128, 128, 8), 1),
    ("thread_tile_8x8_warp4x8", (128, 128, 8), 1), ("warp_tile", (128, 128, 8), 1),
    ("prefetch_smem", (128, 128, 8), 1), ("prefetch_reg", (128, 128, 8), 1), ("split_k", (128, 128, 16), 1),
]


def declared_functions():
    header = (REPO / "include" / "b200_kernels.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header)))


def test_every_declared_symbol_is_exported(abi):
    names = declared_functions()
    assert len(names) >= 17
    for name in names:
        assert hasattr(abi, name), f"{name} is declared in b200_kernels.h but not exported"


def test_status_strings_match_the_dispatcher_vocabulary(abi):
    assert abi.b200_status_string(OK) == b"Success"
    assert abi.b200_status_string(MISALIGNED) == b"Error Misaligned Operand"
    assert abi.b200_status_string(INVALID_PROBLEM) == b"Error Invalid Problem"
    assert abi.b200_status_string(NOT_SUPPORTED) == b"Error Not Supported"
    assert abi.b200_status_string(12345).startswith(b"Error")
    assert b"sm_100a" in abi.b200_build_info()


def test_ladder_names_and_tiles_follow_the_stage_table(abi):
    from cuda_ai_kernels.gemm_stages import GEMM_STAGES

    hand_written = [(name, tile) for _, name, tile in GEMM_STAGES if name != "cublas"]
    assert [(n, t) for n, t, _ in LADDER] == hand_written
    for impl, (name, tile, vectorized) in enumerate(LADDER):
        assert abi.b200_sgemm_impl_name(impl) == name.encode()
        assert abi.b200_sgemm_impl_from_name(name.encode()) == impl
        bm, bn, bk, vec = (ctypes.c_int() for _ in range(4))
        assert abi.b200_sgemm_tile(impl, bm, bn, bk, vec) == OK
        assert (bm.value, bn.value, bk.value) == tile and vec.value == vectorized
    assert abi.b200_sgemm_impl_name(len(LADDER)) is None
    assert abi.b200_sgemm_impl_from_name(b"thread_tile") == 5  # alias of the 4x4 variant
    assert abi.b200_sgemm_impl_from_name(b"cublas") == -1      # library baseline lives in the caller
    assert abi.b200_sgemm_tile(99, None, None, None, None) == INVALID_ARGUMENT


@pytest.mark.parametrize("impl,name", [(i, row[0]) for i, row in enumerate(LADDER)])
def test_sgemm_check_order_and_codes(abi, impl, name):
    bm, bn, bk = LADDER[impl][1]
    aligned, odd = 0x7F0000000000, 0x7F0000000004
    check = abi.b200_sgemm_check
    assert check(impl, aligned, aligned, bm, bn, 2 * bk * 8) == OK
    for m, n, k in [(0, bn, bk), (bm, 0, bk), (bm, bn, 0), (-bm, bn, bk)]:
        assert check(impl, aligned, aligned, m, n, k) == INVALID_ARGUMENT
    assert check(impl, aligned, aligned, bm - 1, bn, bk * 8) == INVALID_PROBLEM
    assert check(impl, aligned, aligned, bm, bn + 1, bk * 8) == INVALID_PROBLEM
    if bk > 1:
        assert check(impl, aligned, aligned, bm, bn, bk * 8 - 1) == INVALID_PROBLEM
    assert check(impl, aligned, aligned, bm * 65536, bn, bk * 8) == INVALID_PROBLEM  # grid.y limit
    expected = MISALIGNED if LADDER[impl][2] else OK
    assert check(impl, odd, aligned, bm, bn, bk * 8) == expected
    assert check(impl, aligned, odd, bm, bn, bk * 8) == expected
    # Sizes are judged before alignment.
    assert check(impl, odd, odd, bm + 1, bn, bk * 8) == INVALID_PROBLEM


def test_split_k_needs_two_k_slices_of_eight(abi):
    impl = abi.b200_sgemm_impl_from_name(b"split_k")
    for k in (8, 24, 40):
        assert abi.b200_sgemm_check(impl, 0, 0, 128, 128, k) == INVALID_PROBLEM
    for k in (16, 32, 48):
        assert abi.b200_sgemm_check(impl, 0, 0, 128, 128, k) == OK


def registry(abi):
    entries = []
    for i in range(abi.b200_tf32_registry_size()):
        meta = KernelMeta()
        assert abi.b200_tf32_registry_entry(i, ctypes.byref(meta)) == OK
        entries.append(meta)
    return entries


def test_registry_keeps_the_reference_ids_aliases_and_order(abi):
    entries = registry(abi)
    # Shape-gated configurations that exist only here come first, then the
    # reference's eight as one block in the reference's order, then the entries
    # that close the dispatch order for GELU (which the reference never runs).
    ids = [e.id for e in entries]
    first, last = ids.index(2), ids.index(9)
    assert ids[first:last + 1] == [2, 3, 4, 5, 6, 7, 8, 9]
    assert all(i >= 16 for i in ids[:first] + ids[last + 1:])
    assert all(e.epilogue == 2 for e in entries[last + 1:])
    reference = [e for e in entries if e.id < 16]
    head = [(e.id, e.alias.decode(), e.epilogue, e.alignment_a) for e in reference]
    assert head == [
        (2, "fast", 0, 4), (3, "fallback", 0, 1), (4, "fast_mwarp", 0, 4), (5, "fallback_mwarp", 0, 1),
        (6, "fast_stage3", 0, 4), (7, "fast_stage2", 0, 4), (8, "fast_relu", 1, 4), (9, "fallback_relu", 1, 1),
    ]
    skinny = [e for e in entries if e.alias.decode().startswith("skinny")]
    assert [(e.id, e.epilogue, e.tile_m, e.tile_n, e.alignment_a, e.alignment_b) for e in skinny] == [
        (27, 0, 16, 128, 1, 4), (28, 1, 16, 128, 1, 4), (29, 2, 16, 128, 1, 4)]
    assert entries[:3] == skinny or [e.id for e in entries[:3]] == [27, 28, 29]   # tried first, behind an M <= 16 gate
    for e in entries:
        assert abi.b200_tf32_kernel_from_name(e.alias) == e.id
        assert abi.b200_tf32_kernel_from_name(e.name) == e.id
        if e in skinny:
            continue
        if e.alias.decode().startswith("swap"):      # D^T = B^T A^T: the MMA's M side runs along N
            assert (e.tile_m, e.tile_n, e.inst_m, e.inst_n, e.inst_k, e.supports_split_k) == (64, 128, 128, 64, 8, 1)
            continue
        assert e.tile_m in (128, 256) and e.inst_m == e.tile_m and e.inst_k == 8 and e.tile_k == 32
        assert e.tile_n in (32, 64, 96, 128, 160, 192, 224, 256) and e.inst_n == e.tile_n
        assert (e.tile_m == 256) == e.alias.decode().startswith("pair")   # 256 rows only as a CTA pair
        assert e.alignment_a == e.alignment_b == e.alignment_c and e.alignment_a in (1, 4)
        assert abi.b200_tf32_kernel_from_name(e.alias) == e.id
        assert abi.b200_tf32_kernel_from_name(e.name) == e.id
    assert len({e.id for e in entries}) == len(entries)
    assert abi.b200_tf32_registry_entry(len(entries), ctypes.byref(KernelMeta())) == INVALID_ARGUMENT


def test_kernel_name_parser(abi):
    parse = abi.b200_tf32_kernel_from_name
    assert parse(b"auto") == 0 and parse(b"cublas") == 1
    assert parse(b"fast_Relu") == parse(b"fast_relu") == 8
    assert parse(b"fallback_Relu") == parse(b"fallback_relu") == 9
    assert parse(b"unknown") == -1 and parse(b"") == -1


def problem(m, n, k, a=0x1000, b=0x2000, c=0x3000, d=0x4000, beta=0.0, epilogue=0, lda=None, ldb=None):
    return GemmProblem(m, n, k, a, b, c, d, lda or k, ldb or n, n, n, 1.0, beta, epilogue)


def test_can_implement_alignment_rules(abi):
    fast, fallback, fast_relu = 2, 3, 8
    ok = problem(33, 68, 20)
    assert abi.b200_tf32_can_implement(fast, ctypes.byref(ok)) == OK           # any M
    for bad in (problem(33, 65, 20), problem(33, 68, 17)):                      # N % 4, K % 4
        assert abi.b200_tf32_can_implement(fast, ctypes.byref(bad)) == MISALIGNED
        assert abi.b200_tf32_can_implement(fallback, ctypes.byref(bad)) == OK
    for field in ("a", "b", "c", "d"):                                         # 16-byte pointers
        shifted = problem(128, 128, 64, **{field: 0x5004})
        assert abi.b200_tf32_can_implement(fast, ctypes.byref(shifted)) == MISALIGNED
        assert abi.b200_tf32_can_implement(fallback, ctypes.byref(shifted)) == OK
    assert abi.b200_tf32_can_implement(fast, ctypes.byref(problem(1, 4, 4))) == OK
    assert abi.b200_tf32_can_implement(fallback, ctypes.byref(problem(1, 1, 1))) == OK
    # Epilogue kind is part of the entry.
    assert abi.b200_tf32_can_implement(fast, ctypes.byref(problem(128, 128, 64, epilogue=1))) == NOT_SUPPORTED
    assert abi.b200_tf32_can_implement(fast_relu, ctypes.byref(problem(128, 128, 64, epilogue=1))) == OK
    assert abi.b200_tf32_can_implement(fast_relu, ctypes.byref(problem(128, 128, 64, epilogue=0))) == NOT_SUPPORTED
    # Malformed problems.
    gelu = abi.b200_tf32_kernel_from_name(b"fast_gelu")
    assert gelu == 25 and abi.b200_tf32_can_implement(gelu, ctypes.byref(problem(128, 128, 64, epilogue=2))) == OK
    assert abi.b200_tf32_can_implement(gelu, ctypes.byref(problem(128, 128, 64, epilogue=1))) == NOT_SUPPORTED
    assert abi.b200_tf32_can_implement(fast, ctypes.byref(problem(128, 128, 64, epilogue=3))) == INVALID_ARGUMENT
    assert abi.b200_tf32_can_implement(fast, ctypes.byref(problem(0, 128, 64))) == INVALID_ARGUMENT
    assert abi.b200_tf32_can_implement(fast, ctypes.byref(problem(128, 128, 64, c=0, beta=1.0))) == INVALID_ARGUMENT
    assert abi.b200_tf32_can_implement(fast, ctypes.byref(problem(128, 128, 64, lda=60))) == INVALID_ARGUMENT
    assert abi.b200_tf32_can_implement(1234, ctypes.byref(ok)) == INVALID_ARGUMENT


def test_missing_source_aliases_destination_for_alignment(abi):
    q = problem(128, 128, 64, c=0)
    assert abi.b200_tf32_can_implement(2, ctypes.byref(q)) == OK
    q = problem(128, 128, 64, c=0, d=0x4004)
    assert abi.b200_tf32_can_implement(2, ctypes.byref(q)) == MISALIGNED


def shard(abi, m, parts, granule=128):
    begin = (ctypes.c_int64 * parts)()
    count = (ctypes.c_int64 * parts)()
    assert abi.b200_shard_rows(m, parts, granule, begin, count) == OK
    return list(begin), list(count)


@pytest.mark.parametrize("m,parts", [(32768, 1), (32768, 2), (32768, 4), (32768, 8), (4096, 8), (1024, 3),
                                     (128, 8), (1000, 4), (0, 2), (77, 3)])
def test_shard_rows_partitions_exactly(abi, m, parts):
    begin, count = shard(abi, m, parts)
    assert sum(count) == m and begin[0] == 0
    for p in range(1, parts):
        assert begin[p] == begin[p - 1] + count[p - 1]
    full = [c for c in count if c % 128 == 0]
    assert len(full) >= parts - 1                      # at most one ragged part
    whole = [c // 128 for c in count]
    assert max(whole) - min(whole) <= 1                # balanced to one tile


def test_shard_rows_rejects_bad_arguments(abi):
    buf = (ctypes.c_int64 * 2)()
    assert abi.b200_shard_rows(128, 0, 128, buf, buf) == INVALID_ARGUMENT
    assert abi.b200_shard_rows(128, 2, 0, buf, buf) == INVALID_ARGUMENT
    assert abi.b200_shard_rows(-1, 2, 128, buf, buf) == INVALID_ARGUMENT
    assert abi.b200_shard_rows(128, 2, 128, None, buf) == INVALID_ARGUMENT


def test_device_launch_entry_points_reject_null_and_bad_ids_without_a_gpu(abi):
    assert abi.b200_sgemm(0, None, None, None, 16, 16, 1, None) == INVALID_ARGUMENT
    assert abi.b200_sgemm(99, 0x1000, 0x1000, 0x1000, 16, 16, 1, None) == INVALID_ARGUMENT
    assert abi.b200_rmsnorm(7, 0x1000, 0x1000, 0x1000, 1, 4, 1e-6, None) == INVALID_ARGUMENT
    assert abi.b200_rmsnorm(1, 0x1000, 0x1000, 0x1000, 1, 8192, 1e-6, None) == NOT_SUPPORTED  # cache_x limit
    assert abi.b200_softmax(3, 0x1000, 0x1000, 1, 4, None) == INVALID_ARGUMENT
    assert abi.b200_softmax(0, 0x1000, 0x1000, 0, 4, None) == OK   # nothing to do
    q = problem(128, 128, 64)
    assert abi.b200_tf32_gemm_dispatch(1, ctypes.byref(q), None, None) == INVALID_ARGUMENT  # cublas id
    mismatched = problem(4, 4, 4, epilogue=1)
    assert abi.b200_tf32_gemm_dispatch(2, ctypes.byref(mismatched), None, None) == NOT_SUPPORTED
    misaligned = problem(33, 65, 20)
    assert abi.b200_tf32_gemm_dispatch(2, ctypes.byref(misaligned), None, None) == NOT_SUPPORTED


def test_gather_entry_points_validate_on_the_host(abi):
    """Argument checks of the fused all-gather entries that return before any CUDA call."""
    from conftest import GemmProblem

    peers = (ctypes.c_void_p * 8)(*[0x1000 * (i + 1) for i in range(8)])
    a = b = c = ctypes.c_void_p(0x10000)
    # Null operands, too many peers, a null peer, a negative count.
    assert abi.b200_sgemm_gather(11, None, b, c, peers, 1, 128, 128, 16, None) == INVALID_ARGUMENT
    assert abi.b200_sgemm_gather(11, a, b, c, peers, 8, 128, 128, 16, None) == INVALID_ARGUMENT
    assert abi.b200_sgemm_gather(11, a, b, c, None, 1, 128, 128, 16, None) == INVALID_ARGUMENT
    assert abi.b200_sgemm_gather(11, a, b, c, peers, -1, 128, 128, 16, None) == INVALID_ARGUMENT
    holes = (ctypes.c_void_p * 2)(0x1000, None)
    assert abi.b200_sgemm_gather(11, a, b, c, holes, 2, 128, 128, 16, None) == INVALID_ARGUMENT
    # Shape rules are the ladder's; entries that cannot fan out are refused; peers must allow 128-bit stores.
    assert abi.b200_sgemm_gather(11, a, b, c, peers, 1, 100, 128, 16, None) == 2
    assert abi.b200_sgemm_gather(12, a, b, c, peers, 1, 128, 128, 16, None) == 3      # split_k
    assert abi.b200_sgemm_gather(5, a, b, c, peers, 1, 128, 128, 16, None) == 3       # a ladder stage
    odd = (ctypes.c_void_p * 1)(0x1004)
    assert abi.b200_sgemm_gather(11, a, b, c, odd, 1, 128, 128, 16, None) == 1
    q = GemmProblem(128, 128, 32, 0x10000, 0x20000, None, 0x30000, 32, 128, 128, 128, 1.0, 0.0, 0, None)
    assert abi.b200_tf32_gemm_dispatch_gather(0, ctypes.byref(q), peers, 8, None, None) == INVALID_ARGUMENT
    assert abi.b200_tf32_gemm_dispatch_gather(0, ctypes.byref(q), None, 2, None, None) == INVALID_ARGUMENT
    assert abi.b200_tf32_gemm_dispatch_gather(1, ctypes.byref(q), peers, 1, None, None) == INVALID_ARGUMENT  # cuBLAS id
