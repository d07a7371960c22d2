"""M-sharded GEMM on real GPUs: one process per GPU over NCCL, each rank runs
the FP32 SIMT and the TF32 kernels on its rows, the optional all-gather
reassembles C. Skipped with fewer than two GPUs (the CPU suite covers the host
logic with gloo)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from oracle import oracle

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, queue):
    """One rank. Work between two device-side barriers runs under try/except; before every barrier
    the ranks agree on the host (gloo) that all of them got there, and skip it otherwise, so no
    rank waits on the GPU for a partner that raised."""
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    host_group = dist.new_group(backend="gloo")
    failure = [None]
    try:
        import cuda_ai_kernels
        from cuda_ai_kernels import sharded

        def phase(fn):
            """Runs fn unless an earlier phase failed somewhere; True when every rank is still fine."""
            if failure[0] is None:
                try:
                    fn()
                except Exception as exc:  # noqa: BLE001 - reported to the parent below
                    failure[0] = f"{type(exc).__name__}: {exc}"
            return sharded.all_ranks_ok(failure[0] is None, host_group)

        state = {}
        errors = {}

        def setup():
            a, b = oracle.ladder_inputs(m, n, k, seed=0)
            plan = sharded.shard_rows(m, world)
            first, rows = plan[rank]
            dev = torch.device("cuda", rank)
            state.update(a=a, b=b, plan=plan, counts=[count for _, count in plan], dev=dev,
                         a_shard=sharded.column_major_shard(a.t().contiguous().to(dev), first, rows), b_dev=b.to(dev),
                         a_rows=a[first:first + rows].contiguous().to(dev),   # TF32 path: a row slab is contiguous
                         expected=oracle.gemm_fp64(a, b), tol=oracle.sgemm_abs_tolerance(a, b))

        def unfused():
            for impl in ("prefetch_reg", "split_k"):
                c_shard = sharded.sharded_gemm(state["a_shard"], state["b_dev"], impl=impl)
                full = sharded.all_gather_rows(c_shard, state["counts"])
                errors[impl] = (full.cpu() - state["expected"]).abs().max().item()
            d_shard = cuda_ai_kernels.adaptive_gemm(state["a_rows"], state["b_dev"])
            full = sharded.all_gather_rows(d_shard, state["counts"])
            state["rel"] = oracle.rel_frobenius(full, state["expected"])

        def allocate():
            # Fused all-gather: the kernels' epilogues store every tile into every rank's copy of C.
            state["gathered"] = sharded.GatheredOutput(m, n, state["plan"])
            state["gathered"].full.fill_(float("nan"))

        def fused_fp32():
            state["reference"] = sharded.all_gather_rows(
                sharded.sharded_gemm(state["a_shard"], state["b_dev"], impl="prefetch_reg"), state["counts"])
            state["fused"] = sharded.sharded_gemm_gather(state["a_shard"], state["b_dev"], state["gathered"],
                                                         impl="prefetch_reg")

        def compare_fp32():
            state["gathered"].check()
            fused = state["fused"]
            errors["fused_fp32_vs_collective"] = 0.0 if torch.equal(fused, state["reference"]) else float("inf")
            errors["fused_fp32"] = (fused.cpu() - state["expected"]).abs().max().item()

        def refill():
            torch.cuda.synchronize()
            state["gathered"].full.fill_(float("nan"))

        def fused_tf32():
            state["fused"] = sharded.sharded_adaptive_gemm_gather(state["a_rows"], state["b_dev"], state["gathered"],
                                                                  epilogue="relu")

        def compare_tf32():
            state["gathered"].check()
            fused = state["fused"]
            state["rel"] = max(state["rel"], oracle.rel_frobenius(fused, state["expected"].relu()))
            reference = sharded.all_gather_rows(
                cuda_ai_kernels.adaptive_gemm(state["a_rows"], state["b_dev"], epilogue="relu"), state["counts"])
            errors["fused_tf32_vs_collective"] = 0.0 if torch.equal(fused, reference) else float("inf")

        # Each entry: (work, barrier after it?). A barrier is enqueued only when every rank agreed.
        for work, barrier_after in ((setup, False), (unfused, False), (allocate, True), (fused_fp32, True),
                                    (compare_fp32, True),   # nobody overwrites a copy a peer is still comparing
                                    (refill, True), (fused_tf32, True), (compare_tf32, True)):
            if not phase(work):
                break
            if barrier_after:
                state["gathered"].barrier()
        if failure[0] is None and sharded.all_ranks_ok(True, host_group):
            torch.cuda.synchronize()
            queue.put((rank, errors, state["tol"], state["rel"], None))
        else:
            queue.put((rank, errors, 0.0, 0.0, failure[0] or "another rank failed"))
    finally:
        torch.cuda.synchronize()
        dist.destroy_process_group()


def test_sharded_gemm_across_gpus():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    # K of three 64-deep blocks (the last one ragged): too short for the plain GEMM to share a tile's K
    # range over a cluster, so the fused and the unfused kernels add in the same order and their
    # results can be compared bit for bit.
    m, n, k = 128 * 3 * world, 512, 160
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, m, n, k, queue)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = [queue.get(timeout=300) for _ in procs]
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        # No child outlives the test, whatever happened above.
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
            if p.is_alive():
                p.kill()
    for rank, errors, tol, rel, failure in results:
        assert failure is None, (rank, failure)
        assert all(err <= tol for err in errors.values()), (rank, errors, tol)
        assert rel <= oracle.TF32_REL_FROBENIUS, (rank, rel)


# ------------------------------------------------- the barrier kernel on a single GPU
# Two flag arrays on one GPU stand in for two ranks. Only ONE barrier kernel runs per case (two
# launches that wait for each other must never share a GPU): the partner's flag is either written
# beforehand by the host or never written at all.


def _barrier(abi, arrays, rank, epoch, polls):
    import ctypes

    from conftest import current_stream_ptr

    ptrs = (ctypes.c_void_p * len(arrays))(*[t.data_ptr() for t in arrays])
    return abi.b200_peer_barrier(ptrs, len(arrays), rank, epoch, polls, current_stream_ptr())


def test_peer_barrier_signals_and_passes_when_the_partner_has_arrived(abi):
    from conftest import assert_device_clean

    arrays = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(3)]
    arrays[0][1] = 5            # "rank 1 reached step 5"
    arrays[0][2] = 6            # "rank 2 is already a step ahead"
    torch.cuda.synchronize()
    assert _barrier(abi, arrays, 0, 5, 1 << 16) == 0
    torch.cuda.synchronize()
    assert arrays[1][0].item() == 5 and arrays[2][0].item() == 5      # rank 0 told both partners
    assert arrays[1][1].item() == 0 and arrays[0][0].item() == 0      # and touched nothing else
    assert_device_clean(abi)
    assert _barrier(abi, arrays[:1], 0, 1, 1) == 0                    # a world of one has nobody to wait for
    assert_device_clean(abi)


def test_peer_barrier_gives_up_when_the_partner_never_arrives(abi):
    import ctypes

    from conftest import current_stream_ptr

    arrays = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    arrays[0][1] = 3            # the partner stopped at step 3
    torch.cuda.synchronize()
    assert _barrier(abi, arrays, 0, 4, 2048) == 0                     # 2048 polls: about a millisecond
    torch.cuda.synchronize()                                          # returns: the kernel ended by itself
    word = ctypes.c_uint32(0)
    assert abi.b200_device_status_read(ctypes.byref(word), ctypes.c_void_p(current_stream_ptr())) == 6
    assert word.value == 1 << 8
    assert abi.b200_device_status_read(ctypes.byref(word), ctypes.c_void_p(current_stream_ptr())) == 0
    assert arrays[1][0].item() == 4                                   # it did signal before waiting
    for bad in ((arrays, 2, 1, 16), (arrays, 0, 1, 0), ([], 0, 1, 16)):
        assert _barrier(abi, *bad) == 4


# ---------------------------------------------------- fan-out on a single GPU
# The fused all-gather entries only ever STORE to their extra destinations, so
# buffers on the same GPU stand in for peers: every destination must receive
# exactly what the local output receives.


def test_sgemm_gather_fans_out_every_tile(abi):
    import ctypes

    from conftest import assert_device_clean, current_stream_ptr

    m, n, k = 256, 384, 192
    a, b = oracle.ladder_inputs(m, n, k, seed=3)
    a_dev, b_dev = oracle.to_device_preserving_strides(a, "cuda"), b.cuda()
    expected = oracle.gemm_fp64(a, b)
    for impl in (10, 11):                                             # prefetch_smem, prefetch_reg
        plain = torch.empty(m, n, device="cuda")
        assert abi.b200_sgemm(impl, a_dev.data_ptr(), b_dev.data_ptr(), plain.data_ptr(), m, n, k, current_stream_ptr()) == 0
        for n_peers in (0, 1, 3, 7):
            # Rows [m, 2m) of taller buffers: the position of a middle rank in a gathered matrix.
            buffers = [torch.full((3 * m, n), float("nan"), device="cuda") for _ in range(n_peers + 1)]
            views = [buf[m:2 * m] for buf in buffers]
            peers = (ctypes.c_void_p * 7)(*[v.data_ptr() for v in views[1:]])
            status = abi.b200_sgemm_gather(impl, a_dev.data_ptr(), b_dev.data_ptr(), views[0].data_ptr(), peers, n_peers,
                                           m, n, k, current_stream_ptr())
            assert status == 0, abi.b200_status_string(status)
            for buf, view in zip(buffers, views):
                assert torch.equal(view, plain)
                assert bool(torch.isnan(buf[:m]).all()) and bool(torch.isnan(buf[2 * m:]).all())   # nothing outside the rows
    assert float((plain.cpu() - expected).abs().max()) <= oracle.sgemm_abs_tolerance(a, b)
    assert_device_clean(abi)


@pytest.mark.parametrize("kernel,shape", [
    (20, (512, 512, 128)),     # CTA pair
    (16, (256, 512, 96)),      # 128 x 256 tiles
    (18, (200, 264, 100)),     # 128 x 64 tiles, ragged
    (8, (130, 136, 64)),       # 128 x 128 + ReLU
    (3, (33, 65, 17)),         # generic loader, scalar epilogue
    (30, (64, 256, 1024)),     # split-K cluster
    (36, (12, 264, 512)),      # operands swapped, K split over a cluster
    (39, (300, 264, 160)),     # CTA pair, 256 x 128 tiles, two issuers, ragged
    (42, (300, 200, 1024)),    # CTA pairs with K split over the cluster
    (57, (200, 136, 100)),     # 128 x 32 tiles: one chunk, the second epilogue warp of a quarter idle
    (48, (200, 296, 100)),     # 128 x 96 tiles, two MMA threads, three chunks on two epilogue warps
    (51, (130, 488, 64)),      # 128 x 160 tiles
    (45, (256, 388, 96)),      # 128 x 192 tiles
    (54, (200, 676, 64)),      # 128 x 224 tiles
])
def test_tf32_gather_fans_out_every_element(abi, kernel, shape):
    import ctypes

    from conftest import GemmProblem, assert_device_clean, current_stream_ptr

    m, n, k = shape
    a, b, c = oracle.adaptive_inputs(m, n, k, seed=k)
    a_dev, b_dev, c_dev = a.cuda(), b.cuda(), c.cuda()
    epilogue = 1 if kernel == 8 else 0
    bias = torch.linspace(-1.0, 1.0, n, device="cuda")
    buffers = [torch.full((m + 2, n), float("nan"), device="cuda") for _ in range(4)]
    views = [buf[1:m + 1] for buf in buffers]                          # odd row offset: alignment follows n
    q = GemmProblem(m, n, k, a_dev.data_ptr(), b_dev.data_ptr(), c_dev.data_ptr(), views[0].data_ptr(), k, n, n, n,
                    0.75, 0.25, epilogue, bias.data_ptr())
    peers = (ctypes.c_void_p * 7)(*[v.data_ptr() for v in views[1:]])
    chosen = ctypes.c_int(-1)
    status = abi.b200_tf32_gemm_dispatch_gather(kernel, ctypes.byref(q), peers, 3, ctypes.byref(chosen), current_stream_ptr())
    assert status == 0 and chosen.value == kernel, abi.b200_status_string(status)
    name = ("bias_relu" if epilogue else "bias")
    expected = oracle.adaptive_gemm_fp64(a, b, c, 0.75, 0.25, name, bias=bias.cpu())
    assert oracle.rel_frobenius(views[0], expected) <= oracle.TF32_REL_FROBENIUS
    for buf, view in zip(buffers, views):
        assert torch.equal(view, views[0])
        assert bool(torch.isnan(buf[0]).all()) and bool(torch.isnan(buf[m + 1]).all())
    assert_device_clean(abi)


def test_skinny_entries_do_not_fan_out(abi):
    import ctypes

    from conftest import GemmProblem, current_stream_ptr

    a, b, _ = oracle.adaptive_inputs(4, 256, 128)
    a_dev, b_dev = a.cuda(), b.cuda()
    outs = [torch.full((4, 256), float("nan"), device="cuda") for _ in range(2)]
    q = GemmProblem(4, 256, 128, a_dev.data_ptr(), b_dev.data_ptr(), None, outs[0].data_ptr(), 128, 256, 256, 256,
                    1.0, 0.0, 0, None)
    peers = (ctypes.c_void_p * 7)(outs[1].data_ptr())
    assert abi.b200_tf32_gemm_dispatch_gather(27, ctypes.byref(q), peers, 1, None, current_stream_ptr()) == 3
    chosen = ctypes.c_int(-1)
    assert abi.b200_tf32_gemm_dispatch_gather(0, ctypes.byref(q), peers, 1, ctypes.byref(chosen), current_stream_ptr()) == 0
    assert chosen.value not in (27, 28, 29) and torch.equal(outs[0], outs[1])
    assert oracle.rel_frobenius(outs[0], oracle.adaptive_gemm_fp64(a, b)) <= oracle.TF32_REL_FROBENIUS
