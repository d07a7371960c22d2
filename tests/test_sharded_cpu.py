"""The M-sharded GEMM's host logic with two gloo ranks on CPU: row plan,
column-major shard materialisation, per-rank product, all-gather of C. The GPU
operator is replaced by an FP32 CPU matmul; the sharding code is the shipped one."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, n: int, k: int, result_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cuda_ai_kernels import sharded

        a, b = oracle.ladder_inputs(m, n, k, seed=0)          # every rank derives the same global problem
        plan = sharded.shard_rows(m, world)
        first, rows = plan[rank]
        a_shard = sharded.column_major_shard(a.t(), first, rows)
        assert a_shard.shape == (rows, k) and (rows == 0 or a_shard.stride() == (1, rows))
        c_shard = sharded.sharded_gemm(a_shard, b, compute=lambda x, y: x @ y)
        full = sharded.all_gather_rows(c_shard, [count for _, count in plan])
        expected = oracle.gemm_fp64(a, b)
        err = (full - expected).abs().max().item()
        shard_err = (c_shard - expected[first:first + rows]).abs().max().item() if rows else 0.0
        result_queue.put((rank, full.shape == expected.shape, err, shard_err, oracle.sgemm_abs_tolerance(a, b)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m", [512, 384, 200])   # even split, uneven tile split, ragged tail
def test_two_rank_sharded_gemm_reassembles_the_full_product(m):
    world, n, k = 2, 96, 64
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, m, n, k, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, shape_ok, err, shard_err, tol in results:
        assert shape_ok and err <= tol and shard_err <= tol, (rank, err, shard_err, tol)


# ------------------------------------------------------------- failures, injected on the host
# A rank that skips a collective, a rank that reports a failure, a rank that never joins: each is
# simulated on the host with gloo ranks; the others must find out within their time-out.


def _skipping_worker(rank: int, world: int, port: int, result_queue, done):
    import time

    from cuda_ai_kernels import sharded

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sharded.init_distributed("gloo", timeout_s=5.0)
    try:
        shard = torch.full((4, 8), float(rank))
        # Step 1: everybody takes part.
        full = sharded.all_gather_rows(shard, [4] * world)
        assert full.shape == (4 * world, 8)
        # Step 2: rank 1 "forgets" the collective. Rank 0 must get an error, not block for ever.
        if rank == 1:
            done.wait(timeout=60)                 # stay alive (a dead peer would be a different failure)
            result_queue.put((rank, "skipped", 0.0))
            return
        t0 = time.monotonic()
        try:
            sharded.all_gather_rows(shard, [4] * world)
            outcome = "returned"
        except Exception as exc:  # noqa: BLE001
            outcome = f"raised {type(exc).__name__}"
        result_queue.put((rank, outcome, time.monotonic() - t0))
        done.set()
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001 - the group is already broken on the rank that timed out
            pass


def test_a_rank_that_skips_the_all_gather_makes_the_others_raise_within_the_timeout():
    ctx = mp.get_context("spawn")
    queue, done = ctx.Queue(), ctx.Event()
    port = _free_port()
    procs = [ctx.Process(target=_skipping_worker, args=(r, 2, port, queue, done)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        results = dict((rank, (outcome, seconds)) for rank, outcome, seconds in (queue.get(timeout=90) for _ in procs))
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    outcome, seconds = results[0]
    assert outcome.startswith("raised"), results
    assert seconds < 30.0, results                # the 5 s time-out, not an endless wait
    assert results[1][0] == "skipped"


def _agreeing_worker(rank: int, world: int, port: int, result_queue):
    from cuda_ai_kernels import sharded

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sharded.init_distributed("gloo", timeout_s=20.0)
    try:
        barriers = 0
        verdicts = []
        for step in range(3):
            ok = not (rank == 1 and step == 1)    # rank 1's work fails in step 1
            agreed = sharded.all_ranks_ok(ok)
            verdicts.append(agreed)
            if not agreed:
                break                             # nobody enqueues the device-side barrier of this step
            barriers += 1
        result_queue.put((rank, verdicts, barriers))
    finally:
        dist.destroy_process_group()


def test_ranks_agree_on_the_host_before_a_device_barrier():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_agreeing_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    for rank, verdicts, barriers in results:
        assert verdicts == [True, False] and barriers == 1, (rank, verdicts, barriers)


def _lonely_worker(port: int, result_queue):
    import time

    from cuda_ai_kernels import sharded

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="2")
    t0 = time.monotonic()
    try:
        sharded.init_distributed("gloo", timeout_s=3.0)
        outcome = "joined"
    except Exception as exc:  # noqa: BLE001
        outcome = f"raised {type(exc).__name__}"
    result_queue.put((outcome, time.monotonic() - t0))


def test_set_up_gives_up_when_a_rank_never_joins():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    proc = ctx.Process(target=_lonely_worker, args=(_free_port(), queue))
    proc.start()
    try:
        outcome, seconds = queue.get(timeout=90)
    finally:
        proc.join(timeout=30)
        if proc.is_alive():
            proc.terminate()
    assert outcome.startswith("raised") and seconds < 45.0, (outcome, seconds)


def test_column_major_shard_rejects_views():
    from cuda_ai_kernels import sharded

    storage = torch.randn(8, 16)
    with pytest.raises(ValueError):
        sharded.column_major_shard(storage.t(), 0, 4)
    shard = sharded.column_major_shard(storage, 4, 8)
    assert torch.equal(shard, storage.t()[4:12]) and shard.stride() == (1, 8)


def test_shard_rows_python_wrapper():
    from cuda_ai_kernels import sharded

    assert sharded.shard_rows(32768, 8) == [(i * 4096, 4096) for i in range(8)]
    assert sharded.shard_rows(384, 2) == [(0, 256), (256, 128)]
    with pytest.raises(ValueError):
        sharded.shard_rows(128, 0)


def test_peer_row_pointers_of_the_fused_all_gather():
    from cuda_ai_kernels import sharded

    bases = [0x1000_0000, 0x2000_0000, 0x3000_0000, 0x4000_0000]
    plan = sharded.shard_rows(1024, 4)
    for rank, (first, _) in enumerate(plan):
        ptrs = sharded.peer_row_pointers(bases, rank, first, n=512)
        assert len(ptrs) == 3 and bases[rank] + first * 512 * 4 not in ptrs
        assert ptrs == [b + first * 512 * 4 for r, b in enumerate(bases) if r != rank]
        assert all(p % 16 == 0 for p in ptrs)
    assert sharded.peer_row_pointers([0x1000], 0, 0, 128) == []      # one rank: nothing to fan out to
    with pytest.raises(ValueError):
        sharded.peer_row_pointers(bases, 4, 0, 512)
    with pytest.raises(ValueError):
        sharded.peer_row_pointers(list(range(1, 10)), 0, 0, 512)       # nine ranks exceed the kernels' seven peers
    with pytest.raises(ValueError):
        sharded.peer_row_pointers(bases, 0, -128, 512)
