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
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import cuda_ai_kernels
        from cuda_ai_kernels import sharded

        a, b = oracle.ladder_inputs(m, n, k, seed=0)
        plan = sharded.shard_rows(m, world)
        first, rows = plan[rank]
        dev = torch.device("cuda", rank)
        a_shard = sharded.column_major_shard(a.t().contiguous().to(dev), first, rows)
        b_dev = b.to(dev)
        expected = oracle.gemm_fp64(a, b)
        tol = oracle.sgemm_abs_tolerance(a, b)
        errors = {}
        for impl in ("prefetch_reg", "split_k"):
            c_shard = sharded.sharded_gemm(a_shard, b_dev, impl=impl)
            full = sharded.all_gather_rows(c_shard, [count for _, count in plan])
            errors[impl] = (full.cpu() - expected).abs().max().item()
        # TF32 path: a row slab of row-major A is already contiguous.
        a_rows = a[first:first + rows].contiguous().to(dev)
        d_shard = cuda_ai_kernels.adaptive_gemm(a_rows, b_dev)
        full = sharded.all_gather_rows(d_shard, [count for _, count in plan])
        rel = oracle.rel_frobenius(full, expected)
        queue.put((rank, errors, tol, rel))
    finally:
        dist.destroy_process_group()


def test_sharded_gemm_across_gpus():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = 128 * 3 * world, 512, 256
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, m, n, k, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, errors, tol, rel in results:
        assert all(err <= tol for err in errors.values()), (rank, errors, tol)
        assert rel <= oracle.TF32_REL_FROBENIUS, (rank, rel)
