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

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
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
        # Fused all-gather: the kernels' epilogues store every tile into every rank's copy of C.
        counts = [count for _, count in plan]
        gathered = sharded.GatheredOutput(m, n, plan)
        gathered.full.fill_(float("nan"))
        gathered.barrier()
        torch.cuda.synchronize()
        reference = sharded.all_gather_rows(sharded.sharded_gemm(a_shard, b_dev, impl="prefetch_reg"), counts)
        fused = sharded.sharded_gemm_gather(a_shard, b_dev, gathered, impl="prefetch_reg")
        gathered.barrier()
        torch.cuda.synchronize()
        errors["fused_fp32_vs_collective"] = 0.0 if torch.equal(fused, reference) else float("inf")
        errors["fused_fp32"] = (fused.cpu() - expected).abs().max().item()
        gathered.barrier()                       # nobody overwrites a copy that a peer is still comparing
        gathered.full.fill_(float("nan"))
        gathered.barrier()
        torch.cuda.synchronize()
        fused = sharded.sharded_adaptive_gemm_gather(a_rows, b_dev, gathered, epilogue="relu")
        gathered.barrier()
        torch.cuda.synchronize()
        rel_fused = oracle.rel_frobenius(fused, expected.relu())
        reference = sharded.all_gather_rows(cuda_ai_kernels.adaptive_gemm(a_rows, b_dev, epilogue="relu"), counts)
        errors["fused_tf32_vs_collective"] = 0.0 if torch.equal(fused, reference) else float("inf")
        gathered.barrier()
        queue.put((rank, errors, tol, max(rel, rel_fused)))
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
