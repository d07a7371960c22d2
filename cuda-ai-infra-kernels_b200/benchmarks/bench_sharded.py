"""M-sharded large GEMM across the GPUs of one node (strong scaling).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 --master-port P \
        cuda-ai-infra-kernels_b200/benchmarks/bench_sharded.py [--m 32768 --n 8192 --k 8192] [--steps 10] [--warmup 3]
    python cuda-ai-infra-kernels_b200/benchmarks/bench_sharded.py          # G = 1

The benchmark configuration: M = 32768, N = K = 8192, FP32 N(0,1) inputs. Rank r
owns rows [r*M/G, (r+1)*M/G) of A (a column-major shard for the FP32 SIMT path,
a contiguous row slab for the TF32 path), B is replicated, C stays sharded: no
collective on the data path. Timing: CUDA events around `steps` calls on each
rank between barriers, MAX over ranks. Gathering C on every rank is timed three
ways: the NCCL all-gather alone, GEMM followed by that all-gather, and the fused
kernels whose epilogues store every tile into every rank's copy of C over
NVLink (`sharded.sharded_gemm_gather`), each step closed by the device-side
barrier that makes the copies readable. Every rank checks sampled rows of its
shard against the FP64 oracle expression on the CPU before anything is timed,
and the fused result against the collective one bit for bit. Rank 0 prints one
JSON line; scaling = T(1) / (G * T(G)) is left to the reader of the per-G lines.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "python"))


def timed_ms(fn, steps: int) -> float:
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / steps


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--m", type=int, default=32768)
    parser.add_argument("--n", type=int, default=8192)
    parser.add_argument("--k", type=int, default=8192)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--sgemm-impl", default="prefetch_reg")
    args = parser.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    import cuda_ai_kernels as pkg
    from cuda_ai_kernels import _C, sharded  # noqa: F401

    plan = sharded.shard_rows(args.m, world)
    first, rows = plan[rank]
    # Same global problem on every rank: row r of A comes from a generator
    # seeded with r's 1024-row block, B from seed 0.
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    b = torch.randn(args.k, args.n, device=dev, generator=g)
    a_rows = torch.empty(rows, args.k, device=dev)
    for block in range(first // 1024, (first + rows + 1023) // 1024):
        g.manual_seed(1000 + block)
        chunk = torch.randn(1024, args.k, device=dev, generator=g)
        lo, hi = max(block * 1024, first), min((block + 1) * 1024, first + rows)
        a_rows[lo - first:hi - first] = chunk[lo - block * 1024:hi - block * 1024]
    a_colmajor = a_rows.t().contiguous().t()   # [rows, K] view of [K, rows] storage: the ladder's layout for this shard

    # Parity gate on sampled rows (a row of C depends on that row of A only).
    sample = torch.randperm(rows, device=dev, generator=g)[:48]
    expected = (a_rows[sample].cpu().double() @ b.cpu().double()).float()
    c_fp32 = pkg.gemm(a_colmajor, b, impl=args.sgemm_impl)
    tol = 1e-4 * args.k ** 0.5 * float(a_rows.abs().max()) * float(b.abs().max())
    err32 = (c_fp32[sample].cpu() - expected).abs().max().item()
    d_tf32 = pkg.adaptive_gemm(a_rows, b)
    rel_tf32 = float((d_tf32[sample].cpu().double() - expected.double()).norm() / expected.double().norm())
    if not (err32 <= tol and rel_tf32 <= 5e-3):
        raise SystemExit(f"rank {rank}: parity gate failed (fp32 err {err32:.3e} > {tol:.3e} or tf32 rel {rel_tf32:.3e})")
    tf32_kernel = _C.adaptive_gemm_last_kernel()
    del d_tf32

    def reduce_max(ms: float) -> float:
        if not distributed:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    results = {}
    for name, fn in (("fp32_simt", lambda: pkg.gemm(a_colmajor, b, impl=args.sgemm_impl)),
                     ("tf32", lambda: pkg.adaptive_gemm(a_rows, b))):
        for _ in range(args.warmup):
            fn()
        if distributed:
            dist.barrier()
        ms = reduce_max(timed_ms(fn, args.steps))
        results[name] = {"ms": ms, "tflops_total": 2.0 * args.m * args.n * args.k / ms / 1e9}

    gather = None
    fused = None
    if distributed:
        counts = [count for _, count in plan]
        for _ in range(2):
            sharded.all_gather_rows(c_fp32, counts)
        dist.barrier()
        ms = reduce_max(timed_ms(lambda: sharded.all_gather_rows(c_fp32, counts), 5))
        received = (args.m - rows) * args.n * 4
        gather = {"ms": ms, "received_gb_per_rank": received / 1e9, "gbs_per_rank": received / ms / 1e6}

        # GEMM + all-gather: two launches (kernel, then NCCL) against one fused kernel + barrier.
        out = sharded.GatheredOutput(args.m, args.n, plan)
        arms = {
            "fp32_simt_then_allgather": lambda: sharded.all_gather_rows(pkg.gemm(a_colmajor, b, impl=args.sgemm_impl), counts),
            "fp32_simt_fused": lambda: (sharded.sharded_gemm_gather(a_colmajor, b, out, impl=args.sgemm_impl), out.barrier()),
            "tf32_then_allgather": lambda: sharded.all_gather_rows(pkg.adaptive_gemm(a_rows, b), counts),
            "tf32_fused": lambda: (sharded.sharded_adaptive_gemm_gather(a_rows, b, out), out.barrier()),
        }
        # Parity of the fused result with the collective one, on every rank.
        reference = arms["fp32_simt_then_allgather"]()
        arms["fp32_simt_fused"]()
        torch.cuda.synchronize()
        same_fp32 = bool(torch.equal(out.full, reference))
        out.barrier()
        reference = arms["tf32_then_allgather"]()
        arms["tf32_fused"]()
        torch.cuda.synchronize()
        same_tf32 = bool(torch.equal(out.full, reference))
        del reference
        flags = torch.tensor([int(same_fp32), int(same_tf32)], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if not bool(flags.min().item()):
            raise SystemExit(f"rank {rank}: fused all-gather differs from GEMM + NCCL all-gather ({flags.tolist()})")
        fused = {"bit_identical_to_collective": True}
        for name, fn in arms.items():
            for _ in range(args.warmup):
                fn()
            dist.barrier()
            ms = reduce_max(timed_ms(fn, args.steps))
            fused[name] = {"ms": ms, "tflops_total": 2.0 * args.m * args.n * args.k / ms / 1e9}

    if rank == 0:
        print(json.dumps({"benchmark": "m_sharded_gemm", "m": args.m, "n": args.n, "k": args.k, "n_gpus": world,
                          "rows_per_rank": rows, "steps": args.steps, "warmup": args.warmup,
                          "sgemm_impl": args.sgemm_impl, "tf32_kernel": tf32_kernel, "parity": {
                              "fp32_max_abs_error": err32, "fp32_tolerance": tol, "tf32_rel_frobenius": rel_tf32},
                          "fp32_simt": results["fp32_simt"], "tf32": results["tf32"], "allgather_c": gather,
                          "gemm_plus_allgather": fused}))
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
