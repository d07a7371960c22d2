"""CUDA-event timing and JSON helpers (python/cuda_ai_kernels/benchmark.py:12-42)."""
from __future__ import annotations

import json
import statistics
import time
from pathlib import Path
from typing import Any, Callable

import torch


def cuda_event_benchmark(fn: Callable[[], Any], warmup: int = 50, repeat: int = 200) -> dict[str, float]:
    """Times ``fn`` ``repeat`` times with events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples: list[float] = []
    for _ in range(repeat):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        fn()
        end.record()
        end.synchronize()
        samples.append(begin.elapsed_time(end))
    return {
        "mean_ms": statistics.fmean(samples),
        "p50_ms": statistics.median(samples),
        "min_ms": min(samples),
        "max_ms": max(samples),
    }


def cuda_graph_benchmark(fn: Callable[[], Any], warmup: int = 10, repeat: int = 50,
                         calls_per_graph: int = 10) -> dict[str, float]:
    """Captures ``calls_per_graph`` calls in a CUDA graph and times replays.

    This is the reference's headline method (benchmarks/bench_gemm_all.py:46-77):
    launch overhead and allocator work are amortised, what remains is device
    time per call.
    """
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for _ in range(calls_per_graph):
            fn()
    samples: list[float] = []
    with torch.cuda.stream(stream):
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        for _ in range(repeat):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
            samples.append(begin.elapsed_time(end) / calls_per_graph)
    torch.cuda.current_stream().wait_stream(stream)
    return {
        "mean_ms": statistics.fmean(samples),
        "p50_ms": statistics.median(samples),
        "min_ms": min(samples),
        "max_ms": max(samples),
    }


def save_json(path: str | Path, payload: dict[str, Any]) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(payload, indent=2), encoding="utf-8")


def now_tag() -> str:
    return time.strftime("%Y%m%d-%H%M%S")
