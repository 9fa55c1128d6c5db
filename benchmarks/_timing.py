"""Timing protocol shared by the benchmark scripts: a few untimed calls, then each of ``repeats`` calls bracketed by its
own pair of CUDA events, and the middle value of the sorted durations.  The reference's scripts time the same way
(3 warm-ups, 20 timed calls, median: ``benchmarks/qwen3.py:16-25``), so the figures are comparable."""
import statistics

import torch


def median_ms(call, repeats: int = 20, warmups: int = 3) -> float:
    for _ in range(warmups):
        call()
    torch.cuda.synchronize()
    durations = []
    for _ in range(repeats):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        call()
        end.record()
        end.synchronize()
        durations.append(begin.elapsed_time(end))
    return statistics.median_high(durations)


def graph_us(call, copies: int = 50) -> float:
    """Microseconds per call when ``copies`` calls replay back to back inside one CUDA graph (includes the
    launch-to-launch gap a forward pass sees)."""
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(copies):
            call()
    graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    graph.replay()
    end.record()
    end.synchronize()
    return begin.elapsed_time(end) / copies * 1e3
