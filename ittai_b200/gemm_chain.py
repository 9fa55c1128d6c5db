"""Host model of the task list a chained GEMM launch walks (``csrc/gemm2_chain_sm100.cu``).

The kernel deals the tiles of all GEMMs of a chain (GEMM after GEMM, row block after row block, column tile fastest) round-robin
to its resident clusters; the producer of a tile of GEMM ``g + 1`` waits until every column tile of GEMM ``g`` in the same row
block has been finished by its epilogue.  ``simulate`` replays that with clusters that advance in a random interleaving, a load
pipeline that runs a bounded number of tiles ahead of the epilogue, and reports the deadlock a device would time out on.  The
reference keeps the same kind of per-row-block counters for every task of its persistent kernel
(``src/ittai/qwen3/engine.py:17-84``); ``ittai_b200.qwen3.tasks.simulate`` is the model of that full list.
"""
from __future__ import annotations

import random

PM = PN = 256          # the pair tile of the two-SM GEMM


def chain_tasks(m: int, ns: list[int]) -> list[tuple[int, int, int]]:
    """``(gemm, tile_m, tile_n)`` in list order for a chain whose GEMMs have ``m`` rows and ``ns[g]`` output columns."""
    tiles_m = (m + PM - 1) // PM
    return [(g, tm, tn) for g, n in enumerate(ns) for tm in range(tiles_m) for tn in range(n // PN)]


def simulate(m: int, ns: list[int], n_clusters: int, rng: random.Random, ahead: int = 2) -> dict:
    """Clusters take tasks ``c, c + n_clusters, ...``.  Per cluster the producer may be up to ``ahead`` tiles in front of the
    epilogue (the kernel's load pipeline and its two accumulators); a producer step needs the row block of the previous GEMM
    complete, an epilogue step needs the tile's loads issued.  Returns the number of steps taken and the largest lead a
    producer had to give up waiting for a flag; raises ``RuntimeError`` on a deadlock."""
    tasks = chain_tasks(m, ns)
    tiles_m = (m + PM - 1) // PM
    need = [n // PN for n in ns]
    done = [[0] * tiles_m for _ in ns]                     # finished column tiles per (gemm, row block)
    mine = [list(range(c, len(tasks), n_clusters)) for c in range(n_clusters)]
    loaded = [0] * n_clusters                              # tiles whose loads the producer has issued
    finished = [0] * n_clusters                            # tiles whose epilogue has signalled
    steps = blocked_max = 0
    while any(finished[c] < len(mine[c]) for c in range(n_clusters)):
        moves = []
        for c in range(n_clusters):
            if loaded[c] < len(mine[c]) and loaded[c] - finished[c] < ahead:
                g, tm, _ = tasks[mine[c][loaded[c]]]
                if g == 0 or done[g - 1][tm] == need[g - 1]:
                    moves.append(("load", c))
            if finished[c] < loaded[c]:
                moves.append(("finish", c))
        if not moves:
            stuck = {c: tasks[mine[c][loaded[c]]] for c in range(n_clusters) if loaded[c] < len(mine[c])}
            raise RuntimeError(f"deadlock: no cluster can move; waiting producers {stuck}")
        kind, c = rng.choice(moves)
        if kind == "load":
            loaded[c] += 1
        else:
            g, tm, _ = tasks[mine[c][finished[c]]]
            done[g][tm] += 1
            finished[c] += 1
        blocked_max = max(blocked_max, sum(1 for c in range(n_clusters) if loaded[c] < len(mine[c]) and loaded[c] - finished[c] < ahead
                                           and tasks[mine[c][loaded[c]]][0] > 0
                                           and done[tasks[mine[c][loaded[c]]][0] - 1][tasks[mine[c][loaded[c]]][1]] < need[tasks[mine[c][loaded[c]]][0] - 1]))
        steps += 1
    assert all(done[g][tm] == need[g] for g in range(len(ns)) for tm in range(tiles_m))
    return {"steps": steps, "tasks": len(tasks), "max_blocked_producers": blocked_max}
