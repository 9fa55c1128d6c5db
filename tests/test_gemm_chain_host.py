"""The chained GEMM launch's task order can always make progress: host model, random interleavings (CPU)."""
import random

import pytest

from ittai_b200.gemm_chain import chain_tasks, simulate

SIGLIP_LAYER = [768, 3072, 768, 2304]          # out-proj, fc1, fc2, next QKV


def test_task_order_is_gemm_then_row_block_then_column():
    t = chain_tasks(700, [512, 256])
    assert t[:7] == [(0, 0, 0), (0, 0, 1), (0, 1, 0), (0, 1, 1), (0, 2, 0), (0, 2, 1), (1, 0, 0)] and len(t) == 9


@pytest.mark.parametrize("m,ns,clusters", [(12544, SIGLIP_LAYER, 74), (12544, [768, 2304], 74), (700, SIGLIP_LAYER, 74),
                                            (300, [256, 256, 256, 256], 3), (2048, [256, 1024], 5), (12544, SIGLIP_LAYER, 33)])
def test_random_interleavings_never_deadlock(m, ns, clusters):
    for seed in range(5):
        r = simulate(m, ns, clusters, random.Random(seed))
        assert r["steps"] == 2 * r["tasks"]


def test_a_task_that_waits_for_a_later_task_is_reported():
    """The model itself: with the GEMMs' dependency reversed by hand (first GEMM waiting on a second one that is listed after
    it) no cluster can move, and the simulator says so instead of spinning."""
    import ittai_b200.gemm_chain as gc
    tasks = gc.chain_tasks(512, [256, 256])
    real = gc.chain_tasks
    try:
        gc.chain_tasks = lambda m, ns: [(1 - g, tm, tn) for g, tm, tn in tasks]      # GEMM 1's tiles first
        with pytest.raises(RuntimeError, match="deadlock"):
            gc.simulate(512, [256, 256], 2, random.Random(0))
    finally:
        gc.chain_tasks = real
