"""The prefill task list (CPU): equal to the reference's own ``build_tasks`` output on the fixture's packings, and
executable by persistent CTAs in any interleaving (a host model of the device queue)."""
import hashlib
import os

import numpy as np
import pytest

from ittai_b200.qwen3 import config as cfg
from ittai_b200.qwen3.tasks import arrivals_of, build_tasks, simulate
from tests.golden.make_golden import TASK_CASES


@pytest.fixture(scope="module")
def golden(golden_dir):
    return np.load(os.path.join(golden_dir, "qwen3_tasks.npz"))


@pytest.mark.parametrize("name", sorted(TASK_CASES))
def test_task_list_equals_the_reference(golden, name):
    lens, mb, bmax, tiles, spt, kvb, gm = TASK_CASES[name]
    tasks, expect, T = build_tasks(lens, mb, bmax, cfg.L + 1, tiles, spt, kvb, gm)
    assert tasks.dtype == np.int32 and expect.dtype == np.int32 and tasks.shape[1] == cfg.TW
    assert T == int(golden[name + "__T"]) == sum(lens)
    sha = hashlib.sha256(tasks.tobytes() + expect.tobytes()).digest()
    assert sha == golden[name + "__sha"].tobytes()
    if name + "__tasks" in golden:
        assert np.array_equal(tasks, golden[name + "__tasks"]) and np.array_equal(expect, golden[name + "__expect"])


@pytest.mark.parametrize("name,n_ctas", [("single_short", 1), ("single_short", 148), ("ragged", 1), ("ragged", 7), ("ragged", 148),
                                         ("straddling_sm90", 3), ("straddling_sm90", 132), ("one_block_each", 148)])
def test_any_interleaving_of_ctas_completes(name, n_ctas):
    """Every flag ends with exactly the arrivals the list announces, no CTA ever waits for something only a later record
    produces (one CTA runs the list strictly in order), and random schedules of many CTAs finish too."""
    lens, mb, bmax, tiles, spt, kvb, gm = TASK_CASES[name]
    tasks, expect, _ = build_tasks(lens, mb, bmax, cfg.L + 1, tiles, spt, kvb, gm)
    arr = lambda t: arrivals_of(t, cfg.L + 1, mb, bmax, spt, lens)
    for seed in range(3 if n_ctas > 1 else 1):
        arrived = simulate(tasks, expect, n_ctas, np.random.default_rng(seed), arr)
        assert np.array_equal(arrived, expect)


def test_a_missing_arrival_is_caught():
    """The model of the queue reports the hang a device would suffer: raise one flag's expectation and nobody gets past it."""
    lens, mb, bmax, tiles, spt, kvb, gm = TASK_CASES["single_short"]
    tasks, expect, _ = build_tasks(lens, mb, bmax, cfg.L + 1, tiles, spt, kvb, gm)
    expect = expect.copy()
    expect[(cfg.SLOT_QKV * (cfg.L + 1) + 3) * mb] += 1
    with pytest.raises(RuntimeError, match="blocked"):
        simulate(tasks, expect, 4, np.random.default_rng(0), lambda t: arrivals_of(t, cfg.L + 1, mb, bmax, spt, lens))


def test_layer_order_guard_for_the_shared_qkv_buffer():
    """The QKV GEMM of layer l > 0 names the per-sequence flags of layer l - 1 of every sequence its row block touches."""
    lens, mb, bmax = [100, 100, 100], 3, 4
    tasks, expect, _ = build_tasks(lens, mb, bmax, cfg.L + 1, (32, 8, 48, 8), 1, 64, 8)
    base = cfg.NSLOT * (cfg.L + 1) * mb
    q = tasks[(tasks[:, 0] == cfg.OP_QKV) & (tasks[:, 1] == 5)]
    blk0, blk1, blk2 = (q[q[:, 2] == b][0] for b in range(3))
    assert (blk0[6], blk0[7]) == (base + 4 * bmax + 0, 2)      # rows 0..127: sequences 0 and 1
    assert (blk1[6], blk1[7]) == (base + 4 * bmax + 1, 2)      # rows 128..255: sequences 1 and 2
    assert (blk2[6], blk2[7]) == (base + 4 * bmax + 2, 1)
    assert (tasks[(tasks[:, 0] == cfg.OP_QKV) & (tasks[:, 1] == 0)][:, 6] == -1).all()


# ---- properties over random packings ---------------------------------------------------------------------------------------
from hypothesis import given, settings, strategies as st  # noqa: E402


@settings(max_examples=12, deadline=None)
@given(lens=st.lists(st.integers(min_value=1, max_value=300), min_size=1, max_size=5), spt=st.sampled_from([1, 2]),
       group_m=st.sampled_from([1, 2, 8]), seed=st.integers(min_value=0, max_value=1000))
def test_random_packings_are_consistent(lens, spt, group_m, seed):
    """For any packing (sequences of length 1, sequences that straddle row blocks, a single block): the announced arrivals
    equal the arrivals the tasks make, every dependency index is a flag that exists, attention items cover every query
    row exactly once per kv head, and a handful of persistent CTAs get through the list."""
    T = sum(lens)
    mb = -(-T // cfg.BM) + 1
    bmax = len(lens) + 1
    tiles = (4, 2, 6, 2)
    tasks, expect, T2 = build_tasks(lens, mb, bmax, cfg.L + 1, tiles, spt, 64, group_m)
    assert T2 == T
    n_flags = len(expect)
    for d, c in ((tasks[:, 4], tasks[:, 5]), (tasks[:, 6], tasks[:, 7])):
        live = d >= 0
        assert (d[live] + c[live] <= n_flags).all() and (c[live] >= 1).all()
    # layer 0's attention items: each sequence's query blocks, all 8 kv heads
    a0 = tasks[(tasks[:, 0] == cfg.OP_ATTN) & (tasks[:, 1] == 0)]
    assert len(a0) == cfg.NKV * sum(-(-n // cfg.QB) for n in lens)
    for s, n in enumerate(lens):
        blocks = sorted(a0[a0[:, 2] == s * cfg.NKV][:, 3].tolist())
        assert blocks == list(range(-(-n // cfg.QB)))
    arr = lambda t: arrivals_of(t, cfg.L + 1, mb, bmax, spt, lens)
    arrived = simulate(tasks, expect, 5, np.random.default_rng(seed), arr)
    assert np.array_equal(arrived, expect)
