"""The device "instruction queue" of the Qwen3 prefill as a host-built table: one 8-word record per unit of work plus
the number of arrivals every dependency flag must collect.  Same contract as the reference's ``build_tasks``
(reference ``src/ittai/qwen3/engine.py:17-84``), so a list built here equals the reference's on the same arguments
(pinned by ``tests/golden/qwen3_tasks.npz``), and ``simulate`` replays a list the way persistent CTAs would.

Record: ``[op, layer, i, j, d0, c0, d1, c1]``.  A task may start once the ``c0`` consecutive flags from ``d0`` and the
``c1`` consecutive flags from ``d1`` have each collected ``expect[flag]`` arrivals (a negative ``d`` means "none").

* GEMM ops (QKV, O-proj, gate/up, down): ``i`` = 128-row block, ``j`` = column tile.  Row blocks go in groups of
  ``group_m``; inside a group the column tile is the outer loop, so consecutive records share a weight tile.  A GEMM
  task waits for its input block (``SPEC[op]['dep']``) and arrives ``spt`` times on its output block
  (``SPEC[op]['out']``, one layer further for the down projection).
* Attention: ``i`` = sequence * 8 + kv head, ``j`` = block of 64 query rows, a sequence's last block first (the longest
  item first).  It waits for the QKV blocks from the start of its sequence through its own rows and arrives on the
  128-row block(s) its rows fall into and on the per-(layer, sequence) flag.
* The QKV GEMM of layer l > 0 also waits for the per-sequence flags of layer l - 1 of every sequence its row block
  touches: it overwrites the buffer that layer's attention still reads.
* One embedding task per row block first, one pooling task per sequence last.
"""
from __future__ import annotations

import numpy as np

from .config import BM, L, NKV, NSLOT, OP_ATTN, OP_DOWN, OP_EMB, OP_FINAL, OP_GU, OP_OPROJ, OP_QKV, QB, SLOT_ATTN, SLOT_QKV, SLOT_X, SPEC, TW


def build_tasks(seqlens, MB_alloc, Bmax, L1, n_tiles, spt, kvb=None, group_m=8):
    """Returns ``(tasks int32 [n, 8], expect int32 [NSLOT * L1 * MB_alloc + L * Bmax], T)``.

    ``MB_alloc``: row blocks the flag table is laid out for; ``Bmax``: sequences it is laid out for; ``L1`` = layers + 1;
    ``n_tiles`` = column tiles of (QKV, O-proj, gate/up, down); ``spt``: arrivals one finished tile makes (2 where two
    consumer groups each arrive); ``kvb`` does not shape the list (kept for the reference's signature)."""
    lens = [int(n) for n in seqlens]
    n_seq = len(lens)
    first_row = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    T = int(first_row[-1])
    n_blocks = -(-T // BM)
    tiles = dict(zip((OP_QKV, OP_OPROJ, OP_GU, OP_DOWN), n_tiles))

    def flag(slot, layer, block):
        return (slot * L1 + layer) * MB_alloc + block

    seq_flags = NSLOT * L1 * MB_alloc

    def seq_flag(layer, s):
        return seq_flags + layer * Bmax + s

    expect = np.zeros(seq_flags + L * Bmax, dtype=np.int32)
    owner = np.repeat(np.arange(n_seq), lens)                       # sequence of every packed row
    blocks = np.arange(n_blocks)
    seq_first = owner[blocks * BM] if n_blocks else np.zeros(0, np.int64)
    seq_last = owner[np.minimum((blocks + 1) * BM, T) - 1] if n_blocks else np.zeros(0, np.int64)

    # attention items, the same for every layer
    items = []
    for s, n in enumerate(lens):
        for qb in range(-(-n // QB) - 1, -1, -1):
            r0 = int(first_row[s]) + qb * QB
            r1 = min(r0 + QB, int(first_row[s + 1])) - 1
            for g in range(NKV):
                items.append((s, g, qb, r0 // BM, r1 // BM, int(first_row[s]) // BM))

    rec = []
    for m in range(n_blocks):
        rec.append((OP_EMB, 0, m, 0, -1, 0, -1, 0))
        expect[flag(SLOT_X, 0, m)] = spt
    for layer in range(L):
        for op in (OP_QKV, OP_ATTN, OP_OPROJ, OP_GU, OP_DOWN):
            if op == OP_ATTN:
                for s, g, qb, b0, b1, bs in items:
                    rec.append((OP_ATTN, layer, s * NKV + g, qb, flag(SLOT_QKV, layer, bs), b1 - bs + 1, -1, 0))
                    expect[flag(SLOT_ATTN, layer, b0)] += spt
                    if b1 != b0:
                        expect[flag(SLOT_ATTN, layer, b1)] += spt
                    expect[seq_flag(layer, s)] += spt
                continue
            spec = SPEC[op]
            for g0 in range(0, n_blocks, group_m):
                for j in range(tiles[op]):
                    for i in range(g0, min(g0 + group_m, n_blocks)):
                        d1, c1 = -1, 0
                        if op == OP_QKV and layer > 0:
                            d1, c1 = seq_flag(layer - 1, int(seq_first[i])), int(seq_last[i] - seq_first[i]) + 1
                        rec.append((op, layer, i, j, flag(spec["dep"], layer, i), 1, d1, c1))
            expect[flag(spec["out"], layer + spec["dl"], blocks)] = spt * tiles[op]
    for s in range(n_seq):
        rec.append((OP_FINAL, 0, s, 0, flag(SLOT_X, L, (int(first_row[s + 1]) - 1) // BM), 1, -1, 0))
    return np.asarray(rec, dtype=np.int32).reshape(-1, TW), expect, T


def arrivals_of(task, L1, MB_alloc, Bmax, spt, seqlens):
    """The (flag, count) arrivals one finished task makes: what the kernels' epilogues do on the device."""
    op, layer, i, j = (int(x) for x in task[:4])
    flag = lambda slot, l, b: (slot * L1 + l) * MB_alloc + b
    if op == OP_EMB:
        return [(flag(SLOT_X, 0, i), spt)]
    if op == OP_FINAL:
        return []
    if op == OP_ATTN:
        first_row = np.concatenate([[0], np.cumsum([int(n) for n in seqlens])])
        s = i // NKV
        r0 = int(first_row[s]) + j * QB
        r1 = min(r0 + QB, int(first_row[s + 1])) - 1
        out = [(flag(SLOT_ATTN, layer, r0 // BM), spt)]
        if r1 // BM != r0 // BM:
            out.append((flag(SLOT_ATTN, layer, r1 // BM), spt))
        out.append((NSLOT * L1 * MB_alloc + layer * Bmax + s, spt))
        return out
    spec = SPEC[op]
    return [(flag(spec["out"], layer + spec["dl"], i), spt)]


def simulate(tasks, expect, n_ctas, rng, arrivals):
    """Replays a task list with ``n_ctas`` persistent CTAs: each claims the next record from one counter, waits until its
    dependency flags are complete, runs, and makes its arrivals (``arrivals(task) -> [(flag, count)]``); which CTA moves
    next is drawn from ``rng``.  Returns the per-flag arrival counts.  Raises if every CTA is blocked (a list that a
    device would hang on) or a flag collects more arrivals than expected."""
    arrived = np.zeros_like(expect)
    nxt, done = 0, 0
    holding = [None] * n_ctas

    def ready(t):
        for d, c in ((int(t[4]), int(t[5])), (int(t[6]), int(t[7]))):
            if d >= 0 and c > 0 and not (arrived[d:d + c] >= expect[d:d + c]).all():
                return False
        return True

    while done < len(tasks):
        for k in range(n_ctas):
            if holding[k] is None and nxt < len(tasks):
                holding[k] = nxt
                nxt += 1
        movable = [k for k in range(n_ctas) if holding[k] is not None and ready(tasks[holding[k]])]
        if not movable:
            stuck = [int(holding[k]) for k in range(n_ctas) if holding[k] is not None]
            raise RuntimeError(f"every CTA is blocked: waiting tasks {stuck[:8]}")
        k = movable[int(rng.integers(len(movable)))]
        for f, c in arrivals(tasks[holding[k]]):
            arrived[f] += c
            if arrived[f] > expect[f]:
                raise RuntimeError(f"flag {f} collected {arrived[f]} arrivals, {expect[f]} expected")
        holding[k] = None
        done += 1
    return arrived
