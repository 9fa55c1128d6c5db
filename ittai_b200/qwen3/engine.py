"""Qwen3-0.6B prefill on the tensor-core kernels, behind the reference's ``Engine`` surface
(reference ``src/ittai/qwen3/engine.py:13-187``).

``Engine.forward(input_ids)`` packs variable-length sequences into one activation matrix, runs 28 layers of
RMSNorm -> QKV GEMM -> QK-norm + RoPE -> causal GQA attention -> O-proj + residual -> RMSNorm -> gate/up GEMM with
SwiGLU -> down-proj + residual, and returns the L2-normalised final-norm of every sequence's last token, the
embedding head of the reference (``src/ittai/qwen3/base.py:131-145``).  ``PrefillCore`` is the layer loop itself; the
decoder reuses it to fill its KV cache from a prompt.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from .. import _C, ops
from .config import BM, D, DGU, DQ, DQKV, EPS, FF, HD, NH, NKV, QB
from .decoder import _strip, pack_weights, rope_table
from .tasks import build_tasks


def rope_perm(n_heads):
    """Row order that puts the two halves of every RoPE pair side by side: within each 128-row head, rows
    0, 64, 1, 65, ... (reference ``src/ittai/qwen3/engine.py:13-14``).

    Kept for callers that import it; this build stores Q/K rows in the eager order and rotates (i, i + 64) directly."""
    within = np.stack([np.arange(HD // 2), np.arange(HD // 2) + HD // 2], axis=1).reshape(-1)
    return (np.arange(n_heads)[:, None] * HD + within[None, :]).reshape(-1)


def packing(seqlens):
    """Host description of one packed forward for the kernels: per-token positions, sequence ids and cache rows, and the
    per-sequence (first row, rows, first key row, key rows) records the attention kernel walks.
    Returns (pos, seq, slot, seqs, T) as int32 numpy arrays."""
    seqlens = [int(x) for x in seqlens]
    cu = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int64)
    T = int(cu[-1])
    pos = np.concatenate([np.arange(n) for n in seqlens]).astype(np.int32) if T else np.zeros(0, np.int32)
    seq = np.zeros(T, np.int32)                       # one packed key/value store: every token lives in "sequence 0"
    slot = np.arange(T, dtype=np.int32)
    seqs = np.array([[cu[s], seqlens[s], cu[s], seqlens[s]] for s in range(len(seqlens))], dtype=np.int32).reshape(-1, 4)
    return pos, seq, slot, seqs, T


class PrefillCore:
    """The 28-layer loop over a packed ``[T, 1024]`` activation matrix.  Owns the activation buffers (torch tensors, as
    the reference's Engine owns its buffers: ``src/ittai/qwen3/engine.py:123-134``); weights and the key/value store are
    borrowed."""

    def __init__(self, w: dict, n_layers: int, max_tokens: int, device, fused_rope: bool = True, fold_norm: bool = False):
        self.w, self.L, self.M, self.dev = w, n_layers, max_tokens, device
        self.fused_rope = fused_rope       # QK-norm + RoPE + cache scatter inside the QKV GEMM's epilogue (needs > 128 rows)
        # ``fold_norm``: the RMSNorms in front of the QKV and gate/up projections are folded into those GEMMs, as in the
        # reference's kernels (``src/ittai/qwen3/engine.py:107-114``: gain folded into the weights in fp32 and rounded once;
        # ``base.py:59-78``: the residual epilogue before leaves per-row partial sums of squares, the consuming epilogue
        # applies rstd): no norm kernel is left in a layer but the very first.  Off, every rounding point is the eager
        # module's (what the decoder's prefill uses: its cache feeds the decode loop).
        self.fold_norm = fold_norm
        if fold_norm:
            fold = lambda W, g: (W.float() * g.float()[:, None, :]).to(torch.bfloat16).contiguous()
            self.wqkv_f, self.wgu_f = fold(w["wqkv"], w["ln1"]), fold(w["wgu"], w["ln2"])
            self.stats = torch.zeros(max_tokens, D // 128, 2, dtype=torch.float32, device=device)
            self.zeros_qkv, self.zeros_gu = (torch.zeros(n, dtype=torch.float32, device=device) for n in (DQKV, DGU))
        z = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=device)
        self.h, self.xn, self.qkv, self.attn, self.act = z(max_tokens, D), z(max_tokens, D), z(max_tokens, DQKV), z(max_tokens, DQ), z(max_tokens, FF)
        self.status = ops.new_status(device)

    def run(self, T, tokens, pos, seq, slot, seqs, max_q_len, rope, kv_layer, kv_cap, k_strides):
        """``tokens/pos/seq/slot``: int32 device ``[T]``; ``seqs``: int32 device ``[n, 4]``; ``kv_layer(l)`` returns the
        (K, V) tensors of layer ``l`` laid out ``[B, 8, kv_cap, 128]``; ``k_strides`` = (row, head, seq) in elements."""
        L, st, w = _C.lib(), self.status, self.w
        h, xn, qkv, attn, act = self.h[:T], self.xn[:T], self.qkv[:T], self.attn[:T], self.act[:T]
        s = ops._stream(h)
        _C.check(L.ittai_embed_rows(tokens.data_ptr(), w["embed"].data_ptr(), h.data_ptr(), T, w["embed"].shape[0], s))
        fold = self.fold_norm and T > 128
        for l in range(self.L):
            kc, vc = kv_layer(l)
            # layer 0 reads the embedding rows, which no GEMM epilogue produced: its first norm is a pass of its own
            folded = fold and l > 0
            if folded:
                x_in, wq, ln = h, self.wqkv_f[l], dict(row_stats=self.stats[:T], col_sums=self.zeros_qkv, stats_eps=EPS, stats_rms=True)
            else:
                ops.rmsnorm_rows(h, w["ln1"][l], EPS, out=xn)
                x_in, wq, ln = xn, w["wqkv"][l], {}
            if T > 128 and self.fused_rope:
                # QK-norm + RoPE + cache scatter inside the QKV GEMM's epilogue (the reference's qkv epilogue, base.py:84-109)
                ops.gemm(x_in, wq, st, out=qkv, epi=_C.EPI_QKROPE, **ln,
                         qk_rope=dict(qn=w["qn"][l], kn=w["kn"][l], rope=rope, pos=pos, seq=seq, slot=slot, kcache=kc, vcache=vc, kv_cap=kv_cap, eps=EPS))
            else:
                ops.gemm(x_in, wq, st, out=qkv, **ln)
                _C.check(L.ittai_qwen3_qk_rope_scatter(qkv.data_ptr(), w["qn"][l].data_ptr(), w["kn"][l].data_ptr(), rope.data_ptr(),
                                                       pos.data_ptr(), seq.data_ptr(), slot.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                       T, kv_cap, EPS, s))
            ops.attention(qkv, kc, vc, attn, seqs, n_heads=NH, group=NH // NKV, head_dim=HD, causal=True, max_q_len=max_q_len,
                          q_strides=(DQKV, HD), k_strides=k_strides, v_strides=k_strides, o_strides=(DQ, HD),
                          q_rows_total=T, kv_rows_total=kc.numel() // HD, status=st)
            ops.gemm(attn, w["wo"][l], st, residual=h, out=h, stats_out=self.stats[:T] if fold else None)
            if fold:
                ops.gemm(h, self.wgu_f[l], st, epi=_C.EPI_SWIGLU, out=act, row_stats=self.stats[:T], col_sums=self.zeros_gu, stats_eps=EPS, stats_rms=True)
            else:
                ops.rmsnorm_rows(h, w["ln2"][l], EPS, out=xn)
                ops.gemm(xn, w["wgu"][l], st, epi=_C.EPI_SWIGLU, out=act)
            ops.gemm(act, w["wd"][l], st, residual=h, out=h, stats_out=self.stats[:T] if fold and l + 1 < self.L else None)
        return h


class Engine:
    """``Engine(sd, max_tokens, max_seqs, ...)`` with ``forward(input_ids: list[list[int]]) -> fp32 [B, 1024]``, a view of
    a persistent buffer (callers clone, as with the reference: ``src/ittai/qwen3/model.py:88``).  The tuning arguments
    of the reference (``arch, tile_n, stages, kv_block, group_m, warps``) are accepted and ignored."""

    @torch.no_grad()
    def __init__(self, sd, max_tokens, max_seqs, arch=None, tile_n=None, stages=None, kv_block=None, group_m=None, warps=8,
                 device="cuda", graph=True, fused_rope=True, fold_norm=True):
        sd = _strip(sd if isinstance(sd, dict) else sd.state_dict())
        self.dev = torch.device(device)
        self.M, self.Bmax = (max_tokens + BM - 1) // BM * BM, max_seqs
        self.L = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
        self.w = pack_weights(sd, self.L, self.dev)
        self.embed, self.fin_w = self.w["embed"], self.w["fin_w"]
        self.rope = rope_table(self.M, self.dev)
        self.core = PrefillCore(self.w, self.L, self.M, self.dev, fused_rope=fused_rope, fold_norm=fold_norm)
        z = lambda *s, dt: torch.zeros(*s, dtype=dt, device=self.dev)
        # one packed key/value store reused by every layer: the embedding pass keeps no cache
        self.kbuf, self.vbuf = z(1, NKV, self.M, HD, dt=torch.bfloat16), z(1, NKV, self.M, HD, dt=torch.bfloat16)
        self.tokens, self.pos, self.seq, self.slot = (z(self.M, dt=torch.int32) for _ in range(4))
        self.seqs, self.last = z(max_seqs, 4, dt=torch.int32), z(max_seqs, dt=torch.int32)
        self.out = z(max_seqs, D, dt=torch.float32)
        self.use_graph, self._graphs, self._meta = graph, {}, {}

    def _tasks(self, seqlens):
        """Packing metadata, cached per tuple of lengths like the reference's task lists (``engine.py:144-151``)."""
        key = tuple(seqlens)
        if key not in self._meta:
            pos, seq, slot, seqs, T = packing(seqlens)
            dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))
            self._meta[key] = (dev(pos), dev(seq), dev(slot), dev(seqs), dev(seqs[:, 0] + seqs[:, 1] - 1), T)
        return self._meta[key]

    def _body(self, T, B, max_len):
        kv = lambda l: (self.kbuf, self.vbuf)
        h = self.core.run(T, self.tokens, self.pos, self.seq, self.slot, self.seqs[:B], max_len, self.rope, kv, self.M,
                          (HD, self.M * HD, 0))
        _C.check(_C.lib().ittai_qwen3_final_pool(h.data_ptr(), self.last.data_ptr(), self.fin_w.data_ptr(), self.out.data_ptr(), B, EPS,
                                                 ops._stream(h)))

    @torch.no_grad()
    def forward(self, input_ids):
        seqlens = [len(x) for x in input_ids]
        T, B = sum(seqlens), len(seqlens)
        assert T <= self.M and B <= self.Bmax and min(seqlens) > 0
        pos, seq, slot, seqs, last, _ = self._tasks(seqlens)
        flat = torch.tensor([t for s in input_ids for t in s], dtype=torch.int32)
        if int(flat.min()) < 0 or int(flat.max()) >= self.embed.shape[0]:
            raise ValueError(f"token id outside [0, {self.embed.shape[0]})")      # the gather kernel would clamp it silently
        self.tokens[:T].copy_(flat, non_blocking=True)
        self.pos[:T].copy_(pos, non_blocking=True)
        self.seq[:T].copy_(seq, non_blocking=True)
        self.slot[:T].copy_(slot, non_blocking=True)
        self.seqs[:B].copy_(seqs, non_blocking=True)
        self.last[:B].copy_(last, non_blocking=True)
        key = tuple(seqlens)
        if not self.use_graph:
            self._body(T, B, max(seqlens))
        else:
            if key not in self._graphs:
                if len(self._graphs) >= 8:
                    self._graphs.pop(next(iter(self._graphs)))
                self.core.status.zero_()
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._body(T, B, max(seqlens))
                torch.cuda.current_stream().wait_stream(s)
                ops.check_status(self.core.status)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._body(T, B, max(seqlens))
                self._graphs[key] = g
            self._graphs[key].replay()
        return self.out[:B]

    def check(self) -> None:
        ops.check_status(self.core.status)

    def task_list(self, seqlens, group_m=8):
        """The forward over ``seqlens`` as the reference's device queue would see it: ``(tasks, expect, T)`` of
        ``build_tasks`` for this engine's geometry (256-column GEMM tiles, one arrival per tile).  The launches this
        engine records into its CUDA graph realise the same dependencies by stream order, phase after phase; the list
        is what a single persistent kernel would walk instead."""
        return build_tasks(seqlens, self.M // BM, self.Bmax, self.L + 1, (DQKV // 256, D // 256, 2 * FF // 256, D // 256), 1, 128, group_m)
