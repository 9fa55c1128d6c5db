"""Host-side handles on the dense kernels shared by the Qwen3 prefill and SigLIP engines (thin ctypes calls)."""
from __future__ import annotations

import ctypes as C

import torch

from . import _C


def new_status(device) -> torch.Tensor:
    """Zeroed device status words; pass to a sequence of launches, then ``check_status``."""
    return torch.zeros(_C.STATUS_WORDS, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor) -> None:
    _C.decode_status(status.cpu().tolist())


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def gemm_desc(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor, bias: torch.Tensor | None = None,
              residual: torch.Tensor | None = None, epi: int = _C.EPI_NONE, out: torch.Tensor | None = None,
              row_stats: torch.Tensor | None = None, col_sums: torch.Tensor | None = None, stats_out: torch.Tensor | None = None,
              stats_eps: float = 0.0, qk_rope: dict | None = None, stats_k: int = 0, stats_rms: bool = False):
    """The ``IttaiGemm`` record of ``gemm(...)`` with the same arguments, and its output tensor: ``(record, out)``.

    ``out = epilogue(a @ w.T)`` on the tcgen05 GEMM: a [M, K] and w [N, K] bf16 (last dim contiguous), bias fp32 [N],
    residual bf16 [M, N].  SwiGLU takes interleaved (gate, up) weight rows and returns [M, N/2].  ``row_stats`` (fp32
    [M, 2] from ``row_stats``) with ``col_sums`` (fp32 [N]) folds a LayerNorm over ``a`` into the GEMM: ``w`` is then the
    weight scaled by the LayerNorm gain along K and ``bias`` includes ``W @ beta`` (see ``fold_layernorm``).  ``stats_out``
    (fp32 [M, N/128, 2]) receives the (sum, sum of squares) of every 128-column slice of the output rows; passed as the
    ``row_stats`` of the next GEMM (3-D, with ``stats_eps``) it replaces the separate statistics pass.  ``epi=EPI_QKROPE``
    (Qwen3 QKV projection, N = 4096, M > 128) takes ``qk_rope`` = dict(qn, kn, rope, pos, seq, slot, kcache, vcache,
    kv_cap, eps) and does the work of the QK-norm + RoPE + cache-scatter pass in its epilogue."""
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k
    n_out = n // 2 if epi == _C.EPI_SWIGLU else n
    if out is None:
        out = torch.empty(m, n_out, dtype=torch.bfloat16, device=a.device)
    g = _C.Gemm()
    g.m, g.n, g.k, g.epi = m, n, k, epi
    g.ld_a, g.ld_w, g.ld_out = a.stride(0), w.stride(0), out.stride(0)
    g.a, g.w, g.out, g.status = a.data_ptr(), w.data_ptr(), out.data_ptr(), status.data_ptr()
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
        g.bias = bias.data_ptr()
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (m, n) and residual.stride(1) == 1
        g.residual, g.ld_res = residual.data_ptr(), residual.stride(0)
    if row_stats is not None:
        assert row_stats.dtype == torch.float32 and row_stats.is_contiguous() and row_stats.shape[0] == m and row_stats.shape[-1] == 2
        assert col_sums is not None and col_sums.dtype == torch.float32 and col_sums.numel() == n
        g.row_stats, g.col_sums = row_stats.data_ptr(), col_sums.data_ptr()
        if row_stats.dim() == 3:
            assert row_stats.shape[1] * 128 == k and stats_eps > 0
            g.stats_parts, g.stats_eps, g.stats_k = row_stats.shape[1], stats_eps, stats_k     # stats_k: true width of a zero-padded A
            g.stats_rms = int(stats_rms)       # RMSNorm: no mean; col_sums unused (zeros)
    if stats_out is not None:
        assert stats_out.dtype == torch.float32 and stats_out.is_contiguous() and tuple(stats_out.shape) == (m, n // 128, 2)
        g.stats_out = stats_out.data_ptr()
    if epi == _C.EPI_QKROPE:
        r = _C.QkRope()
        r.qn, r.kn, r.rope = qk_rope["qn"].data_ptr(), qk_rope["kn"].data_ptr(), qk_rope["rope"].data_ptr()
        r.pos, r.seq, r.slot = qk_rope["pos"].data_ptr(), qk_rope["seq"].data_ptr(), qk_rope["slot"].data_ptr()
        r.kcache_layer, r.vcache_layer = qk_rope["kcache"].data_ptr(), qk_rope["vcache"].data_ptr()
        r.kv_cap, r.eps = qk_rope["kv_cap"], qk_rope["eps"]
        g.qk_rope = C.pointer(r)
        g._keep = r
    return g, out


def gemm(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor, **kw) -> torch.Tensor:
    """One GEMM launch; arguments as in ``gemm_desc``."""
    g, out = gemm_desc(a, w, status, **kw)
    _C.check(_C.lib().ittai_gemm_bf16_launch(C.byref(g), _stream(a)))
    return out


def gemm_chain(descs, flags: torch.Tensor) -> None:
    """Up to four dependent GEMMs (``gemm_desc`` records; each reads its predecessor's output as ``a``) in one persistent
    launch.  ``flags``: int32 / uint32 device words, ``len(descs) * 2 * ceil(M / 256)`` of them, zero at launch."""
    n = len(descs)
    arr = (_C.Gemm * n)(*descs)
    m = descs[0].m
    assert flags.dtype in (torch.int32, torch.uint32) and flags.is_contiguous() and flags.numel() >= n * 2 * ((m + 255) // 256)
    _C.check(_C.lib().ittai_gemm_chain_launch(arr, n, flags.data_ptr(), _stream(flags)))


def row_stats(x: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``[rows, 2]``: mean and ``1/sqrt(var + eps)`` of every row of bf16 ``x``."""
    out = torch.empty(x.shape[0], 2, dtype=torch.float32, device=x.device) if out is None else out
    _C.check(_C.lib().ittai_row_stats(x.data_ptr(), x.stride(0), out.data_ptr(), x.shape[0], x.shape[1], eps, _stream(x)))
    return out


def fold_layernorm(w: torch.Tensor, bias: torch.Tensor | None, gain: torch.Tensor, beta: torch.Tensor):
    """Weights of ``Linear(LayerNorm(x))`` for the folded GEMM: returns (w' bf16 = gain (.) w along K, bias' fp32 = bias + w beta,
    column sums fp32 of the ROUNDED w', so that the epilogue's ``acc - mean * col_sum`` cancels exactly what the tensor
    cores accumulated).  Reference: the fold of ``src/ittai/siglip/kernel.py:523-525``."""
    wf = w.float()
    wp = (wf * gain.float()[None, :]).to(torch.bfloat16).contiguous()
    b = wf @ beta.float()
    if bias is not None:
        b = b + bias.float()
    return wp, b.contiguous(), wp.float().sum(dim=1).contiguous()


def attention(q, k, v, o, seqs: torch.Tensor, *, n_heads: int, group: int, head_dim: int, causal: bool, max_q_len: int,
              q_strides, k_strides, v_strides, o_strides, max_kv_len: int = 0, q_rows_total: int = 0, kv_rows_total: int = 0,
              status: torch.Tensor | None = None) -> None:
    """Flash attention over sequences described by ``seqs`` (int32 [n, 4] device: q row0, q rows, kv row0, kv rows).

    ``q_strides`` = (row, head), ``k_strides`` / ``v_strides`` = (row, head, seq), ``o_strides`` = (row, head), in elements;
    q, k, v, o are any bf16 tensors whose ``data_ptr`` is the origin those strides refer to.  ``q_rows_total``,
    ``kv_rows_total`` (rows of the matrices behind q and k/v) and ``status`` enable the tensor-memory kernel for short
    dense sequences; it reports a timed-out wait through ``status`` (see ``check_status``)."""
    a = _C.Attention()
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.q_row, a.q_head = q_strides
    a.k_row, a.k_head, a.k_seq = k_strides
    a.v_row, a.v_head, a.v_seq = v_strides
    a.o_row, a.o_head = o_strides
    a.seqs = seqs.data_ptr()
    a.n_seqs, a.n_heads, a.group, a.head_dim, a.causal, a.max_q_len = seqs.shape[0], n_heads, group, head_dim, int(causal), max_q_len
    a.max_kv_len, a.q_rows_total, a.kv_rows_total = max_kv_len, q_rows_total, kv_rows_total
    a.status = status.data_ptr() if status is not None else None
    _C.check(_C.lib().ittai_attention_launch(C.byref(a), _stream(q)))


def rmsnorm_rows(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(x) if out is None else out
    _C.check(_C.lib().ittai_rmsnorm_rows(x.data_ptr(), x.stride(0), gain.data_ptr(), out.data_ptr(), out.stride(0), x.shape[0], eps, _stream(x)))
    return out


def layernorm_rows(x: torch.Tensor, gain: torch.Tensor, beta: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(x) if out is None else out
    assert gain.dtype == torch.float32 and beta.dtype == torch.float32
    _C.check(_C.lib().ittai_layernorm_rows(x.data_ptr(), x.stride(0), gain.data_ptr(), beta.data_ptr(), out.data_ptr(), out.stride(0),
                                          x.shape[0], x.shape[1], eps, _stream(x)))
    return out
