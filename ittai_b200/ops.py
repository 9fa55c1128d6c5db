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


def gemm(a: torch.Tensor, w: torch.Tensor, status: torch.Tensor, bias: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, epi: int = _C.EPI_NONE, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = epilogue(a @ w.T)`` on the tcgen05 GEMM: a [M, K] and w [N, K] bf16 (last dim contiguous), bias fp32 [N],
    residual bf16 [M, N].  SwiGLU takes interleaved (gate, up) weight rows and returns [M, N/2]."""
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
    _C.check(_C.lib().ittai_gemm_bf16_launch(C.byref(g), _stream(a)))
    return out


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
