"""CPU restatement of the Qwen3 decoder arithmetic, every bf16 rounding point explicit.

TEST INFRASTRUCTURE ONLY: imported by tests, the smoke check and the benchmark's CPU legs.

The arithmetic follows ``transformers``' Qwen3 modules, the implementation the reference loads and
checks itself against (reference ``src/ittai/qwen3/model.py:19,32-37``): RMSNorm with fp32 variance
then a bf16 cast and a bf16 multiply by the weight; per-head q/k RMSNorm before RoPE; rotate-half
RoPE with cos/sin cast to bf16; GQA with scale head_dim**-0.5; SwiGLU with a bf16 SiLU; bf16
residual adds; tied lm_head.  The reference's own packed formulation of the same math (weights
folded with the norm gain, rstd applied after the GEMM, adjacent-pair RoPE) is in
``src/ittai/qwen3/base.py:80-145`` and ``src/ittai/qwen3/engine.py:100-122``; the values are the
same up to rounding, and this file keeps the unfolded form because its rounding points are the
ones the CUDA decode phases reproduce.

All tensors are fp32 holding bf16-representable values; ``r`` rounds to bf16 and back.
Pinned against Hugging Face outputs in ``tests/test_oracle.py``.
"""
from __future__ import annotations

import torch

from .qwen3_hf import Qwen3Dims


def r(x: torch.Tensor) -> torch.Tensor:
    """Round fp32 to the nearest bf16 (ties to even) and widen back."""
    return x.to(torch.bfloat16).to(torch.float32)


def rope_table(n_pos: int, dims: Qwen3Dims):
    """cos/sin tables [n_pos, head_dim/2] rounded to bf16, as the rotary module hands them to bf16 q/k.

    Angle = pos * theta**(-2i/head_dim) in fp32 (reference ``src/ittai/qwen3/engine.py:118-122``
    builds the same angles; there they stay fp32, in ``transformers`` they are cast to the model dtype).
    """
    hd = dims.head_dim
    inv = 1.0 / (dims.theta ** (torch.arange(0, hd, 2, dtype=torch.int64).to(torch.float32) / hd))
    ang = torch.arange(n_pos, dtype=torch.float32)[:, None] * inv[None, :]
    return r(ang.cos()), r(ang.sin())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """bf16(bf16(x * rsqrt(mean(x^2) + eps)) * w) along the last axis."""
    var = (x * x).mean(-1, keepdim=True)
    return r(r(x * torch.rsqrt(var + eps)) * w)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE in bf16 steps: bf16(bf16(x*cos) + bf16(rot(x)*sin)); x [..., head_dim]."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    lo = r(r(x1 * cos) + r(-x2 * sin))
    hi = r(r(x2 * cos) + r(x1 * sin))
    return torch.cat([lo, hi], -1)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """bf16(x @ w.T) with fp32 accumulation."""
    return r(x @ w.t())


class Qwen3Ref:
    """Batch-1 decoder with a KV cache [L, n_kv, cap, head_dim], driven a token at a time or by prefill."""

    def __init__(self, sd: dict, dims: Qwen3Dims, kv_cap: int):
        self.d = dims
        f = lambda k: sd[k].detach().to(torch.float32).cpu()
        pre = "model." if any(k.startswith("model.") for k in sd) else ""
        self.embed = f(pre + "embed_tokens.weight")
        self.fin_w = f(pre + "norm.weight")
        self.layers = []
        for l in range(dims.n_layers):
            p = f"{pre}layers.{l}."
            self.layers.append(dict(
                ln1=f(p + "input_layernorm.weight"), ln2=f(p + "post_attention_layernorm.weight"),
                wq=f(p + "self_attn.q_proj.weight"), wk=f(p + "self_attn.k_proj.weight"),
                wv=f(p + "self_attn.v_proj.weight"), wo=f(p + "self_attn.o_proj.weight"),
                qn=f(p + "self_attn.q_norm.weight"), kn=f(p + "self_attn.k_norm.weight"),
                wg=f(p + "mlp.gate_proj.weight"), wu=f(p + "mlp.up_proj.weight"),
                wd=f(p + "mlp.down_proj.weight")))
        self.cos, self.sin = rope_table(kv_cap, dims)
        self.k = torch.zeros(dims.n_layers, dims.n_kv_heads, kv_cap, dims.head_dim)
        self.v = torch.zeros_like(self.k)
        self.len = 0

    def forward(self, ids: torch.Tensor, trace: list | None = None) -> torch.Tensor:
        """Append ``ids`` (any count >= 1) at positions len.., return bf16-valued logits of the last one.

        With ``trace`` a dict of the last token's intermediates is appended per layer (what each decode phase
        leaves in its output buffer): qkv (raw projections), attn, h_mid (after o_proj), act, h (after down).
        """
        d = self.d
        T, p0 = len(ids), self.len
        pos = torch.arange(p0, p0 + T)
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]      # [T,1,hd/2]
        h = self.embed[ids]
        scale = d.head_dim ** -0.5
        g = d.n_heads // d.n_kv_heads
        causal = torch.arange(p0 + T)[None, :] <= pos[:, None]               # [T, p0+T]
        for l, w in enumerate(self.layers):
            x = rmsnorm(h, w["ln1"], d.eps)
            q = linear(x, w["wq"]).view(T, d.n_heads, d.head_dim)
            k = linear(x, w["wk"]).view(T, d.n_kv_heads, d.head_dim)
            v = linear(x, w["wv"]).view(T, d.n_kv_heads, d.head_dim)
            t = dict(qkv=torch.cat([q[-1].flatten(), k[-1].flatten(), v[-1].flatten()])) if trace is not None else None
            q = rope(rmsnorm(q, w["qn"], d.eps), cos, sin)
            k = rope(rmsnorm(k, w["kn"], d.eps), cos, sin)
            self.k[l, :, p0:p0 + T] = k.transpose(0, 1)
            self.v[l, :, p0:p0 + T] = v.transpose(0, 1)
            K = self.k[l, :, :p0 + T].repeat_interleave(g, 0)                # [nh, S, hd]
            V = self.v[l, :, :p0 + T].repeat_interleave(g, 0)
            s = torch.einsum("thd,hsd->hts", q, K) * scale
            s = s.masked_fill(~causal[None], float("-inf"))
            a = r(torch.einsum("hts,hsd->thd", torch.softmax(s, -1), V)).reshape(T, -1)
            h = r(h + linear(a, w["wo"]))
            h_mid = h
            x = rmsnorm(h, w["ln2"], d.eps)
            gate, up = linear(x, w["wg"]), linear(x, w["wu"])
            act = r(r(gate * torch.sigmoid(gate)) * up)
            h = r(h + linear(act, w["wd"]))
            if trace is not None:
                t.update(attn=a[-1], h_mid=h_mid[-1], act=act[-1], h=h[-1])
                trace.append(t)
        self.len = p0 + T
        self.h_last = h[-1]
        return linear(rmsnorm(h[-1:], self.fin_w, d.eps), self.embed)[0]

    def greedy(self, ids: torch.Tensor, n_steps: int, forced: torch.Tensor | None = None):
        """Same contract as ``qwen3_hf.greedy``: (next_ids[n_steps], logits[n_steps, V])."""
        logits = [self.forward(ids)]
        picks = [int(logits[-1].argmax())]
        for s in range(1, n_steps):
            feed = picks[-1] if forced is None else int(forced[s - 1])
            logits.append(self.forward(torch.tensor([feed])))
            picks.append(int(logits[-1].argmax()))
        return torch.tensor(picks, dtype=torch.int64), torch.stack(logits)

    def embed_pool(self) -> torch.Tensor:
        """L2-normalised final-norm of the last token (reference ``src/ittai/qwen3/base.py:131-145``)."""
        y = self.h_last * torch.rsqrt((self.h_last ** 2).mean() + self.d.eps) * self.fin_w
        return y / y.norm()
