"""CPU restatement of the SigLIP ViT-B/16 vision tower, every bf16 rounding point explicit.

TEST INFRASTRUCTURE ONLY.  Follows ``transformers``' SigLIP modules, which the reference loads and checks itself
against (reference ``src/ittai/siglip/kernel.py:675,701-702``): Conv2d patch embedding as a matrix product over
(channel, row, col)-ordered patches (``:633-637``), learned position add, pre-LayerNorm blocks with scale
head_dim**-0.5 (``:54``) and GELU-tanh (``:289-291``), post-LayerNorm, and the MAP head (probe attention over the
tokens, then LayerNorm + MLP with a residual; ``:626-629``).  Tensors are fp32 holding bf16 values.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def r(x):
    return x.to(torch.bfloat16).to(torch.float32)


def ln(x, w, b, eps):
    return r(F.layer_norm(x, (x.shape[-1],), w, b, eps))


def lin(x, w, b):
    return r(x @ w.t() + b)


class SiglipRef:
    def __init__(self, vision_model):
        vm = vision_model.vision_model if hasattr(vision_model, "vision_model") else vision_model
        f = lambda t: t.detach().float().cpu()
        self.cfg = vm.config
        e = vm.embeddings
        self.p = self.cfg.patch_size
        self.wpe, self.bpe = f(e.patch_embedding.weight).reshape(self.cfg.hidden_size, -1), f(e.patch_embedding.bias)
        self.pos = f(e.position_embedding.weight)
        self.layers = []
        for lyr in vm.encoder.layers:
            a, m = lyr.self_attn, lyr.mlp
            self.layers.append({k: f(v) for k, v in dict(
                ln1w=lyr.layer_norm1.weight, ln1b=lyr.layer_norm1.bias, ln2w=lyr.layer_norm2.weight, ln2b=lyr.layer_norm2.bias,
                wq=a.q_proj.weight, bq=a.q_proj.bias, wk=a.k_proj.weight, bk=a.k_proj.bias, wv=a.v_proj.weight, bv=a.v_proj.bias,
                wo=a.out_proj.weight, bo=a.out_proj.bias, w1=m.fc1.weight, b1=m.fc1.bias, w2=m.fc2.weight, b2=m.fc2.bias).items()})
        self.postw, self.postb = f(vm.post_layernorm.weight), f(vm.post_layernorm.bias)
        h = vm.head
        self.probe = f(h.probe)[0]
        self.inw, self.inb = f(h.attention.in_proj_weight), f(h.attention.in_proj_bias)
        self.ow, self.ob = f(h.attention.out_proj.weight), f(h.attention.out_proj.bias)
        self.hlnw, self.hlnb = f(h.layernorm.weight), f(h.layernorm.bias)
        self.hw1, self.hb1, self.hw2, self.hb2 = f(h.mlp.fc1.weight), f(h.mlp.fc1.bias), f(h.mlp.fc2.weight), f(h.mlp.fc2.bias)

    def forward(self, pixels: torch.Tensor):
        """pixels fp32 [B, 3, H, W] -> (pooled [B, D], last_hidden_state after post-LayerNorm [B, S, D])."""
        c, p, eps = self.cfg, self.p, self.cfg.layer_norm_eps
        B, D, H = pixels.shape[0], c.hidden_size, c.num_attention_heads
        hd = D // H
        px = r(pixels)
        patches = px.unfold(2, p, p).unfold(3, p, p).permute(0, 2, 3, 1, 4, 5).reshape(B, -1, 3 * p * p)
        x = r(lin(patches, self.wpe, self.bpe) + self.pos)
        S = x.shape[1]
        for w in self.layers:
            y = ln(x, w["ln1w"], w["ln1b"], eps)
            q, k, v = (lin(y, w["w" + n], w["b" + n]).view(B, S, H, hd).transpose(1, 2) for n in "qkv")
            a = r(torch.softmax(q @ k.transpose(-1, -2) * hd ** -0.5, -1) @ v).transpose(1, 2).reshape(B, S, D)
            x = r(x + lin(a, w["wo"], w["bo"]))
            y = ln(x, w["ln2w"], w["ln2b"], eps)
            x = r(x + lin(r(F.gelu(lin(y, w["w1"], w["b1"]), approximate="tanh")), w["w2"], w["b2"]))
        x = ln(x, self.postw, self.postb, eps)
        q = lin(self.probe, self.inw[:D], self.inb[:D]).view(1, H, 1, hd)
        k = lin(x, self.inw[D:2 * D], self.inb[D:2 * D]).view(B, S, H, hd).transpose(1, 2)
        v = lin(x, self.inw[2 * D:], self.inb[2 * D:]).view(B, S, H, hd).transpose(1, 2)
        a = r(torch.softmax(q @ k.transpose(-1, -2) * hd ** -0.5, -1) @ v).transpose(1, 2).reshape(B, D)
        res = lin(a, self.ow, self.ob)
        y = ln(res, self.hlnw, self.hlnb, eps)
        pooled = r(res + lin(r(F.gelu(lin(y, self.hw1, self.hb1), approximate="tanh")), self.hw2, self.hb2))
        return pooled, x
