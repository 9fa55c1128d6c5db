"""SigLIP towers whose geometry the tensor-core kernels do not take as it is (so400m: width 1152, head_dim 72, MLP 4304,
patch 14): the same kernels on zero-padded weights.

The reference pads too (head_dim to a multiple of 16, the MLP width to a multiple of 128, the patch row to a multiple of
32, tokens per image to a multiple of 128: ``src/ittai/siglip/kernel.py:537-539,551-563``).  Here the widths go up to what
the kernels of this build take: model width and MLP width to multiples of 256 (the two-SM GEMM's tile), head_dim to 128
(the attention kernels know 64 and 128), the patch row to a multiple of 64.  Everything that is padding is zero and stays
zero: padded weight rows and bias entries are zero, so the padded columns of every activation are zero, so the padded
weight columns never contribute.  The softmax scale of the attention kernels is ``padded head_dim ** -0.5``; the q
projection is pre-scaled by ``sqrt(padded / true)`` so that the scores carry the true ``head_dim ** -0.5``.  LayerNorm runs
as its own pass over the true width (the statistics must not see the padding).  Tokens are packed, not padded.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.nn.functional as F

from .. import _C, ops


def _up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class PaddedEngine:
    """Same surface as ``Engine``: ``forward(inputs) -> bf16 [B, D]`` view of a persistent buffer, ``check()``, ``flops()``."""

    @torch.no_grad()
    def __init__(self, vm, B, graph=True, fold_ln=True, chain=True, **ignored):
        from .kernel import _vision_model
        vm = _vision_model(vm)
        cfg, emb = vm.config, vm.embeddings
        self.vm, self.B = vm, B
        self.conv = isinstance(emb.patch_embedding, torch.nn.Conv2d)
        D, Fm, H, p = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.patch_size
        self.D, self.F, self.H, self.L, self.p, self.eps = D, Fm, H, cfg.num_hidden_layers, p, cfg.layer_norm_eps
        self.img = getattr(cfg, "image_size", 0)
        hd = D // H
        if hd > 128 or hd * H != D:
            raise NotImplementedError(f"head_dim {hd}: the attention kernels take at most 128")
        self.hd, self.hdp = hd, 64 if hd <= 64 else 128
        self.Dp, self.Fp, self.Kp0 = _up(D, 256), _up(Fm, 256), 3 * p * p
        self.Kp = _up(self.Kp0, 64)
        self.S0 = emb.num_patches
        dev = next(vm.parameters()).device
        self.dev = dev
        Dp, Fp, hdp, Hp = self.Dp, self.Fp, self.hdp, H * self.hdp
        self.M = M = B * self.S0
        f = lambda t: t.detach().to(dev, torch.float32)
        bf = lambda t: t.to(torch.bfloat16).contiguous()

        def pad2(w, rows, cols):                     # fp32 [r, c] -> fp32 [rows, cols], zero-filled
            return F.pad(f(w), (0, cols - w.shape[1], 0, rows - w.shape[0]))

        def heads_out(w, b, scale=1.0):              # a projection INTO head space: [H*hd, D], [H*hd] -> [H*hdp, Dp], [H*hdp]
            w = F.pad(f(w).view(H, hd, D) * scale, (0, Dp - D, 0, hdp - hd)).reshape(Hp, Dp)
            b = F.pad(f(b).view(H, hd) * scale, (0, hdp - hd)).reshape(Hp)
            return w, b

        def heads_in(w):                             # a projection OUT OF head space: [D, H*hd] -> [Dp, H*hdp]
            return F.pad(f(w).view(D, H, hd), (0, hdp - hd, 0, 0, 0, Dp - D)).reshape(Dp, Hp)

        qs = math.sqrt(hdp / hd)
        pe = emb.patch_embedding
        self.wpe, self.bpe = bf(pad2(pe.weight.reshape(D, -1), Dp, self.Kp)), F.pad(f(pe.bias), (0, Dp - D)).contiguous()
        self.layers = []
        for lyr in vm.encoder.layers:
            a, m = lyr.self_attn, lyr.mlp
            parts = [heads_out(a.q_proj.weight, a.q_proj.bias, qs), heads_out(a.k_proj.weight, a.k_proj.bias), heads_out(a.v_proj.weight, a.v_proj.bias)]
            self.layers.append(dict(
                ln1=(f(lyr.layer_norm1.weight).contiguous(), f(lyr.layer_norm1.bias).contiguous()),
                ln2=(f(lyr.layer_norm2.weight).contiguous(), f(lyr.layer_norm2.bias).contiguous()),
                wqkv=bf(torch.cat([w for w, _ in parts])), bqkv=torch.cat([b for _, b in parts]).contiguous(),
                wo=bf(heads_in(a.out_proj.weight)), bo=F.pad(f(a.out_proj.bias), (0, Dp - D)).contiguous(),
                w1=bf(pad2(m.fc1.weight, Fp, Dp)), b1=F.pad(f(m.fc1.bias), (0, Fp - Fm)).contiguous(),
                w2=bf(pad2(m.fc2.weight, Dp, Fp)), b2=F.pad(f(m.fc2.bias), (0, Dp - D)).contiguous()))
        self.post = (f(vm.post_layernorm.weight).contiguous(), f(vm.post_layernorm.bias).contiguous())
        h = vm.head
        inw, inb = h.attention.in_proj_weight, h.attention.in_proj_bias
        # the probe's query does not depend on the image: projected once, as the eager module would (bf16 Linear), then laid
        # out in padded head space with the score scale folded in
        q = F.linear(h.probe[0].to(dev, torch.bfloat16), inw[:D].to(dev, torch.bfloat16), inb[:D].to(dev, torch.bfloat16)).float()
        self.probe_q = bf(F.pad(q.view(H, hd) * qs, (0, hdp - hd)).reshape(1, Hp))
        kv = [heads_out(inw[D:2 * D], inb[D:2 * D]), heads_out(inw[2 * D:], inb[2 * D:])]
        self.wkv, self.bkv = bf(torch.cat([w for w, _ in kv])), torch.cat([b for _, b in kv]).contiguous()
        self.who, self.bho = bf(heads_in(h.attention.out_proj.weight)), F.pad(f(h.attention.out_proj.bias), (0, Dp - D)).contiguous()
        self.hln = (f(h.layernorm.weight).contiguous(), f(h.layernorm.bias).contiguous())
        self.hw1, self.hb1 = bf(pad2(h.mlp.fc1.weight, Fp, Dp)), F.pad(f(h.mlp.fc1.bias), (0, Fp - Fm)).contiguous()
        self.hw2, self.hb2 = bf(pad2(h.mlp.fc2.weight, Dp, Fp)), F.pad(f(h.mlp.fc2.bias), (0, Dp - D)).contiguous()
        # LayerNorm folded into the GEMM that follows it (as in ``Engine``): W' = W * gain along K (zero in the padding
        # columns), row sums of the rounded W', bias' = bias + W beta; the producing GEMM's epilogue writes the row sums
        # and the consuming epilogue finishes mean and rstd over the TRUE width (``stats_k``).
        self.fold_ln = bool(fold_ln) and M > 128
        self.chain = bool(chain) and self.fold_ln and M >= 1024

        def folded(w_bf16, bias, ln):
            g, beta = (F.pad(t, (0, Dp - D)) for t in ln)
            wf = w_bf16.float()
            wp = (wf * g).to(torch.bfloat16).contiguous()
            return wp, (bias + wf @ beta).contiguous(), wp.float().sum(1).contiguous()

        if self.fold_ln:
            for w in self.layers:
                w["qkv_f"] = folded(w["wqkv"], w["bqkv"], w["ln1"])
                w["fc1_f"] = folded(w["w1"], w["b1"], w["ln2"])
            self.kv_f = folded(self.wkv, self.bkv, self.post)
            self.stats_a = torch.zeros(M, Dp // 128, 2, dtype=torch.float32, device=dev)
            self.stats_m = torch.zeros(M, Dp // 128, 2, dtype=torch.float32, device=dev)
            self.chain_flags = torch.zeros(len(self.layers) + 1, 4 * 2 * ((M + 255) // 256), dtype=torch.int32, device=dev)
        z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
        self.pos = z(M, Dp)
        if self.conv:
            self.pos[:, :D] = emb.position_embedding.weight.detach().to(dev, torch.bfloat16).repeat(B, 1)
            self.pixels = torch.empty(B, 3, self.img, self.img, dtype=torch.float32, device=dev)
        else:
            side = int(round(self.S0 ** 0.5))
            self.pos_grid = f(emb.position_embedding.weight).reshape(side, side, D)
        self.patches, self.x, self.y = z(M, self.Kp), z(M, Dp), z(M, Dp)
        self.qkv, self.attn, self.h = z(M, 3 * Hp), z(M, Hp), z(M, Fp)
        self.kv, self.pool_a, self.pool_r, self.pool_y, self.pool_h = z(M, 2 * Hp), z(B, Hp), z(B, Dp), z(B, Dp), z(B, Fp)
        self.embeds_p = z(B, Dp)
        S = self.S0
        self.seqs = torch.tensor([[b * S, S, b * S, S] for b in range(B)], dtype=torch.int32, device=dev)
        self.pool_seqs = torch.tensor([[b, 1, b * S, S] for b in range(B)], dtype=torch.int32, device=dev)
        self.status = ops.new_status(dev)
        self.graph = None if graph else False

    def _body(self):
        D, S, B, H, hdp, eps, st = self.D, self.S0, self.B, self.H, self.hdp, self.eps, self.status
        Hp = H * hdp
        if self.conv:       # patch rows in (channel, row, column) order: what a Conv2d weight flattens to; the padding columns stay zero
            _C.check(_C.lib().ittai_siglip_im2col(self.pixels.data_ptr(), self.patches.data_ptr(), B, self.img, self.img, self.p, self.Kp,
                                                  ops._stream(self.pixels)))
        att = dict(n_heads=H, group=1, head_dim=hdp, causal=False)

        def attention():
            # row totals + status words: the tcgen05 key-loop kernel (head_dim 128, keys and values packed like the queries)
            ops.attention(self.qkv, self.qkv[:, Hp:], self.qkv[:, 2 * Hp:], self.attn, self.seqs, max_q_len=S, q_strides=(3 * Hp, hdp),
                          k_strides=(3 * Hp, hdp, 0), v_strides=(3 * Hp, hdp, 0), o_strides=(Hp, hdp), max_kv_len=S,
                          q_rows_total=self.M, kv_rows_total=self.M, status=st, **att)

        if self.fold_ln:
            ln = dict(stats_eps=eps, stats_k=D)
            embed = ops.gemm_desc(self.patches, self.wpe, st, bias=self.bpe, residual=self.pos, out=self.x, stats_out=self.stats_m)[0]
            qkv = lambda w: ops.gemm_desc(self.x, w["qkv_f"][0], st, bias=w["qkv_f"][1], out=self.qkv, row_stats=self.stats_m,
                                          col_sums=w["qkv_f"][2], **ln)[0]
            run = (lambda descs, flags: ops.gemm_chain(descs, flags)) if self.chain else \
                  (lambda descs, flags: [_C.check(_C.lib().ittai_gemm_bf16_launch(C.byref(d), ops._stream(self.x))) for d in descs])
            if self.chain:
                self.chain_flags.zero_()
            run([embed, qkv(self.layers[0])], self.chain_flags[len(self.layers)])
            for i, w in enumerate(self.layers):
                attention()
                descs = [ops.gemm_desc(self.attn, w["wo"], st, bias=w["bo"], residual=self.x, out=self.x, stats_out=self.stats_a)[0],
                         ops.gemm_desc(self.x, w["fc1_f"][0], st, bias=w["fc1_f"][1], epi=_C.EPI_GELU, out=self.h, row_stats=self.stats_a,
                                       col_sums=w["fc1_f"][2], **ln)[0],
                         ops.gemm_desc(self.h, w["w2"], st, bias=w["b2"], residual=self.x, out=self.x, stats_out=self.stats_m)[0]]
                descs.append(qkv(self.layers[i + 1]) if i + 1 < len(self.layers) else
                             ops.gemm_desc(self.x, self.kv_f[0], st, bias=self.kv_f[1], out=self.kv, row_stats=self.stats_m, col_sums=self.kv_f[2], **ln)[0])
                run(descs, self.chain_flags[i])
        else:
            ops.gemm(self.patches, self.wpe, st, bias=self.bpe, residual=self.pos, out=self.x)
            for w in self.layers:
                ops.layernorm_rows(self.x[:, :D], *w["ln1"], eps, out=self.y[:, :D])
                ops.gemm(self.y, w["wqkv"], st, bias=w["bqkv"], out=self.qkv)
                attention()
                ops.gemm(self.attn, w["wo"], st, bias=w["bo"], residual=self.x, out=self.x)
                ops.layernorm_rows(self.x[:, :D], *w["ln2"], eps, out=self.y[:, :D])
                ops.gemm(self.y, w["w1"], st, bias=w["b1"], epi=_C.EPI_GELU, out=self.h)
                ops.gemm(self.h, w["w2"], st, bias=w["b2"], residual=self.x, out=self.x)
            # post-LayerNorm + MAP head: the probe attends over the image's tokens, then LayerNorm + MLP with a residual
            ops.layernorm_rows(self.x[:, :D], *self.post, eps, out=self.y[:, :D])
            ops.gemm(self.y, self.wkv, st, bias=self.bkv, out=self.kv)
        ops.attention(self.probe_q, self.kv, self.kv[:, Hp:], self.pool_a, self.pool_seqs, max_q_len=1, q_strides=(0, hdp),
                      k_strides=(2 * Hp, hdp, 0), v_strides=(2 * Hp, hdp, 0), o_strides=(Hp, hdp), **att)
        ops.gemm(self.pool_a, self.who, st, bias=self.bho, out=self.pool_r)
        ops.layernorm_rows(self.pool_r[:, :D], *self.hln, eps, out=self.pool_y[:, :D])
        ops.gemm(self.pool_y, self.hw1, st, bias=self.hb1, epi=_C.EPI_GELU, out=self.pool_h)
        ops.gemm(self.pool_h, self.hw2, st, bias=self.hb2, residual=self.pool_r, out=self.embeds_p)

    @torch.no_grad()
    def forward(self, inp):
        from .kernel import resize_positions
        px = inp["pixel_values"]
        if self.conv:
            assert tuple(px.shape) == tuple(self.pixels.shape), f"expected {tuple(self.pixels.shape)}, got {tuple(px.shape)}"
            self.pixels.copy_(px, non_blocking=True)
        else:
            S = self.S0
            assert tuple(px.shape) == (self.B, S, self.Kp0), f"expected {(self.B, S, self.Kp0)}, got {tuple(px.shape)}"
            mask, shapes = inp["pixel_attention_mask"], torch.as_tensor(inp["spatial_shapes"])
            key_len = mask.to(torch.int64).sum(1).cpu()
            if not torch.equal(key_len, shapes.to(torch.int64).cpu().prod(1)) or int(key_len.min()) < 1:
                raise ValueError("pixel_attention_mask must mark exactly height * width leading rows of every image")
            self.patches[:, :self.Kp0].copy_(px.reshape(self.M, -1), non_blocking=True)
            self.pos[:, :self.D].copy_(resize_positions(self.pos_grid, shapes.tolist(), S).reshape(self.M, -1))
            kl = key_len.to(torch.int32).to(self.dev, non_blocking=True)
            self.seqs[:, 3].copy_(kl)
            self.pool_seqs[:, 3].copy_(kl)
        if self.graph is None:
            self.status.zero_()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._body()
            torch.cuda.current_stream().wait_stream(s)
            ops.check_status(self.status)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._body()
        if self.graph:
            self.graph.replay()
        else:
            self._body()
        return self.embeds_p[:, :self.D]

    def check(self) -> None:
        ops.check_status(self.status)

    def launches_per_forward(self) -> int:
        """Kernels in one forward (all inside one CUDA graph)."""
        n_l = len(self.layers)
        encoder = (n_l + 1) + n_l if self.chain else 1 + n_l * (5 if self.fold_ln else 7) + (1 if self.fold_ln else 2)
        return (1 if self.conv else 0) + encoder + 5

    def flops(self, formula: str = "reference") -> float:
        """FLOPs of one forward at the TRUE widths (the padding is overhead, not work); formulas as in ``Engine.flops``."""
        B, L, S, D, Fm = self.B, self.L, self.S0, self.D, self.F
        ref = B * L * (2 * S * D * (4 * D + 2 * Fm) + 4 * S * S * D)
        if formula == "reference":
            return float(ref)
        head = 2 * S * D * 2 * D + 4 * S * D + 2 * D * D + 4 * D * Fm
        return float(ref + B * (2 * S * D * self.Kp0 + head))
