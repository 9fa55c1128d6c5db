"""SigLIP vision tower on the B200 kernels, behind the reference's ``Engine`` / ``Siglip2Embedder`` surface
(reference ``src/ittai/siglip/kernel.py:532-723``).

What runs where: patch gather, LayerNorm and attention are row-wise / flash kernels; every Linear (patch embedding,
qkv, out-proj, fc1 + GELU-tanh, fc2 + residual, and the MAP head's projections) is the tcgen05 GEMM with its fused
epilogue; the whole forward, MAP pooling head included, is one CUDA graph.  The reference keeps the post-LayerNorm and
the MAP head in torch (``:626-629``) and computes in fp16 with fp16 accumulation (``:42,73``); here everything is bf16
storage with fp32 accumulation, and the rounding points are the eager modules'.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _C, ops


def fold_ln(W, b, g, beta, dtype=torch.bfloat16):
    """LayerNorm folded into the Linear that follows it, under the reference's name and return order
    (``src/ittai/siglip/kernel.py:523-525``): ``(W' = W * gain in `dtype`, row sums of the rounded W' in fp32,
    b' = b + W beta in fp32)``."""
    wp, bias, sums = ops.fold_layernorm(W, b, g, beta)
    return wp.to(dtype), sums, bias


def gemm_tasks(op, l, nm, nn, group_m):
    """``(op, layer, row block, column tile)`` of one GEMM in queue order: row blocks in groups of ``group_m``, and inside a
    group the column tile outermost, so that neighbouring tasks share a weight tile (reference ``kernel.py:528-529``)."""
    order = []
    for first in range(0, nm, group_m):
        rows = range(first, min(first + group_m, nm))
        order.extend((op, l, i, j) for j in range(nn) for i in rows)
    return order


def resize_positions(grid: torch.Tensor, shapes, max_len: int) -> torch.Tensor:
    """Position rows of variable-resolution (NaFlex) images: the learned ``[side, side, D]`` grid resized to every image's
    ``(height, width)`` patch grid (bilinear, antialiased, in fp32), flattened row-major and padded to ``max_len`` rows with
    the image's first row, as the eager embedding module does and the reference's ``_prepare`` restates
    (``src/ittai/siglip/kernel.py:638-649``).  ``grid``: fp32 ``[side, side, D]``; returns fp32 ``[B, max_len, D]``."""
    g = grid.permute(2, 0, 1)[None].float()
    shapes = [tuple(int(v) for v in hw) for hw in shapes]
    out = torch.empty(len(shapes), max_len, grid.shape[-1], dtype=torch.float32, device=grid.device)
    for hw in set(shapes):
        if hw[0] < 1 or hw[1] < 1 or hw[0] * hw[1] > max_len:
            raise ValueError(f"patch grid {hw} does not fit {max_len} positions")
        rows = torch.nn.functional.interpolate(g, size=hw, mode="bilinear", align_corners=False, antialias=True)[0].flatten(1).t()
        idx = [k for k, v in enumerate(shapes) if v == hw]
        out[idx, :len(rows)] = rows
        out[idx, len(rows):] = rows[0]
    return out


def _vision_model(m):
    return m.vision_model if hasattr(m, "vision_model") else m


def fits_fast_path(cfg) -> bool:
    """Whether a tower's widths are the ones the fused path is written for: head_dim 64, model and MLP width multiples of
    128 (256 for the two-SM GEMM's tile comes with them for ViT-B), patch rows a multiple of 64 values."""
    D, H, Fm, p = cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size, cfg.patch_size
    return D % H == 0 and D // H == 64 and D % 256 == 0 and Fm % 256 == 0 and (3 * p * p) % 64 == 0


class Engine:
    """``Engine(vm, B)``: fixed batch ``B``; ``forward({"pixel_values": fp32 [B,3,H,W]})`` returns bf16 ``[B, D]`` pooled
    embeddings (a persistent buffer, like the reference's ``self.embeds``).  The reference's tuning arguments
    (``tile_n, stages, warps, fold_k, group_m, kv_block``) are accepted and ignored: there is one sm_100a kernel."""

    def __new__(cls, vm, B, *args, **kw):
        """ViT-B-like geometries (head_dim 64, widths in multiples of 128) get this class; anything else (so400m: width
        1152, head_dim 72, MLP 4304, patch 14) the same kernels on zero-padded weights (``padded.PaddedEngine``)."""
        if cls is Engine and not fits_fast_path(_vision_model(vm).config):
            from .padded import PaddedEngine
            return PaddedEngine(vm, B, **{k: v for k, v in kw.items() if k in ("graph", "fold_ln", "chain")})
        return super().__new__(cls)

    @torch.no_grad()
    def __init__(self, vm, B, tile_n=None, stages=None, warps=None, fold_k=None, group_m=None, kv_block=64, graph=True, fold_ln=True, chain=True):
        vm = _vision_model(vm)
        cfg, emb = vm.config, vm.embeddings
        # Conv2d patch embedding: fixed resolution.  Linear: SigLIP2 NaFlex, whose inputs arrive as patch rows with a
        # validity mask and a per-image patch grid (reference ``:574-578, 638-649``).
        self.conv = isinstance(emb.patch_embedding, torch.nn.Conv2d)
        self.vm, self.B = vm, B
        self.D, self.F, self.H, self.L = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_hidden_layers
        self.p, self.eps, self.img = cfg.patch_size, cfg.layer_norm_eps, getattr(cfg, "image_size", 0)
        self.hd = self.D // self.H
        self.S0 = emb.num_patches
        if self.hd != 64 or self.D % 128 or self.F % 128 or (3 * self.p * self.p) % 64:
            raise NotImplementedError("this build covers head_dim 64 and widths that are multiples of 128 (ViT-B/16)")
        dev = next(vm.parameters()).device
        self.dev = dev
        D, S, M = self.D, self.S0, B * self.S0
        self.M = M
        bf = lambda t: t.detach().to(dev, torch.bfloat16).contiguous()
        f32 = lambda t: t.detach().to(dev, torch.float32).contiguous()
        self.wpe, self.bpe = bf(emb.patch_embedding.weight.reshape(D, -1)), f32(emb.patch_embedding.bias)
        # position table repeated per image: the patch-embedding GEMM adds it as its residual (reference :569-571)
        if self.conv:
            self.pos = bf(emb.position_embedding.weight).repeat(B, 1)
        else:
            side = int(round(S ** 0.5))
            self.pos_grid = f32(emb.position_embedding.weight).reshape(side, side, D)
            self.pos = torch.zeros(M, D, dtype=torch.bfloat16, device=dev)
        self.layers = []
        for lyr in vm.encoder.layers:
            a, m = lyr.self_attn, lyr.mlp
            self.layers.append(dict(
                ln1=(f32(lyr.layer_norm1.weight), f32(lyr.layer_norm1.bias)), ln2=(f32(lyr.layer_norm2.weight), f32(lyr.layer_norm2.bias)),
                wqkv=bf(torch.cat([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight])),
                bqkv=f32(torch.cat([a.q_proj.bias, a.k_proj.bias, a.v_proj.bias])),
                wo=bf(a.out_proj.weight), bo=f32(a.out_proj.bias), w1=bf(m.fc1.weight), b1=f32(m.fc1.bias),
                w2=bf(m.fc2.weight), b2=f32(m.fc2.bias)))
        self.post = (f32(vm.post_layernorm.weight), f32(vm.post_layernorm.bias))
        # LayerNorm folded into the GEMMs around it, as the reference does (``:284-288, 335-364, 523-525``): the GEMM that
        # writes the residual stream also writes its row statistics, the GEMM that consumes it reads the stream itself and
        # applies mean / rstd in its epilogue, so there is no LayerNorm pass and the normalised activations are never
        # written.  ``fold_ln=False`` keeps the separate LayerNorm kernel, whose rounding points are exactly the eager
        # module's (the folded path rounds the gain-scaled weights instead of the normalised activations).
        self.fold_ln = fold_ln and B * emb.num_patches > 128
        if self.fold_ln:
            for w in self.layers:
                w["qkv_f"] = ops.fold_layernorm(w["wqkv"], w["bqkv"], *w["ln1"])
                w["fc1_f"] = ops.fold_layernorm(w["w1"], w["b1"], *w["ln2"])
        h = vm.head
        inw, inb = h.attention.in_proj_weight, h.attention.in_proj_bias
        # the probe is a parameter, so its query projection does not depend on the image: computed once, as the eager
        # module would (bf16 Linear)
        self.probe_q = bf(torch.nn.functional.linear(h.probe[0].to(torch.bfloat16), inw[:D].to(torch.bfloat16), inb[:D].to(torch.bfloat16)))
        self.wkv, self.bkv = bf(inw[D:]), f32(inb[D:])
        if self.fold_ln:
            self.kv_f = ops.fold_layernorm(self.wkv, self.bkv, *self.post)
        self.who, self.bho = bf(h.attention.out_proj.weight), f32(h.attention.out_proj.bias)
        self.hln = (f32(h.layernorm.weight), f32(h.layernorm.bias))
        self.hw1, self.hb1, self.hw2, self.hb2 = bf(h.mlp.fc1.weight), f32(h.mlp.fc1.bias), bf(h.mlp.fc2.weight), f32(h.mlp.fc2.bias)
        z = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)
        self.pixels = torch.empty(B, 3, self.img, self.img, dtype=torch.float32, device=dev) if self.conv else None
        self.patches, self.x, self.y = z(M, 3 * self.p * self.p), z(M, D), z(M, D)
        self.qkv, self.attn, self.h = z(M, 3 * D), z(M, D), z(M, self.F)
        self.kv, self.pool_a, self.pool_r, self.pool_y, self.pool_h = z(M, 2 * D), z(B, D), z(B, D), z(B, D), z(B, self.F)
        self.embeds = z(B, D)
        self.seqs = torch.tensor([[b * S, S, b * S, S] for b in range(B)], dtype=torch.int32, device=dev)
        self.pool_seqs = torch.tensor([[b, 1, b * S, S] for b in range(B)], dtype=torch.int32, device=dev)
        # per-row (sum, sum of squares) of the residual stream in 128-column slices, written by the epilogue of the GEMM that
        # produces it: one buffer for the stream after attention, one for the stream after the MLP
        self.stats_a = torch.zeros(M, D // 128, 2, dtype=torch.float32, device=dev)
        self.stats_m = torch.zeros(M, D // 128, 2, dtype=torch.float32, device=dev)
        # ``chain``: the GEMMs between two attention kernels (out-proj, fc1, fc2, the next layer's QKV) run as ONE
        # persistent launch whose tiles wait on per-row-block counters, like the tasks of the reference's persistent kernel
        # (reference ``:197-333``); needs the folded LayerNorms (no kernel of another kind between the GEMMs) and M > 128
        self.chain = bool(chain) and self.fold_ln and M >= 1024      # a few row blocks only: nothing to overlap, one launch per GEMM is faster
        self.chain_flags = torch.zeros(len(self.layers) + 1, 4 * 2 * ((M + 255) // 256), dtype=torch.int32, device=dev)
        self.status = ops.new_status(dev)
        self.graph = None if graph else False

    def _body(self):
        D, S, B, H, hd, eps = self.D, self.S0, self.B, self.H, self.hd, self.eps
        L, st = _C.lib(), self.status
        if self.conv:
            _C.check(L.ittai_siglip_im2col(self.pixels.data_ptr(), self.patches.data_ptr(), B, self.img, self.img, self.p, 0,
                                           ops._stream(self.pixels)))
        fold = self.fold_ln
        # with variable-resolution inputs an image's keys are its first key_len rows (the records in `seqs` say how many);
        # the tensor-memory kernel takes up to 256 keys and queries per image, longer sequences fall to the register tiles
        kv_max = S
        embed = dict(bias=self.bpe, residual=self.pos, out=self.x, stats_out=self.stats_m if fold else None)
        if not self.chain:
            ops.gemm(self.patches, self.wpe, st, **embed)
        def attention():
            ops.attention(self.qkv, self.qkv[:, D:], self.qkv[:, 2 * D:], self.attn, self.seqs, n_heads=H, group=1, head_dim=hd,
                          causal=False, max_q_len=S, q_strides=(3 * D, hd), k_strides=(3 * D, hd, 0), v_strides=(3 * D, hd, 0),
                          o_strides=(D, hd), max_kv_len=kv_max, q_rows_total=self.M, kv_rows_total=self.M, status=st)

        if self.chain:
            self.chain_flags.zero_()
            qkv = lambda w: ops.gemm_desc(self.x, w["qkv_f"][0], st, bias=w["qkv_f"][1], out=self.qkv, row_stats=self.stats_m,
                                          col_sums=w["qkv_f"][2], stats_eps=eps)[0]
            # patch embedding + the first QKV projection; then per layer out-proj, fc1, fc2 and the next layer's QKV (after
            # the last layer: the K/V projection of the pooling head)
            ops.gemm_chain([ops.gemm_desc(self.patches, self.wpe, st, **embed)[0], qkv(self.layers[0])], self.chain_flags[len(self.layers)])
            for i, w in enumerate(self.layers):
                attention()
                descs = [ops.gemm_desc(self.attn, w["wo"], st, bias=w["bo"], residual=self.x, out=self.x, stats_out=self.stats_a)[0],
                         ops.gemm_desc(self.x, w["fc1_f"][0], st, bias=w["fc1_f"][1], epi=_C.EPI_GELU, out=self.h, row_stats=self.stats_a,
                                       col_sums=w["fc1_f"][2], stats_eps=eps)[0],
                         ops.gemm_desc(self.h, w["w2"], st, bias=w["b2"], residual=self.x, out=self.x, stats_out=self.stats_m)[0]]
                if i + 1 < len(self.layers):
                    descs.append(qkv(self.layers[i + 1]))
                else:
                    descs.append(ops.gemm_desc(self.x, self.kv_f[0], st, bias=self.kv_f[1], out=self.kv, row_stats=self.stats_m,
                                               col_sums=self.kv_f[2], stats_eps=eps)[0])
                ops.gemm_chain(descs, self.chain_flags[i])
        for w in (() if self.chain else self.layers):
            if fold:
                ops.gemm(self.x, w["qkv_f"][0], st, bias=w["qkv_f"][1], out=self.qkv, row_stats=self.stats_m, col_sums=w["qkv_f"][2], stats_eps=eps)
            else:
                ops.layernorm_rows(self.x, *w["ln1"], eps, out=self.y)
                ops.gemm(self.y, w["wqkv"], st, bias=w["bqkv"], out=self.qkv)
            attention()
            ops.gemm(self.attn, w["wo"], st, bias=w["bo"], residual=self.x, out=self.x, stats_out=self.stats_a if fold else None)
            if fold:
                ops.gemm(self.x, w["fc1_f"][0], st, bias=w["fc1_f"][1], epi=_C.EPI_GELU, out=self.h, row_stats=self.stats_a, col_sums=w["fc1_f"][2],
                         stats_eps=eps)
            else:
                ops.layernorm_rows(self.x, *w["ln2"], eps, out=self.y)
                ops.gemm(self.y, w["w1"], st, bias=w["b1"], epi=_C.EPI_GELU, out=self.h)
            ops.gemm(self.h, w["w2"], st, bias=w["b2"], residual=self.x, out=self.x, stats_out=self.stats_m if fold else None)
        # post-LayerNorm + MAP head: probe attends over the tokens, then LayerNorm + MLP with a residual
        if self.chain:
            pass                                         # the last chain wrote self.kv
        elif fold:
            ops.gemm(self.x, self.kv_f[0], st, bias=self.kv_f[1], out=self.kv, row_stats=self.stats_m, col_sums=self.kv_f[2], stats_eps=eps)
        else:
            ops.layernorm_rows(self.x, *self.post, eps, out=self.y)
            ops.gemm(self.y, self.wkv, st, bias=self.bkv, out=self.kv)
        ops.attention(self.probe_q, self.kv, self.kv[:, D:], self.pool_a, self.pool_seqs, n_heads=H, group=1, head_dim=hd,
                      causal=False, max_q_len=1, q_strides=(0, hd), k_strides=(2 * D, hd, 0), v_strides=(2 * D, hd, 0),
                      o_strides=(D, hd))
        ops.gemm(self.pool_a, self.who, st, bias=self.bho, out=self.pool_r)
        ops.layernorm_rows(self.pool_r, *self.hln, eps, out=self.pool_y)
        ops.gemm(self.pool_y, self.hw1, st, bias=self.hb1, epi=_C.EPI_GELU, out=self.pool_h)
        ops.gemm(self.pool_h, self.hw2, st, bias=self.hb2, residual=self.pool_r, out=self.embeds)

    @torch.no_grad()
    def forward(self, inp):
        """``inp["pixel_values"]``: ``[B, 3, H, W]`` on any device; copied into the engine's buffer, then one graph replay.
        A NaFlex tower takes ``pixel_values`` ``[B, S, 3 p p]`` (patch rows), ``pixel_attention_mask`` ``[B, S]`` (valid rows
        first) and ``spatial_shapes`` ``[B, 2]``, like the reference's engine (``:638-649``)."""
        px = inp["pixel_values"]
        if self.conv:
            if "spatial_shapes" in inp:
                raise ValueError("this tower has a fixed-resolution patch embedding; it takes [B, 3, H, W] pixels only")
            assert tuple(px.shape) == tuple(self.pixels.shape), f"expected {tuple(self.pixels.shape)}, got {tuple(px.shape)}"
            self.pixels.copy_(px, non_blocking=True)
        else:
            S = self.S0
            assert tuple(px.shape) == (self.B, S, self.patches.shape[1]), f"expected {(self.B, S, self.patches.shape[1])}, got {tuple(px.shape)}"
            mask, shapes = inp["pixel_attention_mask"], inp["spatial_shapes"]
            key_len = mask.to(torch.int64).sum(1).cpu()
            area = torch.as_tensor(shapes).to(torch.int64).cpu().prod(1)
            if not torch.equal(key_len, area) or int(key_len.min()) < 1:
                raise ValueError("pixel_attention_mask must mark exactly height * width leading rows of every image")
            self.patches.copy_(px.reshape(self.M, -1), non_blocking=True)
            self.pos.copy_(resize_positions(self.pos_grid, torch.as_tensor(shapes).tolist(), S).reshape(self.M, -1))
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
        return self.embeds

    def launches_per_forward(self) -> int:
        """Kernels in one forward (all inside one CUDA graph)."""
        n_l = len(self.layers)
        encoder = (n_l + 1) + n_l if self.chain else 1 + n_l * (5 if self.fold_ln else 7) + (1 if self.fold_ln else 2)
        return (1 if self.conv else 0) + encoder + 5       # + pooling head: attention, projection, LayerNorm, two MLP GEMMs

    def check(self) -> None:
        """Synchronise and raise if any GEMM pipeline wait ran out since construction."""
        ops.check_status(self.status)

    def flops(self, formula: str = "reference") -> float:
        """FLOPs of one forward.  ``reference``: the reference benchmark's formula (``benchmarks/siglip.py:35``), which
        leaves out the patch embedding and the MAP head; ``full`` counts them."""
        B, L, S, D, F = self.B, self.L, self.S0, self.D, self.F
        ref = B * L * (2 * S * D * (4 * D + 2 * F) + 4 * S * S * D)
        if formula == "reference":
            return float(ref)
        head = 2 * S * D * 2 * D + 4 * S * D + 2 * D * D + 4 * D * F
        return float(ref + B * (2 * S * D * 3 * self.p * self.p + head))


class Siglip2Embedder:
    """``Siglip2Embedder(model, batch_size=64)``: ``model`` is a Hugging Face SigLIP vision module (or a model that has
    ``.vision_model``), or a hub id when a checkpoint cache is available.  Attributes as in the reference: ``.processor``
    (``None`` without a checkpoint), ``.vm``, ``.engine``; ``.embed(pixel_values)`` batches and pads like the reference's
    ``embed`` (``:715-723``: the last batch repeats its final image)."""

    CANDIDATES = ({"fold_ln": True, "chain": True}, {"fold_ln": True, "chain": False}, {"fold_ln": False})

    def __init__(self, model_id="google/siglip2-base-patch16-naflex", batch_size=64, device="cuda", tune=None, engine=None):
        self.processor = None
        name = model_id if isinstance(model_id, str) else type(model_id).__name__
        tune = isinstance(model_id, str) if tune is None else tune
        if isinstance(model_id, str):
            from transformers import AutoImageProcessor, AutoModel
            self.processor = AutoImageProcessor.from_pretrained(model_id)
            model_id = AutoModel.from_pretrained(model_id, dtype=torch.bfloat16)
        self.vm = _vision_model(model_id).to(device, torch.bfloat16).eval()
        self.B, self.device = batch_size, device
        # `engine`: an Engine already built for this module and batch size (skips a second graph capture)
        self.engine = engine if engine is not None else Engine(self.vm, batch_size, **(self._tune(name) if tune else {}))

    def _probe_inputs(self) -> dict:
        """Seeded random inputs of the tower's own input kind, as the reference's ``_tune`` draws them (``:695-700``)."""
        cfg, B = self.vm.config, self.B
        g = torch.Generator().manual_seed(13)
        if isinstance(self.vm.embeddings.patch_embedding, torch.nn.Conv2d):
            return {"pixel_values": torch.randn(B, 3, cfg.image_size, cfg.image_size, generator=g)}
        S = cfg.num_patches
        side = int(S ** 0.5)
        return {"pixel_values": torch.randn(B, S, 3 * cfg.patch_size ** 2, generator=g), "pixel_attention_mask": torch.ones(B, S, dtype=torch.long),
                "spatial_shapes": torch.tensor([[side, side]] * B)}

    def _tune(self, name: str, path=None) -> dict:
        """Fastest engine configuration whose pooled embeddings agree with the eager tower (minimum cosine above 0.999),
        remembered per GPU, model and batch size: the reference's ``_tune`` (``:690-713``) over this build's switches."""
        from .. import tuning
        inp = self._probe_inputs()
        with torch.no_grad():
            kw = {k: v.to(self.device) for k, v in inp.items()}
            kw["pixel_values"] = kw["pixel_values"].to(torch.bfloat16)
            ref = self.vm(**kw).pooler_output.float()

        def time_ms(engine, iters=10):
            for _ in range(3):
                engine.forward(inp)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                engine.forward(inp)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / iters

        key = f"{torch.cuda.get_device_name()}|{name}|{self.B}"
        return tuning.choose(key, self.CANDIDATES, lambda c: Engine(self.vm, self.B, **c),
                             lambda e: torch.nn.functional.cosine_similarity(e.forward(inp).float(), ref, dim=-1).min().item(), time_ms, path=path)

    @torch.no_grad()
    def embed_batches(self, batches, to_host=False):
        """Embeddings of an iterable of input dicts (or fp32 pixel tensors) of exactly ``batch_size`` images each, one device
        tensor ``[B, D]`` per batch.  Pixel values that live in host memory are staged through two device buffers on a copy
        stream of their own: batch k + 1 crosses PCIe while batch k is in the encoder (pinned host tensors make the copy
        asynchronous for the host as well).  Inputs already on the device go straight to the engine.  ``to_host=True``
        returns pinned host tensors instead, each copied back right behind its batch (synchronise before reading them)."""
        dev = torch.device(self.device)
        main = torch.cuda.current_stream(dev)
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(dev)
            self._staged = [None, None]                    # per slot: device copy of the pixel values
            self._free = [torch.cuda.Event(), torch.cuda.Event()]      # slot read by the engine: may be overwritten
            for e in self._free:
                e.record(main)

        def stage(inp, slot):
            inp = {"pixel_values": inp} if torch.is_tensor(inp) else dict(inp)
            px = inp["pixel_values"]
            if px.device.type == "cuda":
                return inp, None
            buf = self._staged[slot]
            if buf is None or buf.shape != px.shape or buf.dtype != px.dtype:
                buf = self._staged[slot] = torch.empty(px.shape, dtype=px.dtype, device=dev)
            ready = torch.cuda.Event()
            with torch.cuda.stream(self._copy_stream):
                self._copy_stream.wait_event(self._free[slot])
                buf.copy_(px, non_blocking=True)
                ready.record(self._copy_stream)
            inp["pixel_values"] = buf                      # the small NaFlex tensors (mask, shapes) stay where they are
            return inp, ready

        out, it, k = [], iter(batches), 0
        nxt = next(it, None)
        staged = stage(nxt, 0) if nxt is not None else None
        while staged is not None:
            cur, ready = staged
            nxt = next(it, None)
            staged = stage(nxt, (k + 1) & 1) if nxt is not None else None      # issued before this batch's forward
            if ready is not None:
                main.wait_event(ready)
            emb = self.engine.forward(cur)
            if to_host:
                host = torch.empty(emb.shape, dtype=emb.dtype).pin_memory()
                host.copy_(emb, non_blocking=True)
                out.append(host)
            else:
                out.append(emb.clone())
            if ready is not None:
                self._free[k & 1].record(main)
            k += 1
        return out

    @torch.no_grad()
    def embed(self, images):
        """``images``: fp32 ``[N, 3, H, W]`` pixel values, a dict of processor outputs (NaFlex: ``pixel_values``,
        ``pixel_attention_mask``, ``spatial_shapes``), or PIL images when a processor is loaded.  Host inputs are fed
        through ``embed_batches``: the copy of a batch overlaps the encoder pass of the one before."""
        if torch.is_tensor(images):
            inp = {"pixel_values": images}
        elif isinstance(images, dict):
            inp = dict(images)
        else:
            inp = dict(self.processor(images=images, return_tensors="pt"))
        total = len(inp["pixel_values"])
        counts = [min(self.B, total - k) for k in range(0, total, self.B)]

        def batches():
            for k, n in zip(range(0, total, self.B), counts):
                # a short last batch is filled up with copies of its final image (reference ``:720-723``)
                fill = lambda t: t[k:k + n] if n == self.B else torch.cat([t[k:k + n], t[k + n - 1:k + n].expand(self.B - n, *t.shape[1:])])
                yield {name: fill(t) for name, t in inp.items()}

        return torch.cat([e[:n] for e, n in zip(self.embed_batches(batches()), counts)])
