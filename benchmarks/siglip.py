"""SigLIP vision-tower benchmark with the reference's protocol and output columns (reference ``benchmarks/siglip.py``):
3 warm-ups, median of 20 CUDA-event timings (``:16-25``), FLOPs by its formula (``:35``), minimum cosine against the eager
tower (``:33``).  The reference's inputs (a hub checkpoint and one COCO image) are not available offline, so the tower
is the ViT-B/16-224 configuration with seeded random weights and the pixels are N(0, 1) (seed 3).

  python benchmarks/siglip.py [batch=64] [--ours-only] [--compile] [--per-op] [--so400m] [--naflex]

``--naflex`` takes the variable-resolution base tower (the reference wrapper's default model family: patch rows, 256 patches
per image, here all of them valid).  ``--so400m`` takes the reference benchmark's default geometry instead (so400m-patch14-384: 27 layers, width 1152, 16 heads
of 72, MLP 4304, 729 tokens per image), which runs on zero-padded weights.

``--per-op`` prints the timings of one encoder layer's kernels instead (each repeated inside one CUDA graph).
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bench import measured_peaks  # noqa: E402
from ittai_b200.siglip.kernel import Siglip2Embedder  # noqa: E402
from oracle import siglip_hf as hf  # noqa: E402  (the eager tower is the comparison column, as in the reference script)
from benchmarks._timing import graph_us, median_ms as ms  # noqa: E402


def per_op(B: int) -> None:
    """Timings of one encoder layer's kernels at batch B, each repeated inside one CUDA graph."""
    from ittai_b200 import ops
    S, D, H = 196, 768, 12
    M = B * S
    st = ops.new_status("cuda")
    x = torch.randn(M, D, device="cuda").bfloat16()
    y = torch.empty_like(x)
    gw, gb = torch.randn(D, device="cuda"), torch.randn(D, device="cuda")
    print("layernorm  %.1f us" % graph_us(lambda: ops.layernorm_rows(x, gw, gb, 1e-6, out=y)))
    qkv = torch.randn(M, 3 * D, device="cuda").bfloat16()
    o = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    seqs = torch.tensor([[b * S, S, b * S, S] for b in range(B)], dtype=torch.int32, device="cuda")
    print("attention  %.1f us" % graph_us(lambda: ops.attention(
        qkv, qkv[:, D:], qkv[:, 2 * D:], o, seqs, n_heads=H, group=1, head_dim=64, causal=False, max_q_len=S, q_strides=(3 * D, 64),
        k_strides=(3 * D, 64, 0), v_strides=(3 * D, 64, 0), o_strides=(D, 64), max_kv_len=S, q_rows_total=M, kv_rows_total=M, status=st)))
    for n, k, epi, res in ((2304, 768, 0, False), (768, 768, 0, True), (3072, 768, 1, False), (768, 3072, 0, True)):
        a = torch.randn(M, k, device="cuda").bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        bias = torch.randn(n, device="cuda")
        r = torch.randn(M, n, device="cuda").bfloat16() if res else None
        out = torch.empty(M, n, device="cuda", dtype=torch.bfloat16)
        t = graph_us(lambda: ops.gemm(a, w, st, bias=bias, residual=r, epi=epi, out=out), 20)
        print("gemm N=%d K=%d epi=%d res=%d  %.1f us  %.0f TF" % (n, k, epi, res, t, 2.0 * M * n * k / t / 1e6))
    # the four GEMMs between two attention kernels as the encoder runs them (in-place residuals, folded LayerNorms, output
    # statistics): one by one, and as one chained launch
    F = 4 * D
    attn, xx = (torch.randn(M, D, device="cuda").bfloat16() for _ in range(2))
    h = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    ws = [(torch.randn(n, k, device="cuda") * 0.03).bfloat16() for n, k in ((D, D), (F, D), (D, F), (3 * D, D))]
    bs = [torch.randn(n, device="cuda") * 0.1 for n in (D, F, D, 3 * D)]
    cs1, csq = ws[1].float().sum(1), ws[3].float().sum(1)
    sa, sm = (torch.zeros(M, D // 128, 2, device="cuda") for _ in range(2))
    flags = torch.zeros(4 * 2 * ((M + 255) // 256), dtype=torch.int32, device="cuda")
    layer = [dict(a=attn, w=ws[0], bias=bs[0], residual=xx, out=xx, stats_out=sa),
             dict(a=xx, w=ws[1], bias=bs[1], epi=1, out=h, row_stats=sa, col_sums=cs1, stats_eps=1e-6),
             dict(a=h, w=ws[2], bias=bs[2], residual=xx, out=xx, stats_out=sm),
             dict(a=xx, w=ws[3], bias=bs[3], out=qkv, row_stats=sm, col_sums=csq, stats_eps=1e-6)]
    descs = [ops.gemm_desc(d["a"], d["w"], st, **{k: v for k, v in d.items() if k not in ("a", "w")})[0] for d in layer]

    def one_by_one():
        for d in layer:
            ops.gemm(d["a"], d["w"], st, **{k: v for k, v in d.items() if k not in ("a", "w")})

    def chained():
        flags.zero_()
        ops.gemm_chain(descs, flags)

    flop = 2.0 * M * (D * D + F * D + D * F + 3 * D * D)
    for name, fn in (("four GEMMs one by one", one_by_one), ("four GEMMs chained   ", chained)):
        t = graph_us(fn, 10)
        print("%s  %.1f us  %.0f TF" % (name, t, flop / t / 1e6))
    ops.check_status(st)


def main():
    B = int(sys.argv[1]) if len(sys.argv) > 1 and sys.argv[1].isdigit() else 64
    if "--per-op" in sys.argv:
        per_op(B)
        return
    so400m, naflex = "--so400m" in sys.argv, "--naflex" in sys.argv
    vm = hf.build_hf_so400m(device="cuda") if so400m else hf.build_hf_naflex(device="cuda") if naflex else hf.build_hf(seed=2, device="cuda")
    emb = Siglip2Embedder(vm, batch_size=B)
    if naflex:
        inp = {k: v.cuda() for k, v in hf.naflex_inputs([(16, 16)] * B).items()}
        kw = dict(inp, pixel_values=inp["pixel_values"].to(torch.bfloat16))
    else:
        px = torch.randn(B, 3, 384, 384, generator=torch.Generator().manual_seed(3)).cuda() if so400m else hf.pixels(B, seed=3).cuda()
        inp = {"pixel_values": px}
        kw = {"pixel_values": px.to(torch.bfloat16)}
    with torch.inference_mode():
        t_eager = float("nan") if "--ours-only" in sys.argv else ms(lambda: vm(**kw))
        ref = vm(**kw).pooler_output.float()
    t_comp = float("nan")
    if "--compile" in sys.argv:
        # the reference's second comparison column (benchmarks/siglip.py:13,30): the eager tower through torch.compile
        vm_c = torch.compile(vm, mode="max-autotune")
        with torch.inference_mode():
            t_comp = ms(lambda: vm_c(**kw))
    t_mega = ms(lambda: emb.engine.forward(inp))
    emb.engine.check()
    cos = torch.nn.functional.cosine_similarity(emb.engine.forward(inp).float(), ref, dim=-1).min().item()
    flops, full = emb.engine.flops("reference"), emb.engine.flops("full")
    peaks, kind = measured_peaks()
    for n, t in (("hf eager", t_eager), ("hf max-autotune", t_comp), ("ittai_b200", t_mega)):
        print(f"{n:16s} {t:8.3f} ms  {flops / t / 1e9:7.1f} TFLOPS  {t_eager / t:.2f}x vs eager")
    print(json.dumps({"batch": B, "ms": t_mega, "img_per_s": B / t_mega * 1e3, "tflops_reference_formula": flops / t_mega / 1e9,
                      "tflops_full_count": full / t_mega / 1e9, "frac_of_" + kind + "_bf16_peak": flops / t_mega / 1e9 / peaks["bf16_tflops"],
                      "frac_of_nominal_2250": flops / t_mega / 1e9 / 2250.0, "min_cos_vs_eager": cos, "eager_ms": t_eager, "compile_ms": t_comp}))


if __name__ == "__main__":
    main()
