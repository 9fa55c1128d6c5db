"""SigLIP vision-tower benchmark with the reference's protocol and output columns (reference ``benchmarks/siglip.py``):
3 warm-ups, median of 20 CUDA-event timings (``:16-25``), FLOPs by its formula (``:35``), minimum cosine against the eager
tower (``:33``).  The reference's inputs (a hub checkpoint and one COCO image) are not available offline, so the tower
is the ViT-B/16-224 configuration with seeded random weights and the pixels are N(0, 1) (seed 3).

  python benchmarks/siglip.py [batch=64] [--ours-only]
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


def ms(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record(); torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return sorted(ts)[iters // 2]


def main():
    B = int(sys.argv[1]) if len(sys.argv) > 1 and sys.argv[1].isdigit() else 64
    vm = hf.build_hf(seed=2, device="cuda")
    emb = Siglip2Embedder(vm, batch_size=B)
    px = hf.pixels(B, seed=3).cuda()
    inp = {"pixel_values": px}
    kw = {"pixel_values": px.to(torch.bfloat16)}
    with torch.inference_mode():
        t_eager = float("nan") if "--ours-only" in sys.argv else ms(lambda: vm(**kw))
        ref = vm(**kw).pooler_output.float()
    t_mega = ms(lambda: emb.engine.forward(inp))
    emb.engine.check()
    cos = torch.nn.functional.cosine_similarity(emb.engine.forward(inp).float(), ref, dim=-1).min().item()
    flops, full = emb.engine.flops("reference"), emb.engine.flops("full")
    peaks, kind = measured_peaks()
    for n, t in (("hf eager", t_eager), ("ittai_b200", t_mega)):
        print(f"{n:16s} {t:8.3f} ms  {flops / t / 1e9:7.1f} TFLOPS  {t_eager / t:.2f}x vs eager")
    print(json.dumps({"batch": B, "ms": t_mega, "img_per_s": B / t_mega * 1e3, "tflops_reference_formula": flops / t_mega / 1e9,
                      "tflops_full_count": full / t_mega / 1e9, "frac_of_" + kind + "_bf16_peak": flops / t_mega / 1e9 / peaks["bf16_tflops"],
                      "frac_of_nominal_2250": flops / t_mega / 1e9 / 2250.0, "min_cos_vs_eager": cos, "eager_ms": t_eager}))


if __name__ == "__main__":
    main()
