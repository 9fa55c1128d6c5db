"""Qwen3-0.6B embedding (prefill) benchmark: B sequences of S tokens packed into one forward, last-token pooled.
Counterpart of the reference's ``benchmarks/qwen3.py`` with its shapes (B=64, S=512 by default), its FLOP formula
(``:34``) and its timing protocol (3 warm-ups, median of 20 CUDA-event timings, ``:16-25``).

  python benchmarks/qwen3.py [B] [S] [--ragged] [--layers 28] [--eager [--compile [MODE]]]

There is no checkpoint or tokenizer offline: the weights are the seeded random-init state dict of ``bench.py`` and the
ids are uniform random (``--ragged`` draws lengths uniformly from [S/4, S], the varlen case the reference packs).
``--eager`` also times the Hugging Face eager module on the same GPU and reports the minimum cosine against it.
"""
import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bench import measured_peaks, synthetic_state_dict  # noqa: E402
from ittai_b200.qwen3 import D, DGU, DQ, DQKV, FF, Qwen3Embedder  # noqa: E402
from benchmarks._timing import median_ms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("B", nargs="?", type=int, default=64)
    ap.add_argument("S", nargs="?", type=int, default=512)
    ap.add_argument("--ragged", action="store_true")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--compile", nargs="?", const="max-autotune", default=None, metavar="MODE",
                    help="with --eager: also time the eager module through torch.compile (default mode max-autotune, as the reference does)")
    a = ap.parse_args()
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(max(1, a.S // 4), a.S + 1, (a.B,), generator=g).tolist() if a.ragged else [a.S] * a.B
    ids = [torch.randint(0, 151936, (n,), generator=g).tolist() for n in lens]
    T = sum(lens)
    sd = synthetic_state_dict(n_layers=a.layers)
    emb = Qwen3Embedder(sd, max_tokens=T, max_seqs=a.B)
    t = median_ms(lambda: emb.engine.forward(ids))
    out = emb.engine.forward(ids).clone()
    torch.cuda.synchronize()
    flops = a.layers * (2 * T * D * (DQKV + DQ + DGU + FF) + 2 * sum(n * n for n in lens) * DQ)
    peaks, peaks_kind = measured_peaks()
    res = {"B": a.B, "S": a.S, "ragged": a.ragged, "tokens": T, "ms": t, "tok_per_s": T / t * 1e3, "tflops_reference_formula": flops / t / 1e9,
           f"frac_of_{peaks_kind}_bf16_peak": flops / t / 1e9 / peaks["bf16_tflops"], "finite": bool(torch.isfinite(out).all())}
    if a.eager:
        from transformers import Qwen3Config, Qwen3Model
        cfg = Qwen3Config(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=a.layers, num_attention_heads=16,
                          num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960,
                          tie_word_embeddings=True, attention_bias=False)
        cfg._attn_implementation = "sdpa"
        with torch.device("meta"):
            body = Qwen3Model(cfg)
        body = body.to_empty(device="cuda").to(torch.bfloat16)
        body.load_state_dict(sd, strict=False)
        body.eval()
        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=torch.float32, device="cuda") / 128))
        body.rotary_emb.inv_freq = inv                      # .to(bf16) rounded the buffer; the load path of a checkpoint does not
        S_max = max(lens)
        pad = torch.zeros(a.B, S_max, dtype=torch.long, device="cuda")
        mask = torch.zeros(a.B, S_max, dtype=torch.long, device="cuda")
        for i, s in enumerate(ids):                         # left padding, as the reference's tokenizer is configured
            pad[i, S_max - len(s):] = torch.tensor(s, device="cuda")
            mask[i, S_max - len(s):] = 1
        with torch.inference_mode():
            te = median_ms(lambda: body(input_ids=pad, attention_mask=mask), repeats=5)
            ref = F.normalize(body(input_ids=pad, attention_mask=mask).last_hidden_state[:, -1].float(), dim=-1)
        res["eager_ms"] = te
        res["min_cos_vs_eager"] = F.cosine_similarity(out.float(), ref, dim=-1).min().item()
        print(f"hf eager (sdpa)  {te:8.2f} ms  {flops / te / 1e9:6.1f} TFLOPS")
        if a.compile:
            # the reference's second comparison column (benchmarks/qwen3.py:13,30): the same module through torch.compile
            body_c = torch.compile(body, mode=a.compile)
            with torch.inference_mode():
                tc = median_ms(lambda: body_c(input_ids=pad, attention_mask=mask), repeats=5)
                ref_c = F.normalize(body_c(input_ids=pad, attention_mask=mask).last_hidden_state[:, -1].float(), dim=-1)
            res["compile_ms"], res["compile_mode"] = tc, a.compile
            res["min_cos_vs_compile"] = F.cosine_similarity(out.float(), ref_c, dim=-1).min().item()
            print(f"hf {a.compile:13s} {tc:8.2f} ms  {flops / tc / 1e9:6.1f} TFLOPS  ittai_b200 is {tc / t:.2f}x vs compile")
    print(f"ittai_b200       {t:8.2f} ms  {flops / t / 1e9:6.1f} TFLOPS  {T / t:.0f}k tok/s")
    print(json.dumps(res))


if __name__ == "__main__":
    main()
