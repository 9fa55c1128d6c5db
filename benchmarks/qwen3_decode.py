"""Qwen3-0.6B batch decode benchmark: tokens/s, microseconds per token, HBM roofline fraction and the in-kernel
per-phase profile.  The decode counterpart of the reference's prefill benchmark (reference ``benchmarks/qwen3.py``),
with its timing protocol: 3 warm-ups, then the median of 20 CUDA-event timings (``:16-25``).

  python benchmarks/qwen3_decode.py [--batch 1] [--ctx 4096] [--steps 256] [--cap 8192] [--iters 20] [--phases]

The cache is filled with N(0,1) keys and values up to ``--ctx`` (a decode step's cost depends on the cache length, not
its contents), so no prompt has to be fed first; ``--prefill`` feeds a random prompt through the kernel instead.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bench import measured_peaks, synthetic_state_dict  # noqa: E402
from ittai_b200.qwen3 import PHASE_NAMES, Qwen3Decoder, decode_bytes_per_token  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--cap", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--prefill", action="store_true")
    ap.add_argument("--phases", action="store_true", help="print CTA 0's per-phase wait / work times")
    a = ap.parse_args()
    dec = Qwen3Decoder(synthetic_state_dict(n_layers=a.layers), max_batch=a.batch, kv_capacity=a.cap)
    g = torch.Generator().manual_seed(1)
    if a.prefill:
        dec.prefill(torch.randint(0, dec.V, (a.batch, a.ctx), generator=g, dtype=torch.int32))
    else:
        dec.kcache[:, :, :, :a.ctx].normal_()
        dec.vcache[:, :, :, :a.ctx].normal_()
    first = torch.randint(0, dec.V, (a.batch,), generator=g, dtype=torch.int32).cuda()

    def rewind():
        dec.rewind(a.ctx)
        dec.next_id.copy_(first)

    times = []
    for it in range(3 + a.iters):
        rewind()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        dec.decode(a.steps, check=False)
        e.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(s.elapsed_time(e))
    dec.check_status()
    ms = sorted(times)[len(times) // 2]
    us_tok = ms * 1e3 / a.steps
    peaks, kind = measured_peaks()
    weights = decode_bytes_per_token(0, n_layers=a.layers)
    kv_row = decode_bytes_per_token(1, n_layers=a.layers) - weights
    mean_ctx = a.ctx + (a.steps - 1) / 2
    bytes_step = weights + a.batch * kv_row * mean_ctx
    out = {"batch": a.batch, "ctx": a.ctx, "steps": a.steps, "us_per_step": us_tok, "tok_per_s": a.batch * a.steps / (ms / 1e3),
           "bytes_per_step": bytes_step, "GBs": bytes_step / us_tok / 1e3, "frac_of_" + kind + "_hbm": bytes_step / us_tok / 1e3 / peaks["hbm_gbs"],
           "frac_of_nominal_8TBs": bytes_step / us_tok / 1e3 / 8000.0}
    print(json.dumps(out))
    if a.phases:
        rewind()
        n = min(a.steps, 16)
        clk = dec.decode_profiled(n).cpu().double()
        flat = clk.reshape(n, -1)
        prev = torch.cat([torch.full((n, 1), float("nan"), dtype=torch.float64), flat[:, :-1]], 1)
        dt = (flat - prev).reshape(n, -1, 2)[2:] / (peaks.get("sm_max_mhz", 1965.0))      # cycles -> us at the max SM clock
        wait, work = dt[..., 0].nanmean(0), dt[..., 1].nanmean(0)
        print("phase     wait_us  work_us   (CTA 0, mean over layers 1.. and steps 2..)")
        for i, name in enumerate(PHASE_NAMES[:5]):
            print(f"{name:8s} {wait[i:-1:5][1:].mean():8.2f} {work[i:-1:5][1:].mean():8.2f}")
        print(f"{'head':8s} {wait[-1]:8.2f} {work[-1]:8.2f}")


if __name__ == "__main__":
    main()
