"""Headline benchmark: Qwen3-0.6B batch-1 bf16 greedy decode, tokens per second, against the HBM roofline.

Workload (BASELINE config 2): random-init Qwen3-0.6B, 4096-token prompt (uniform ids, seed 1) prefilled into
a bf16 KV cache of capacity 8192, then 256 greedy decode steps.  One bench "step" is one such 256-token decode
run starting at cache length 4096 (the cache length is rewound between steps; the prompt is prefilled once, before
the timed region).  Every token streams about 1.66 GB of weights and cache, far more than the 126 MB L2, so no L2
flush is needed between steps.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 runs N independent replicas (one process per GPU, launched by torchrun; no data-path collective) and sums
their tokens.  ``--impl reference`` times the reference's eager PyTorch path (the Hugging Face modules it loads
and validates against) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT, CAP, DECODE = 4096, 8192, 256
METRIC, UNIT = "qwen3_0.6b_bs1_decode_tok_per_s", "tok/s"


def synthetic_state_dict(n_layers=28, vocab=151936, seed=0, device="cuda"):
    """Random-init Qwen3-0.6B weights under the Hugging Face key names: normal(0, 0.02) matrices, unit norm gains."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: (torch.randn(*s, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    one = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
    sd = {"embed_tokens.weight": rn(vocab, 1024), "norm.weight": one(1024)}
    for l in range(n_layers):
        p = f"layers.{l}."
        sd[p + "self_attn.q_proj.weight"] = rn(2048, 1024)
        sd[p + "self_attn.k_proj.weight"] = rn(1024, 1024)
        sd[p + "self_attn.v_proj.weight"] = rn(1024, 1024)
        sd[p + "self_attn.o_proj.weight"] = rn(1024, 2048)
        sd[p + "mlp.gate_proj.weight"] = rn(3072, 1024)
        sd[p + "mlp.up_proj.weight"] = rn(3072, 1024)
        sd[p + "mlp.down_proj.weight"] = rn(1024, 3072)
        sd[p + "input_layernorm.weight"] = one(1024)
        sd[p + "post_attention_layernorm.weight"] = one(1024)
        sd[p + "self_attn.q_norm.weight"] = one(128)
        sd[p + "self_attn.k_norm.weight"] = one(128)
    return sd


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.summary = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                            "samples": len(sm)}


SIGLIP_BATCH = 64


def ncu_traffic_per_token():
    """DRAM bytes (read + write) of the decode kernel per decoded token from the last ncu capture, or None.  The figures
    sit in a small JSON beside the capture's summary, with the commit they were measured at: traffic grows with the
    tokens of a launch, so the bench scales the per-token figure by its own 256."""
    path = os.path.join(ROOT, "profiles", "qwen3_decode_kernel_b1_ctx4096.traffic.json")
    try:
        t = json.load(open(path))
        return (t["dram_bytes_read"] + t["dram_bytes_write"]) / t["tokens_per_launch"], t.get("measured_at_commit")
    except (OSError, KeyError, ValueError):
        return None, None


def siglip_leg(dev, rank, barrier, iters: int = 20):
    """SigLIP ViT-B/16-224 batch-64 forward (random-init bf16 tower, N(0,1) pixels resident on the device): images per
    second over `iters` graph replays after 3 warm-ups, timed with CUDA events between barriers."""
    from transformers import SiglipVisionConfig, SiglipVisionModel
    from ittai_b200.siglip.kernel import Engine
    cfg = SiglipVisionConfig(hidden_size=768, intermediate_size=3072, num_hidden_layers=12, num_attention_heads=12, image_size=224,
                             patch_size=16, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6)
    torch.manual_seed(2 + rank)
    vm = SiglipVisionModel(cfg).to(torch.bfloat16).eval().to(dev)
    eng = Engine(vm, SIGLIP_BATCH)
    px = torch.randn(SIGLIP_BATCH, 3, 224, 224, generator=torch.Generator().manual_seed(3 + rank)).to(dev)
    inp = {"pixel_values": px}
    for _ in range(3):
        eng.forward(inp)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        eng.forward(inp)
    e1.record()
    barrier()
    eng.check()
    # the reference benchmark's protocol (benchmarks/siglip.py: every forward timed on its own, median of 20)
    singles = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); eng.forward(inp); b.record(); torch.cuda.synchronize()
        singles.append(a.elapsed_time(b))
    # end to end through the embedder (the call a user makes): every batch's pixels come from pinned host memory and its
    # embeddings go back to pinned host memory inside the timed region; the embedder stages batch k + 1 on a copy stream
    # while batch k is in the encoder
    from ittai_b200.siglip.kernel import Siglip2Embedder
    emb = Siglip2Embedder(vm, batch_size=SIGLIP_BATCH, device=dev, engine=eng)
    host_px = px.cpu().pin_memory()
    host_out = emb.embed_batches([host_px] * 2, to_host=True)      # warm-up: staging buffers, copy stream
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    host_out = emb.embed_batches((host_px for _ in range(iters)), to_host=True)
    f1.record()
    barrier()
    eng.check()
    assert len(host_out) == iters and bool(torch.isfinite(host_out[-1].float()).all())
    return {"ms": e0.elapsed_time(e1), "iters": iters, "median_single_ms": sorted(singles)[iters // 2], "images": iters * SIGLIP_BATCH, "flops_reference_formula": iters * eng.flops("reference"),
            "launches_per_forward": eng.launches_per_forward(), "e2e_ms": f0.elapsed_time(f1), "h2d_bytes": host_px.numel() * 4, "d2h_bytes": host_out[0].numel() * 2}


def config4_leg(sd, dev, barrier):
    """BASELINE config 4 on one GPU: eight 2048-token prompts (seed 4) prefilled on the tensor cores, then batch-8 greedy
    decode with the caches at length 2048 and at 8192 - 32 (filled with N(0,1) rows up to there: a decode step's cost
    depends on the cache length, not its contents).  Prefill FLOPs by the reference's formula (benchmarks/qwen3.py:35),
    decode bytes as weights + 8 caches."""
    from ittai_b200.qwen3 import Qwen3Decoder, decode_bytes_per_token
    from ittai_b200.qwen3.config import D, DGU, DQ, DQKV, FF, L
    B, T, STEPS = 8, 2048, 32
    dec = Qwen3Decoder(sd, max_batch=B, kv_capacity=CAP, device=dev)
    g = torch.Generator().manual_seed(4)
    prompts = torch.randint(0, dec.V, (B, T), generator=g, dtype=torch.int32)
    out = {}
    times = []
    for it in range(4):
        dec.reset()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        dec.prefill_cache(prompts)
        b.record()
        barrier()
        times.append(a.elapsed_time(b))
    ms = sorted(times[1:])[1]
    flops = L * (2 * B * T * D * (DQKV + DQ + DGU + FF) + 2 * B * T * T * DQ)
    out["prefill"] = {"tokens": B * T, "ms": ms, "tok_per_s": B * T / (ms / 1e3), "tflops_reference_formula": flops / (ms / 1e3) / 1e12}
    first = torch.randint(0, dec.V, (B,), generator=g, dtype=torch.int32).to(dev)
    weights = decode_bytes_per_token(0)
    kv_row = decode_bytes_per_token(1) - weights
    for ctx in (T, CAP - STEPS):
        if ctx > T:
            dec.kcache[:, :, :, T:ctx].normal_()
            dec.vcache[:, :, :, T:ctx].normal_()
        times = []
        for it in range(4):
            dec.rewind(ctx)
            dec.next_id.copy_(first)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dec.decode(STEPS, check=False)
            b.record()
            barrier()
            times.append(a.elapsed_time(b))
        dec.check_status()
        ms = sorted(times[1:])[1]
        bytes_step = weights + B * kv_row * (ctx + (STEPS - 1) / 2)
        out[f"decode_ctx{ctx}"] = {"batch": B, "steps": STEPS, "us_per_step": ms * 1e3 / STEPS, "tok_per_s": B * STEPS / (ms / 1e3),
                                   "bytes_per_step": bytes_step, "GBs": bytes_step * STEPS / (ms / 1e3) / 1e9}
    del dec
    torch.cuda.empty_cache()
    return out


def cpu_reference(steps: int, warmup: int):
    """The reference's eager PyTorch path on host cores: batch-1 decode at cache length 4096 (see oracle/qwen3_hf.py)."""
    from oracle import qwen3_hf as hf
    r = hf.time_decode_cpu(hf.FULL, kv_len=PROMPT, n_steps=max(steps, 1))
    sample = (f"{r['steps']} eager decode steps at cache length {PROMPT} (cache filled with N(0,1) values instead of a "
              f"CPU prefill), after 2 warm-up steps, {r['threads']} threads")
    return r, sample


REF_TOKENS_PER_STEP = 16      # the reference arm's step: a bounded sample of the 256-token step (about 0.7 s of host work)


def run_reference(args, rank):
    """The reference's eager path on the host cores.  One step here is REF_TOKENS_PER_STEP decoded tokens at cache length
    4096 (a bounded sample of the GPU arm's 256-token step); `value` is tokens per second, `ms_per_step` the measured time
    of one sampled step, so steps x ms_per_step is the time the run really took."""
    if rank != 0:
        return
    n = max(args.steps, 1) * REF_TOKENS_PER_STEP
    r, sample = cpu_reference(n, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": r["tok_s"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_tok"] * REF_TOKENS_PER_STEP, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"qwen3-0.6b random-init bf16, batch 1, cache length {PROMPT}, greedy decode on host cores; one step = "
                                   f"{REF_TOKENS_PER_STEP} tokens (bounded sample of the {DECODE}-token step)"},
            "cpu_baseline": {"value": r["tok_s"], "unit": UNIT, "cores": r["threads"], "kind": "reference", "sample": sample},
            "e2e": {"value": r["tok_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the host-core baseline leg")
    ap.add_argument("--no-siglip", action="store_true", help="skip the SigLIP images/s leg")
    ap.add_argument("--no-config4", action="store_true", help="skip the 2048-token prefill + batch-8 decode leg (1 GPU only)")
    ap.add_argument("--siglip-iters", type=int, default=20, help="timed SigLIP forwards per measurement (fewer for a profiler's launch list)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torchrun), got WORLD_SIZE={world}")

    import torch.distributed as dist
    from ittai_b200 import replicas
    from ittai_b200.qwen3 import Qwen3Decoder, decode_bytes_per_token

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)

    sd = synthetic_state_dict(seed=rank, device=dev)
    dec = Qwen3Decoder(sd, max_batch=1, kv_capacity=CAP, device=dev)
    del sd
    g = torch.Generator().manual_seed(1 + rank)
    prompt = torch.randint(0, dec.V, (1, PROMPT), generator=g, dtype=torch.int32)
    first = dec.prefill(prompt).clone()          # outside the timed region: cache resident in HBM

    def rewind():
        dec.rewind(PROMPT)
        dec.next_id.copy_(first)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    launches = 0
    ids_seen = []
    for _ in range(warmup):
        rewind()
        ids_seen.append(dec.decode(DECODE).clone())
    # ---- device-resident timing ------------------------------------------------------------------------
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    with ClockSampler(local) as clk:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for k in range(args.steps):
            rewind()
            ev[k][0].record()
            ids_seen.append(dec.decode(DECODE, check=False))
            ev[k][1].record()
            launches += 1
        t1.record()
        barrier()
    dec.check_status()
    # every timed step decodes the same 256 tokens from the same state: the ids have to repeat exactly
    if not all(torch.equal(ids_seen[0], x) for x in ids_seen[1:]):
        raise SystemExit("decode steps that start from the same state returned different ids")
    total_ms = t0.elapsed_time(t1)
    kern_ms = [a.elapsed_time(b) for a, b in ev]
    # per-token times of one more run (device globaltimer stamps)
    rewind()
    _, ns = dec.decode(DECODE, timed=True)
    per_tok_us = (ns[1:] - ns[:-1]).float().cpu() / 1e3
    # ---- end to end from host buffers ------------------------------------------------------------------
    host_in = first.cpu().pin_memory()
    host_out = torch.empty(1, DECODE, dtype=torch.int32).pin_memory()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(args.steps):
        dec.rewind(PROMPT)
        dec.next_id.copy_(host_in, non_blocking=True)
        out = dec.decode(DECODE, check=False)
        host_out.copy_(out, non_blocking=True)
        launches += 1
    e1.record()
    barrier()
    dec.check_status()
    e2e_ms = e0.elapsed_time(e1)

    # the two headline legs first, the config-4 leg (which frees the batch-1 decoder) last
    sig = siglip_leg(dev, rank, barrier, iters=max(args.siglip_iters, 1)) if not args.no_siglip else None
    c4 = None
    if world == 1 and not args.no_config4:
        del dec
        torch.cuda.empty_cache()
        c4 = config4_leg(synthetic_state_dict(seed=rank, device=dev), dev, barrier)
    (total_ms, e2e_ms, sig_ms, sig_e2e_ms), toks = replicas.aggregate(
        [total_ms, e2e_ms, sig["ms"] if sig else 0.0, sig["e2e_ms"] if sig else 0.0], units=args.steps * DECODE, device=dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    value = toks / (total_ms / 1e3)
    peaks, peak_kind = measured_peaks()
    mean_bytes = sum(decode_bytes_per_token(PROMPT + i) for i in range(DECODE)) / DECODE
    kern_ms_avg = sum(kern_ms) / len(kern_ms)
    achieved = mean_bytes * DECODE / (kern_ms_avg / 1e3) / 1e9
    ncu_tok, ncu_commit = ncu_traffic_per_token()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"qwen3-0.6b random-init bf16, batch 1, {PROMPT}-token prompt, kv capacity {CAP}, "
                               f"{DECODE} greedy decode steps per step", "l2": "inputs larger than L2 (1.66 GB streamed per token)",
                   "replicas": world, "parallelism": f"{world} independent replicas, no data-path collective"},
        "us_per_token": {"median": float(per_tok_us.median()), "p99": float(per_tok_us.quantile(0.99)),
                         "mean_kernel": kern_ms_avg * 1e3 / DECODE},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": ncu_tok * DECODE / 1e9 if ncu_tok else None,
                     "traffic_unit": f"GB per launch (ncu dram read+write of an 8-token launch at commit {ncu_commit}, scaled by tokens)",
                     "peak_kind": peak_kind,
                     "frac_of_nominal_8TBs": achieved / 8000.0, "bytes_per_token": mean_bytes},
        "e2e": {"value": toks / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4 * DECODE},
        "gpu_launches": launches,
        "clocks": clk.summary,
    }
    if sig:
        flops = sig["flops_reference_formula"]
        tf = world * flops / (sig_ms / 1e3) / 1e12
        line["siglip"] = {"metric": "siglip_vit_b16_224_images_per_s", "value": world * sig["images"] / (sig_ms / 1e3), "unit": "img/s",
                          "batch": SIGLIP_BATCH, "ms_per_batch": sig_ms / sig["iters"], "dtype": "bf16",
                          "roofline": {"bound": "tensor", "achieved": tf / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                       "frac": tf / world / peaks["bf16_tflops"], "peak_kind": peak_kind,
                                       "frac_of_sustained_peak": (tf / world / peaks["bf16_tflops_sustained"]) if "bf16_tflops_sustained" in peaks else None,
                                       "timing": "20 forwards back to back (sustained, power-capped clocks)",
                                       "single_forward": {"ms": sig["median_single_ms"], "frac": sig["flops_reference_formula"] / sig["iters"] / (sig["median_single_ms"] / 1e3) / 1e12 / peaks["bf16_tflops"],
                                                          "timing": "median of 20 forwards timed one by one, the reference benchmark's protocol"},
                                       "flops": "reference benchmark formula: B*L*(2*S*D*(4D+2F) + 4*S*S*D)"},
                          "gpu_launches_per_forward": sig["launches_per_forward"],
                          "e2e": {"value": world * sig["images"] / (sig_e2e_ms / 1e3), "unit": "img/s", "h2d_bytes_per_step": sig["h2d_bytes"],
                                  "d2h_bytes_per_step": sig["d2h_bytes"], "step": "one batch of 64 images: pixels from pinned host memory, embeddings back"}}
    if c4:
        tf = c4["prefill"]["tflops_reference_formula"]
        c4["prefill"]["roofline"] = {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"], "peak_kind": peak_kind}
        for k, v in c4.items():
            if k.startswith("decode"):
                v["roofline"] = {"bound": "hbm", "achieved": v["GBs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": v["GBs"] / peaks["hbm_gbs"],
                                 "frac_of_nominal_8TBs": v["GBs"] / 8000.0, "peak_kind": peak_kind}
        line["config4"] = dict(c4, workload="qwen3-0.6b random-init bf16: eight 2048-token prompts prefilled, then batch-8 greedy decode at cache length 2048 and 8160")
    if not args.no_cpu_baseline and world == 1:
        r, sample = cpu_reference(16, 2)
        line["cpu_baseline"] = {"value": r["tok_s"], "unit": UNIT, "cores": r["threads"], "kind": "reference", "sample": sample}
        if sig:
            from oracle import siglip_hf
            c = siglip_hf.time_cpu(SIGLIP_BATCH, iters=2)
            line["siglip"]["cpu_baseline"] = {"value": c["img_s"], "unit": "img/s", "cores": c["threads"], "kind": "reference",
                                              "sample": f"2 eager bf16 forwards of one batch of {SIGLIP_BATCH} images on host cores after 1 warm-up"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
