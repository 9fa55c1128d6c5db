"""Parity of the CUDA decode path (through the C ABI) against the CPU oracle and the golden fixtures.

Tolerances (BASELINE north star): bf16 logits max-abs <= 3e-2 and cosine >= 0.9995 against the eager
model, teacher-forced; cache placement bit-exact.  Free-running greedy ids are compared too, and a
mismatch is accepted only where the oracle's own top-2 logits are within bf16 rounding of each other
(two eager backends with identical weights already flip such steps).
"""
import json
import os

import pytest
import torch
import torch.nn.functional as F

from oracle import qwen3_hf as hf
from oracle import qwen3_ref as ref

gpu = pytest.mark.gpu
TIE_GAP = 0.0625      # two bf16 logits of magnitude 2..4 closer than this are within 2 ulp
RMS_SLACK = 1.05      # the rms over the 151-column sample of a 151 936-column row is itself an estimate


def _load(golden_dir, name):
    return torch.load(f"{golden_dir}/{name}", weights_only=True)


def _close(got, want, what, rel=2.0 ** -6, cos_min=0.99999):
    got, want = got.float().cpu().flatten(), want.float().cpu().flatten()
    err = (got - want).abs().max().item()
    cos = F.cosine_similarity(got, want, dim=0).item()
    lim = rel * want.abs().max().item()
    assert err <= lim and cos >= cos_min, f"{what}: max-abs {err:.4g} (limit {lim:.4g}), cos {cos:.6f}"


@pytest.fixture(scope="module")
def tiny_dec(tiny_hf):
    from ittai_b200.qwen3 import Qwen3Decoder
    model, dims = tiny_hf
    return Qwen3Decoder(model, max_batch=1, kv_capacity=64)


@gpu
def test_phases_match_oracle_trace(tiny_hf, tiny_dec, golden_dir):
    """Token 16 of the tiny prompt, phase by phase as separate kernels, against the restatement's intermediates."""
    from ittai_b200 import _C
    model, dims = tiny_hf
    g = _load(golden_dir, "qwen3_tiny.pt")
    prompt = g["prompt"]
    R = ref.Qwen3Ref(model.state_dict(), dims, 64)
    R.forward(prompt[:15])
    trace = []
    want_logits = R.forward(prompt[15:16], trace=trace)

    d = tiny_dec
    d.reset()
    d.prefill(prompt[:15])
    # the restatement's cache for the first 15 tokens, so each phase is checked on identical inputs
    d.kcache[:, 0, :, :15] = R.k[:, :, :15].to(torch.bfloat16).cuda()
    d.vcache[:, 0, :, :15] = R.v[:, :, :15].to(torch.bfloat16).cuda()
    d.next_id.fill_(int(prompt[15]))
    # every phase reads the oracle's value of its input (planted with the tag the phase waits for), so an error in one
    # phase does not leak into the check of the next
    for l in range(dims.n_layers):
        t = trace[l]
        if l > 0:
            d.write_buf("h", trace[l - 1]["h"], l)
        d.run_phase(_C.PH_QKV, l)
        _close(d.read_buf("qkv")[0], t["qkv"], f"layer {l} qkv")
        d.write_buf("qkv", t["qkv"], l)
        d.run_phase(_C.PH_ATTN, l)
        _close(d.read_buf("attn")[0], t["attn"], f"layer {l} attn", rel=2.0 ** -5, cos_min=0.9999)
        _close(d.kcache[l, 0, :, 15], R.k[l, :, 15], f"layer {l} appended key")
        assert torch.equal(d.vcache[l, 0, :, 15].float().cpu(), R.v[l, :, 15]), f"layer {l} appended value"
        d.write_buf("attn", t["attn"], l)
        d.run_phase(_C.PH_OPROJ, l)
        _close(d.read_buf("hmid")[0], t["h_mid"], f"layer {l} o_proj + residual")
        d.write_buf("hmid", t["h_mid"], l)
        d.run_phase(_C.PH_GU, l)
        _close(d.read_buf("act")[0], t["act"], f"layer {l} swiglu", rel=2.0 ** -5)
        d.write_buf("act", t["act"], l)
        d.run_phase(_C.PH_DOWN, l)
        _close(d.read_buf("h")[0], t["h"], f"layer {l} down + residual")
    d.write_buf("h", trace[-1]["h"], dims.n_layers)
    d.run_phase(_C.PH_HEAD, 0)
    _close(d.logits[0], want_logits, "logits", cos_min=0.9999)
    assert int(d.next_id[0]) == int(want_logits.argmax())


@gpu
def test_tiny_teacher_forced_against_golden(tiny_hf, tiny_dec, golden_dir):
    g = _load(golden_dir, "qwen3_tiny.pt")
    d = tiny_dec
    d.reset()
    first = d.prefill(g["prompt"])
    logits = [d.logits[0].float().cpu()]
    picks = [int(first[0])]
    for s in range(1, 8):
        d.next_id.fill_(int(g["ids"][s - 1]))
        picks.append(int(d.decode(1)[0, 0]))
        logits.append(d.logits[0].float().cpu())
    logits = torch.stack(logits)
    gl = g["logits"].float()
    assert (logits - gl).abs().max() <= 3e-2
    assert F.cosine_similarity(logits, gl, dim=-1).min() >= 0.9995
    assert picks == g["ids"].tolist()


@gpu
def test_tiny_free_running_ids(tiny_dec, golden_dir):
    g = _load(golden_dir, "qwen3_tiny.pt")
    out = tiny_dec.generate(g["prompt"], 8)
    assert out[0].tolist() == g["ids"].tolist()


@gpu
def test_cache_placement_bit_exact(tiny_hf, golden_dir):
    """Token t of the sequence lands in slot t of every layer and head, and no other slot is written."""
    from ittai_b200.qwen3 import Qwen3Decoder
    model, dims = tiny_hf
    g = _load(golden_dir, "qwen3_tiny.pt")
    d = Qwen3Decoder(model, max_batch=1, kv_capacity=48)
    sentinel = torch.tensor(-24576.0, dtype=torch.bfloat16)
    d.kcache.fill_(sentinel)
    d.vcache.fill_(sentinel)
    d.prefill(g["prompt"])
    d.decode(5)
    n = 16 + 5
    for c in (d.kcache, d.vcache):
        assert (c[:, :, :, n:] == sentinel).all(), "a slot beyond the sequence was written"
        assert (c[:, :, :, :n] != sentinel).any(-1).all(), "a slot inside the sequence was not written"
    assert d.pos.tolist() == [n]
    # values in the slots: the eager model's layer-1 keys for the prompt (rounding noise only)
    gk = g["k_layer1"].float()[:, :16]
    _close(d.kcache[1, 0, :, :16], gk, "layer-1 keys vs eager cache", rel=2.0 ** -4, cos_min=0.9995)


@gpu
def test_batch2_matches_two_batch1_runs(tiny_hf):
    from ittai_b200.qwen3 import Qwen3Decoder
    model, dims = tiny_hf
    prompts = torch.stack([hf.prompt_ids(12, 5, dims.vocab), hf.prompt_ids(12, 6, dims.vocab)])
    d2 = Qwen3Decoder(model, max_batch=2, kv_capacity=32)
    out2 = d2.generate(prompts, 6)
    l2 = d2.logits.float().cpu()
    d1 = Qwen3Decoder(model, max_batch=1, kv_capacity=32)
    for b in range(2):
        out1 = d1.generate(prompts[b], 6)
        assert out1[0].tolist() == out2[b].tolist()
        _close(l2[b], d1.logits[0], f"sequence {b} logits, batch 2 vs batch 1", cos_min=0.9999)


@gpu
def test_bad_token_reports_status(tiny_dec):
    from ittai_b200._C import IttaiError
    d = tiny_dec
    d.reset()
    d.next_id.fill_(10 ** 6)
    with pytest.raises(IttaiError, match="out of range"):
        d.decode(1)
    # the aborted launch left the device positions alone, and the host mirror follows them
    assert d.lengths == d.pos.tolist() == [0]
    d.reset()
    d.next_id.fill_(3)
    d.decode(1)            # the context is still usable


@gpu
def test_wait_runs_out_and_reports(tiny_dec):
    """A CTA that never publishes its words: the others give up after the (shortened) poll limit and report it."""
    from ittai_b200 import _C
    d = tiny_dec
    d.reset()
    d.next_id.fill_(3)
    flags = d.flags
    d.flags, d.spin_limit = flags | _C.F_TEST_DROP_CTA, 8192
    try:
        with pytest.raises(_C.IttaiError, match="flag wait ran out"):
            d.decode(1)
    finally:
        d.flags, d.spin_limit = flags, 0
    d.reset()
    d.next_id.fill_(3)
    d.decode(1)


@pytest.fixture(scope="module")
def full_hf():
    return hf.build_hf(hf.FULL, seed=0)


@gpu
def test_full_model_config1(full_hf, golden_dir):
    """BASELINE config 1 on the B200: 32-id prompt, 64 greedy steps, against the CPU eager fixture."""
    from ittai_b200.qwen3 import Qwen3Decoder
    g = _load(golden_dir, "qwen3_full_c1.pt")
    d = Qwen3Decoder(full_hf, max_batch=1, kv_capacity=128)
    # teacher-forced on the oracle's ids: every step is judged on its own
    first = d.prefill(g["prompt"])
    picks, worst_abs, worst_cos = [int(first[0])], 0.0, 1.0
    rows = [d.logits[0].float().cpu()]
    for s in range(1, 64):
        d.next_id.fill_(int(g["ids"][s - 1]))
        picks.append(int(d.decode(1)[0, 0]))
        rows.append(d.logits[0].float().cpu())
    logits = torch.stack(rows)
    strided = logits[:, ::1009]
    gs = g["strided_logits"].float()
    worst_abs = (strided - gs).abs().max().item()
    rms = (strided - gs).pow(2).mean().sqrt().item()
    worst_cos = F.cosine_similarity(strided, gs, dim=-1).min().item()
    top = torch.gather(logits, 1, g["top_indices"].long())
    top_abs = (top - g["top_values"].float()).abs().max().item()
    norm_rel = ((logits.norm(dim=-1) - g["logit_norm"]).abs() / g["logit_norm"]).max().item()
    agree = sum(int(a == b) for a, b in zip(picks, g["ids"].tolist()))
    gaps = (g["top_values"][:, 0].float() - g["top_values"][:, 1].float())
    bad = [s for s in range(64) if picks[s] != int(g["ids"][s]) and gaps[s] > TIE_GAP]
    report = dict(teacher_forced_argmax_agree=agree, strided_max_abs=worst_abs, strided_rms=rms, strided_min_cos=worst_cos,
                  top8_max_abs=top_abs, norm_rel=norm_rel)
    # free-running
    out = d.generate(g["prompt"], 64)[0].tolist()
    same = 0
    while same < 64 and out[same] == int(g["ids"][same]):
        same += 1
    report.update(free_running_prefix_equal=same, first_flip_gap=float(gaps[same]) if same < 64 else None)
    # The noise floor of the comparison, from the fixture: how far the oracle's own variants (bf16 with the eager attention
    # backend, fp32) are from the pinned run on the same weights and ids.  The kernel has to be no further from the pinned
    # run than they are.  The strict north-star figures (max-abs 3e-2, 64 of 64 ids) are printed beside them: the variants
    # themselves miss those.
    floor = g["variant_distance"]
    lim_abs = max(v["full_max_abs"] for v in floor.values())        # any sample of the columns stays below the full maximum
    lim_rms = max(v["strided_rms"] for v in floor.values())
    lim_cos = min(v["strided_min_cos"] for v in floor.values())
    lim_agree = min(v["argmax_agree"] for v in floor.values())
    report.update(floor=dict(max_abs=lim_abs, strided_rms=lim_rms, strided_min_cos=lim_cos, argmax_agree=lim_agree,
                             free_running_prefix_equal={k: v["free_running_prefix_equal"] for k, v in floor.items()}),
                  strict=dict(max_abs_le_3e_2=worst_abs <= 3e-2 and top_abs <= 3e-2, ids_64_of_64=same == 64))
    report_dir = os.environ.get("ITTAI_REPORT_DIR")
    if report_dir and os.path.isdir(report_dir):
        json.dump(report, open(os.path.join(report_dir, "parity_config1.json"), "w"), indent=1)
    print(report)
    assert worst_cos >= 0.9995 and norm_rel <= 5e-3
    assert worst_abs <= lim_abs and top_abs <= lim_abs, f"max-abs {worst_abs:.4f} / {top_abs:.4f} beyond the oracle variants' {lim_abs:.4f}"
    assert rms <= RMS_SLACK * lim_rms, f"rms {rms:.5f} beyond the oracle variants' {lim_rms:.5f}"
    assert agree >= lim_agree, f"teacher-forced argmax agrees on {agree} steps, the oracle's variants on {lim_agree}"
    assert not bad, f"argmax differs at steps {bad} where the oracle's top-2 gap exceeds {TIE_GAP}"
    assert same == 64 or gaps[same] <= TIE_GAP, f"free-running ids diverge at step {same} with top-2 gap {gaps[same]}"


@gpu
def test_long_context_against_eager_on_device(full_hf, golden_dir):
    """BASELINE config 2 shape: 4096-id prompt (seed 1), capacity 8192, then teacher-forced steps; the checker is the
    eager model run on the same GPU.  The max-abs gate is the distance between the eager model's own variants recorded
    in the config-1 fixture."""
    from ittai_b200.qwen3 import Qwen3Decoder
    lim_abs = max(v["full_max_abs"] for v in _load(golden_dir, "qwen3_full_c1.pt")["variant_distance"].values())
    ids = hf.prompt_ids(4096, seed=1)
    m = full_hf.to("cuda")
    try:
        want_ids, want_logits, cache = hf.greedy(m, ids, 8)
        k_last, _ = hf.cache_kv(cache, hf.FULL.n_layers - 1)
        k_last = k_last[0].float().cpu()
    finally:
        full_hf.to("cpu")
    d = Qwen3Decoder(full_hf, max_batch=1, kv_capacity=8192)
    first = d.prefill(ids)
    rows, picks = [d.logits[0].float().cpu()], [int(first[0])]
    for s in range(1, 8):
        d.next_id.fill_(int(want_ids[s - 1]))
        picks.append(int(d.decode(1)[0, 0]))
        rows.append(d.logits[0].float().cpu())
    logits = torch.stack(rows)
    wl = want_logits.float()
    cos = F.cosine_similarity(logits, wl, dim=-1).min().item()
    err = (logits - wl).abs().max().item()
    print(dict(cos=cos, max_abs=err, floor=lim_abs, picks=picks, want=want_ids.tolist()))
    assert cos >= 0.9995 and err <= lim_abs
    assert d.pos.tolist() == [4096 + 7]
    kc = d.kcache[hf.FULL.n_layers - 1, 0, :, :4096 + 7].float().cpu()
    assert F.cosine_similarity(kc.flatten(), k_last[:, :4096 + 7].flatten(), dim=0) >= 0.999
    assert (d.kcache[:, :, :, 4096 + 7:] == 0).all()
