"""Attention and row-wise kernels of the prefill / SigLIP paths against fp32 torch references (GPU).

Tolerances: one bf16 rounding of the output (2^-8 relative) plus, for attention, the bf16 rounding of the probabilities
before the PV product: |err| <= 2^-6 |want| + 2^-6 rms(want)."""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

gpu = pytest.mark.gpu


def _check(got, want, what, rel=2.0 ** -6):
    got, want = got.float(), want.float()
    tol = rel * want.abs() + 2.0 ** -6 * want.pow(2).mean().sqrt()
    bad = (got - want).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} outside tolerance, max err {(got - want).abs().max():.4g}"


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@gpu
@pytest.mark.parametrize("B,S", [(1, 196), (3, 196), (2, 77)])
def test_attention_dense_packed_qkv(B, S):
    """SigLIP layout: one [B*S, 3*768] matrix holding q | k | v, 12 heads of 64, no mask inside a sequence."""
    from ittai_b200 import ops
    H, hd, D = 12, 64, 768
    qkv = _rand(B * S, 3 * D, seed=1)
    out = torch.zeros(B * S, D, dtype=torch.bfloat16, device="cuda")
    seqs = torch.tensor([[b * S, S, b * S, S] for b in range(B)], dtype=torch.int32, device="cuda")
    ops.attention(qkv, qkv[:, D:], qkv[:, 2 * D:], out, seqs, n_heads=H, group=1, head_dim=hd, causal=False, max_q_len=S,
                  q_strides=(3 * D, hd), k_strides=(3 * D, hd, 0), v_strides=(3 * D, hd, 0), o_strides=(D, hd), max_kv_len=S)
    q, k, v = (qkv[:, i * D:(i + 1) * D].float().view(B, S, H, hd).transpose(1, 2) for i in range(3))
    want = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B * S, D)
    _check(out, want, f"dense attention B={B} S={S}")


@gpu
@pytest.mark.parametrize("lens", [[196] * 5, [224, 65, 130, 200], [128, 129], [70], [112, 113, 100, 97], [208, 81, 127],
                                  [256, 256, 225], [240, 96, 256, 241]])
def test_attention_tensor_memory_kernel(lens):
    """The tcgen05 kernel (row totals + status words given): ragged sequences packed in one q | k | v matrix, with rows
    past the last sequence left as NaN-free garbage.  Same reference and tolerance as the register-tile kernels."""
    from ittai_b200 import ops
    H, hd, D = 12, 64, 768
    T = sum(lens)
    qkv = _rand(T + 3, 3 * D, seed=5)
    out = torch.zeros(T + 3, D, dtype=torch.bfloat16, device="cuda")
    starts = [sum(lens[:i]) for i in range(len(lens))]
    seqs = torch.tensor([[s, n, s, n] for s, n in zip(starts, lens)], dtype=torch.int32, device="cuda")
    st = ops.new_status(qkv.device)
    ops.attention(qkv, qkv[:, D:], qkv[:, 2 * D:], out, seqs, n_heads=H, group=1, head_dim=hd, causal=False, max_q_len=max(lens),
                  q_strides=(3 * D, hd), k_strides=(3 * D, hd, 0), v_strides=(3 * D, hd, 0), o_strides=(D, hd),
                  max_kv_len=max(lens), q_rows_total=T + 3, kv_rows_total=T + 3, status=st)
    ops.check_status(st)
    for s, n in zip(starts, lens):
        q, k, v = (qkv[s:s + n, i * D:(i + 1) * D].float().view(n, H, hd).transpose(0, 1) for i in range(3))
        want = F.scaled_dot_product_attention(q, k, v).transpose(0, 1).reshape(n, D)
        _check(out[s:s + n], want, f"tensor-memory attention rows {s}..{s + n}")
    assert not out[T:].any(), "rows past the last sequence were written"


@gpu
@pytest.mark.parametrize("kind", ["ramp", "step"])
@pytest.mark.parametrize("n", [196, 224, 120, 256])
def test_attention_tensor_memory_kernel_rising_scores(n, kind):
    """Scores that grow along the keys by far more than a row's softmax reference may lag behind: the one-pass softmax
    has to raise its reference and rescale the probabilities it has already written, in both halves of the keys, and the
    halves end with references hundreds of log2 units apart.  Head 0, "ramp": key j is (j / 4) x the query direction
    (+1.08 log2 units per key); "step": keys 0..39 are zero and the rest 50 x the query direction (+216 log2 units inside
    one chunk, so the stale reference makes 2^x overflow before it is raised).  Head 1: the same keys in reverse order
    (the first chunk already holds the maximum); the other heads are random."""
    from ittai_b200 import ops
    H, hd, D = 12, 64, 768
    qkv = _rand(n, 3 * D, seed=9)
    u = torch.nn.functional.normalize(torch.randn(hd, generator=torch.Generator().manual_seed(3)), dim=0).cuda()
    ramp = torch.arange(n, device="cuda", dtype=torch.float32)
    mag = ramp / 4 if kind == "ramp" else (ramp >= 40).float() * 50
    qkv[:, 0:hd] = (u * 24.0).to(torch.bfloat16)                                   # q of head 0: |q| = 24 for every row
    qkv[:, D:D + hd] = (mag[:, None] * u).to(torch.bfloat16)                       # k of head 0
    qkv[:, hd:2 * hd] = (u * 24.0).to(torch.bfloat16)
    qkv[:, D + hd:D + 2 * hd] = (mag.flip(0)[:, None] * u).to(torch.bfloat16)
    out = torch.zeros(n, D, dtype=torch.bfloat16, device="cuda")
    seqs = torch.tensor([[0, n, 0, n]], dtype=torch.int32, device="cuda")
    st = ops.new_status(qkv.device)
    ops.attention(qkv, qkv[:, D:], qkv[:, 2 * D:], out, seqs, n_heads=H, group=1, head_dim=hd, causal=False, max_q_len=n,
                  q_strides=(3 * D, hd), k_strides=(3 * D, hd, 0), v_strides=(3 * D, hd, 0), o_strides=(D, hd),
                  max_kv_len=n, q_rows_total=n, kv_rows_total=n, status=st)
    ops.check_status(st)
    q, k, v = (qkv[:, i * D:(i + 1) * D].float().view(n, H, hd).transpose(0, 1) for i in range(3))
    sc = q[0] @ k[0].T / 8
    assert float((sc.amax(1) - sc[:, :16].amax(1)).min()) * 1.4427 > 64, "the case no longer forces a raise of the reference"
    want = F.scaled_dot_product_attention(q, k, v).transpose(0, 1).reshape(n, D)
    assert torch.isfinite(out.float()).all()
    _check(out, want, f"rising scores ({kind}), {n} keys")


@gpu
@pytest.mark.parametrize("q_len,prefix", [(300, 0), (64, 0), (130, 70), (1, 500)])
def test_attention_causal_gqa_cache_layout(q_len, prefix):
    """Qwen3 layout: q in a [T, 4096] qkv matrix (16 heads of 128), k/v in a cache [B, 8, cap, 128], causal with a prefix."""
    from ittai_b200 import ops
    NH, NKV, hd, cap, B = 16, 8, 128, 640, 2
    kv_len = prefix + q_len
    qkv = _rand(B * q_len, 4096, seed=2)
    kc, vc = _rand(B, NKV, cap, hd, seed=3), _rand(B, NKV, cap, hd, seed=4)
    out = torch.zeros(B * q_len, NH * hd, dtype=torch.bfloat16, device="cuda")
    seqs = torch.tensor([[b * q_len, q_len, 0, kv_len] for b in range(B)], dtype=torch.int32, device="cuda")
    ops.attention(qkv, kc, vc, out, seqs, n_heads=NH, group=2, head_dim=hd, causal=True, max_q_len=q_len,
                  q_strides=(4096, hd), k_strides=(hd, cap * hd, NKV * cap * hd), v_strides=(hd, cap * hd, NKV * cap * hd),
                  o_strides=(NH * hd, hd))
    q = qkv[:, :NH * hd].float().view(B, q_len, NH, hd).transpose(1, 2)
    k = kc[:, :, :kv_len].float().repeat_interleave(2, 1)
    v = vc[:, :, :kv_len].float().repeat_interleave(2, 1)
    mask = torch.arange(kv_len, device="cuda")[None, :] <= torch.arange(q_len, device="cuda")[:, None] + prefix
    want = F.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(B * q_len, NH * hd)
    _check(out, want, f"causal attention q_len={q_len} prefix={prefix}")


@gpu
@pytest.mark.parametrize("q_len,prefix,causal", [(300, 0, True), (130, 70, True), (512, 0, True), (128, 1000, True), (65, 3, True), (200, 56, False)])
def test_attention_key_loop_tensor_memory_kernel(q_len, prefix, causal):
    """The tcgen05 key-loop kernel (row totals + status words given) on the Qwen3 layout: q in a [T, 4096] qkv matrix, k/v in
    a cache [B, 8, cap, 128] whose rows past each sequence hold NaN (unwritten cache must not leak into the result)."""
    from ittai_b200 import ops
    NH, NKV, hd, cap, B = 16, 8, 128, 1280, 2
    kv_len = prefix + q_len
    qkv = _rand(B * q_len, 4096, seed=6)
    kc, vc = _rand(B, NKV, cap, hd, seed=7), _rand(B, NKV, cap, hd, seed=8)
    kc[:, :, kv_len:] = float("nan")
    vc[:, :, kv_len:] = float("nan")
    out = torch.zeros(B * q_len, NH * hd, dtype=torch.bfloat16, device="cuda")
    seqs = torch.tensor([[b * q_len, q_len, 0, kv_len] for b in range(B)], dtype=torch.int32, device="cuda")
    st = ops.new_status(qkv.device)
    ops.attention(qkv, kc, vc, out, seqs, n_heads=NH, group=2, head_dim=hd, causal=causal, max_q_len=q_len,
                  q_strides=(4096, hd), k_strides=(hd, cap * hd, NKV * cap * hd), v_strides=(hd, cap * hd, NKV * cap * hd),
                  o_strides=(NH * hd, hd), q_rows_total=B * q_len, kv_rows_total=B * NKV * cap, status=st)
    ops.check_status(st)
    q = qkv[:, :NH * hd].float().view(B, q_len, NH, hd).transpose(1, 2)
    k = kc[:, :, :kv_len].float().repeat_interleave(2, 1)
    v = vc[:, :, :kv_len].float().repeat_interleave(2, 1)
    mask = torch.arange(kv_len, device="cuda")[None, :] <= torch.arange(q_len, device="cuda")[:, None] + prefix if causal else None
    want = F.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(B * q_len, NH * hd)
    _check(out, want, f"key-loop attention q={q_len} prefix={prefix} causal={causal}")


@gpu
def test_norm_rows():
    from ittai_b200 import ops
    x = _rand(777, 1024, scale=3.0, seed=5)
    g = _rand(1024, seed=6)
    xf = x.float()
    rb = lambda t: t.to(torch.bfloat16).float()
    want = rb(rb(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)) * g.float())
    got = ops.rmsnorm_rows(x, g, 1e-6)
    assert (got.float() != want).float().mean() < 1e-3 and (got.float() - want).abs().max() <= 2.0 ** -6 * want.abs().max()
    x7 = _rand(500, 768, scale=2.0, seed=7)
    gain, beta = torch.randn(768, device="cuda"), torch.randn(768, device="cuda")
    _check(ops.layernorm_rows(x7, gain, beta, 1e-6), F.layer_norm(x7.float(), (768,), gain, beta, 1e-6), "layernorm", rel=2.0 ** -7)


@gpu
def test_qk_rope_scatter_matches_oracle(tiny_hf):
    from ittai_b200 import _C
    from ittai_b200.qwen3.decoder import rope_table
    from oracle import qwen3_ref as ref
    model, dims = tiny_hf
    T, cap, B = 37, 64, 2
    qkv = _rand(T, 4096, seed=8)
    sd = model.state_dict()
    qn, kn = sd["model.layers.0.self_attn.q_norm.weight"].cuda(), sd["model.layers.0.self_attn.k_norm.weight"].cuda()
    pos = torch.arange(T, dtype=torch.int32, device="cuda") % 20 + 3
    seq = (torch.arange(T, device="cuda") >= 20).to(torch.int32)
    kc = torch.zeros(B, 8, cap, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    rope = rope_table(cap, "cuda")
    want_in = qkv.clone()
    _C.check(_C.lib().ittai_qwen3_qk_rope_scatter(qkv.data_ptr(), qn.data_ptr(), kn.data_ptr(), rope.data_ptr(), pos.data_ptr(),
                                                   seq.data_ptr(), pos.data_ptr(), kc.data_ptr(), vc.data_ptr(), T, cap, 1e-6, None))
    cos, sin = ref.rope_table(cap, dims)
    cs, sn = cos[pos.cpu().long()][:, None, :], sin[pos.cpu().long()][:, None, :]
    x = want_in.float().cpu()
    q = ref.rope(ref.rmsnorm(x[:, :2048].view(T, 16, 128), qn.float().cpu(), 1e-6), cs, sn)
    k = ref.rope(ref.rmsnorm(x[:, 2048:3072].view(T, 8, 128), kn.float().cpu(), 1e-6), cs, sn)
    v = x[:, 3072:].view(T, 8, 128)
    got_q = qkv[:, :2048].float().cpu().view(T, 16, 128)
    assert (got_q != q).float().mean() < 2e-3 and (got_q - q).abs().max() <= 2.0 ** -6 * q.abs().max()
    for t in range(T):
        b, p = int(seq[t]), int(pos[t])
        assert torch.equal(vc[b, :, p].float().cpu(), v[t])
        assert (kc[b, :, p].float().cpu() - k[t]).abs().max() <= 2.0 ** -6 * k.abs().max()
    written = torch.zeros(B, cap, dtype=torch.bool)
    written[seq.cpu().long(), pos.cpu().long()] = True
    assert (kc.float().cpu().abs().sum((1, 3)) > 0).eq(written).all(), "a cache row outside (seq, pos) was written"


@gpu
def test_qkv_gemm_with_rope_epilogue_matches_the_separate_pass():
    """QKV projection with QK-norm + RoPE + cache scatter in the GEMM epilogue against GEMM followed by the row-wise pass:
    same rounding steps, so q, the K cache and the V cache agree except where the different summation order of the
    RMS statistic flips a rounding (a handful of values, by one bf16 step)."""
    from ittai_b200 import _C, ops
    from ittai_b200.qwen3.decoder import rope_table
    T, cap, B = 700, 512, 2
    x, w = _rand(T, 1024, seed=31), _rand(4096, 1024, scale=0.05, seed=32)
    qn, kn = (_rand(128, seed=33).float() * 0.2 + 1).to(torch.bfloat16), (_rand(128, seed=34).float() * 0.2 + 1).to(torch.bfloat16)
    rope = rope_table(cap, "cuda")
    pos = (torch.arange(T, device="cuda") % 350).int()
    seq = (torch.arange(T, device="cuda") // 350).int()
    slot = pos.clone()
    st = ops.new_status("cuda")
    L = _C.lib()
    kc1, vc1 = torch.zeros(B, 8, cap, 128, dtype=torch.bfloat16, device="cuda"), torch.zeros(B, 8, cap, 128, dtype=torch.bfloat16, device="cuda")
    qkv1 = ops.gemm(x, w, st)
    _C.check(L.ittai_qwen3_qk_rope_scatter(qkv1.data_ptr(), qn.data_ptr(), kn.data_ptr(), rope.data_ptr(), pos.data_ptr(), seq.data_ptr(),
                                           slot.data_ptr(), kc1.data_ptr(), vc1.data_ptr(), T, cap, 1e-6, ops._stream(x)))
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    qkv2 = torch.zeros(T, 4096, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, w, st, out=qkv2, epi=_C.EPI_QKROPE,
             qk_rope=dict(qn=qn, kn=kn, rope=rope, pos=pos, seq=seq, slot=slot, kcache=kc2, vcache=vc2, kv_cap=cap, eps=1e-6))
    ops.check_status(st)
    assert torch.equal(vc1, vc2), "V cache differs"
    for name, a, b in (("q", qkv1[:, :2048], qkv2[:, :2048]), ("K cache", kc1, kc2)):
        diff = (a.float() - b.float()).abs()
        frac = (diff > 0).float().mean().item()
        assert frac < 1e-3 and diff.max().item() <= 2.0 ** -6 * a.float().abs().max().item(), f"{name}: {frac:.2e} of the values differ, max {diff.max().item():.4g}"
    assert not qkv2[:, 2048:].any(), "k / v columns of the output matrix were written"


@gpu
def test_im2col_embed_pool():
    from ittai_b200 import _C
    L = _C.lib()
    px = torch.randn(3, 3, 224, 224, device="cuda")
    out = torch.empty(3 * 196, 768, dtype=torch.bfloat16, device="cuda")
    _C.check(L.ittai_siglip_im2col(px.data_ptr(), out.data_ptr(), 3, 224, 224, 16, 0, None))
    want = px.unfold(2, 16, 16).unfold(3, 16, 16).permute(0, 2, 3, 1, 4, 5).reshape(3 * 196, 768).to(torch.bfloat16)
    assert torch.equal(out, want)
    # patch 14 (two pixels per thread) into rows padded from 588 to 640 columns: the padding is left alone
    px14 = torch.randn(2, 3, 60, 76, device="cuda")   # 4 and 6 pixels beyond the last whole patch
    out14 = torch.full((2 * 4 * 5, 640), 7.0, dtype=torch.bfloat16, device="cuda")
    _C.check(L.ittai_siglip_im2col(px14.data_ptr(), out14.data_ptr(), 2, 60, 76, 14, 640, None))
    want14 = px14[:, :, :56, :70].unfold(2, 14, 14).unfold(3, 14, 14).permute(0, 2, 3, 1, 4, 5).reshape(40, 588).to(torch.bfloat16)
    assert torch.equal(out14[:, :588], want14) and bool((out14[:, 588:] == 7.0).all())
    table = _rand(500, 1024, seed=9)
    ids = torch.tensor([3, 499, 0, 17], dtype=torch.int32, device="cuda")
    rows = torch.empty(4, 1024, dtype=torch.bfloat16, device="cuda")
    _C.check(L.ittai_embed_rows(ids.data_ptr(), table.data_ptr(), rows.data_ptr(), 4, 500, None))
    assert torch.equal(rows, table[ids.long()])
    gain = _rand(1024, seed=10)
    pooled = torch.empty(2, 1024, device="cuda")
    sel = torch.tensor([1, 3], dtype=torch.int32, device="cuda")
    _C.check(L.ittai_qwen3_final_pool(rows.data_ptr(), sel.data_ptr(), gain.data_ptr(), pooled.data_ptr(), 2, 1e-6, None))
    x = rows[sel.long()].float()
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * gain.float()
    assert torch.allclose(pooled, F.normalize(y, dim=-1), atol=1e-5)


@gpu
@pytest.mark.parametrize("lens", [[729, 729], [256, 100, 300], [130]])
def test_attention_key_loop_kernel_packed_keys(lens):
    """The tcgen05 key-loop kernel with keys and values packed like the queries (one [T, 3 * H * 128] matrix, dense, no
    cache): the layout of the zero-padded so400m tower."""
    from ittai_b200 import ops
    H, hd = 4, 128
    D = H * hd
    T = sum(lens)
    qkv = _rand(T + 2, 3 * D, seed=13)
    out = torch.zeros(T + 2, D, dtype=torch.bfloat16, device="cuda")
    starts = [sum(lens[:i]) for i in range(len(lens))]
    seqs = torch.tensor([[s, n, s, n] for s, n in zip(starts, lens)], dtype=torch.int32, device="cuda")
    st = ops.new_status(qkv.device)
    ops.attention(qkv, qkv[:, D:], qkv[:, 2 * D:], out, seqs, n_heads=H, group=1, head_dim=hd, causal=False, max_q_len=max(lens),
                  q_strides=(3 * D, hd), k_strides=(3 * D, hd, 0), v_strides=(3 * D, hd, 0), o_strides=(D, hd), max_kv_len=max(lens),
                  q_rows_total=T + 2, kv_rows_total=T + 2, status=st)
    ops.check_status(st)
    for s, n in zip(starts, lens):
        q, k, v = (qkv[s:s + n, i * D:(i + 1) * D].float().view(n, H, hd).transpose(0, 1) for i in range(3))
        want = F.scaled_dot_product_attention(q, k, v).transpose(0, 1).reshape(n, D)
        _check(out[s:s + n], want, f"key-loop attention, packed keys, rows {s}..{s + n}")
    assert not out[T:].any()
