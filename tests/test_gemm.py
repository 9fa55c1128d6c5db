"""tcgen05 GEMM and its fused epilogues against fp32 torch references of the same bf16 inputs (GPU).

Tolerance: the kernel accumulates in fp32 and rounds to bf16, so it agrees with the fp32 reference to one bf16 rounding
(2^-8 relative), twice where an epilogue rounds before a non-linearity and a tie falls the other way:
|got - want| <= 2^-6 * |want| + 2^-7 * rms(want)."""
import pytest
import torch

gpu = pytest.mark.gpu


def _check(got, want, what, mid=None):
    """``mid``: an intermediate the epilogue rounds to bf16 before adding something to it (the module output ahead of a
    residual add); one ulp of it is allowed on top, since it does not shrink when the sum cancels."""
    got, want = got.float(), want.float()
    tol = 2.0 ** -6 * want.abs() + 2.0 ** -7 * want.pow(2).mean().sqrt()
    if mid is not None:
        tol = tol + 2.0 ** -7 * mid.float().abs()
    bad = (got - want).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} outside tolerance, max err {(got - want).abs().max():.4g}"


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@gpu
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (1, 256, 512), (64, 768, 768), (200, 256, 768), (1000, 2304, 768), (4096, 1024, 3072), (12544, 768, 3072)])
def test_gemm_plain(m, n, k):
    from ittai_b200 import ops
    a, w = _rand(m, k, seed=1), _rand(n, k, scale=0.05, seed=2)
    st = ops.new_status("cuda")
    out = ops.gemm(a, w, st)
    ops.check_status(st)
    _check(out, a.float() @ w.float().t(), f"gemm {m}x{n}x{k}")


@gpu
def test_gemm_row_identity():
    """A = rows of the identity picks out columns of W: catches a wrong swizzle or K-step in the operand descriptors."""
    from ittai_b200 import ops
    k, n = 256, 256
    a = torch.eye(k, device="cuda", dtype=torch.bfloat16)
    w = _rand(n, k, seed=3)
    st = ops.new_status("cuda")
    out = ops.gemm(a, w, st)
    ops.check_status(st)
    assert torch.equal(out, w.t().contiguous())


@gpu
def test_gemm_bias_gelu_residual_swiglu():
    from ittai_b200 import _C, ops
    m, n, k = 392, 3072, 768
    a, w = _rand(m, k, seed=4), _rand(n, k, scale=0.05, seed=5)
    bias = _rand(n, seed=7).float() * 0.1
    res = _rand(m, n, seed=6)
    st = ops.new_status("cuda")
    acc = a.float() @ w.float().t()
    rb = lambda x: x.to(torch.bfloat16).float()
    _check(ops.gemm(a, w, st, bias=bias), acc + bias, "bias")
    _check(ops.gemm(a, w, st, bias=bias, epi=_C.EPI_GELU),
           torch.nn.functional.gelu(rb(acc + bias), approximate="tanh"), "bias + gelu")
    _check(ops.gemm(a, w, st, bias=bias, residual=res), res.float() + rb(acc + bias), "bias + residual", mid=acc + bias)
    _check(ops.gemm(a, w, st, residual=res), res.float() + rb(acc), "residual", mid=acc)
    g, u = rb(acc[:, 0::2]), rb(acc[:, 1::2])
    _check(ops.gemm(a, w, st, epi=_C.EPI_SWIGLU), rb(torch.nn.functional.silu(g)) * u, "swiglu")
    ops.check_status(st)


@gpu
@pytest.mark.parametrize("m,n,k,epi", [(1000, 2304, 768, 0), (12544, 3072, 768, 1), (196, 1536, 768, 0)])
def test_gemm_folded_layernorm(m, n, k, epi):
    """Linear(LayerNorm(x)) with the LayerNorm folded into the GEMM (row statistics in the epilogue) against the unfused
    fp32 computation; rows carry a large common offset so that a wrong mean term would show."""
    import torch.nn.functional as F
    from ittai_b200 import _C, ops
    x = (_rand(m, k, seed=11).float() * 1.5 + 3.0).to(torch.bfloat16)
    w, bias = _rand(n, k, scale=0.05, seed=12), torch.randn(n, device="cuda")
    gain, beta = torch.rand(k, device="cuda") + 0.5, torch.randn(k, device="cuda") * 0.1
    st = ops.new_status("cuda")
    stats = ops.row_stats(x, 1e-6)
    xf = x.float()
    assert torch.allclose(stats[:, 0], xf.mean(-1), atol=1e-5, rtol=1e-5)
    assert torch.allclose(stats[:, 1], torch.rsqrt(xf.var(-1, unbiased=False) + 1e-6), rtol=1e-4)
    wp, bp, cs = ops.fold_layernorm(w, bias, gain, beta)
    out = ops.gemm(x, wp, st, bias=bp, epi=_C.EPI_GELU if epi else _C.EPI_NONE, row_stats=stats, col_sums=cs)
    ops.check_status(st)
    want = F.linear(F.layer_norm(xf, (k,), gain, beta, 1e-6), w.float(), bias)
    if epi:
        want = F.gelu(want.to(torch.bfloat16).float(), approximate="tanh")
    _check(out, want, f"folded LayerNorm gemm {m}x{n}x{k} epi={epi}")


@gpu
def test_gemm_statistics_from_the_producing_epilogue():
    """A GEMM writes (sum, sum of squares) of its output rows per 128-column slice; the next GEMM finishes mean / rstd
    from them and applies the folded LayerNorm: the pair must match LayerNorm + Linear on the stored bf16 rows."""
    import torch.nn.functional as F
    from ittai_b200 import ops
    m, d, n = 1000, 768, 2304
    a0, w0, r0 = _rand(m, d, seed=21), _rand(d, d, scale=0.05, seed=22), (_rand(m, d, seed=23).float() * 2 + 1).to(torch.bfloat16)
    st = ops.new_status("cuda")
    parts = torch.full((m, d // 128, 2), float("nan"), device="cuda")
    x = ops.gemm(a0, w0, st, residual=r0, stats_out=parts)
    xf = x.float().view(m, d // 128, 128)
    assert torch.allclose(parts[..., 0], xf.sum(-1), rtol=1e-5, atol=1e-3)
    assert torch.allclose(parts[..., 1], xf.pow(2).sum(-1), rtol=1e-5, atol=1e-3)
    w, bias = _rand(n, d, scale=0.05, seed=24), torch.randn(n, device="cuda")
    gain, beta = torch.rand(d, device="cuda") + 0.5, torch.randn(d, device="cuda") * 0.1
    wp, bp, cs = ops.fold_layernorm(w, bias, gain, beta)
    out = ops.gemm(x, wp, st, bias=bp, row_stats=parts, col_sums=cs, stats_eps=1e-6)
    ops.check_status(st)
    _check(out, F.linear(F.layer_norm(x.float(), (d,), gain, beta, 1e-6), w.float(), bias), "folded LayerNorm from epilogue statistics")


@gpu
def test_gemm_strided_views():
    """Operands and output as column slices of wider buffers (leading dimension > width)."""
    from ittai_b200 import ops
    big_a, big_w = _rand(256, 1024, seed=7), _rand(512, 1024, scale=0.05, seed=8)
    a, w = big_a[:, 256:768], big_w[:, 512:1024]
    out_big = torch.zeros(256, 1024, dtype=torch.bfloat16, device="cuda")  # columns 128..640 receive the product
    st = ops.new_status("cuda")
    ops.gemm(a, w, st, out=out_big[:, 128:640])
    ops.check_status(st)
    _check(out_big[:, 128:640], a.float() @ w.float().t(), "strided")
    assert (out_big[:, :128] == 0).all() and (out_big[:, 640:] == 0).all()


def test_gemm_argument_errors():
    import ctypes as C
    from ittai_b200 import _C
    g = _C.Gemm()
    assert _C.lib().ittai_gemm_bf16_launch(C.byref(g), None) == -1


@gpu
@pytest.mark.parametrize("m", [12544, 700])
def test_gemm_chain_equals_separate_launches(m):
    """Four dependent GEMMs of the SigLIP layer shapes (out-proj with an in-place residual and output statistics, fc1 with
    a folded LayerNorm and GELU, fc2 with an in-place residual, the next QKV projection with a folded LayerNorm) in one
    persistent launch: bit-identical to the same GEMMs launched one by one, on a second run over the same flag buffer
    (cleared in between) as well."""
    from ittai_b200 import _C, ops
    D, F = 768, 3072
    gen = torch.Generator(device="cuda").manual_seed(4)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, generator=gen, device="cuda") * scale)
    attn, x0 = rnd(m, D).bfloat16(), rnd(m, D).bfloat16()
    wo, w1, w2, wq = rnd(D, D, scale=0.03).bfloat16(), rnd(F, D, scale=0.03).bfloat16(), rnd(D, F, scale=0.02).bfloat16(), rnd(3 * D, D, scale=0.03).bfloat16()
    bo, b1, b2, bq = rnd(D, scale=0.1), rnd(F, scale=0.1), rnd(D, scale=0.1), rnd(3 * D, scale=0.1)
    cs1, csq = w1.float().sum(1), wq.float().sum(1)
    st = ops.new_status(attn.device)

    def run(chained):
        x, h, qkv = x0.clone(), torch.empty(m, F, dtype=torch.bfloat16, device="cuda"), torch.empty(m, 3 * D, dtype=torch.bfloat16, device="cuda")
        sa, sm = (torch.zeros(m, D // 128, 2, device="cuda") for _ in range(2))
        args = [dict(a=attn, w=wo, bias=bo, residual=x, out=x, stats_out=sa),
                dict(a=x, w=w1, bias=b1, epi=_C.EPI_GELU, out=h, row_stats=sa, col_sums=cs1, stats_eps=1e-6),
                dict(a=h, w=w2, bias=b2, residual=x, out=x, stats_out=sm),
                dict(a=x, w=wq, bias=bq, out=qkv, row_stats=sm, col_sums=csq, stats_eps=1e-6)]
        if chained:
            flags = torch.zeros(4 * 2 * ((m + 255) // 256), dtype=torch.int32, device="cuda")
            for _ in range(2):
                x.copy_(x0)
                flags.zero_()
                ops.gemm_chain([ops.gemm_desc(k.pop("a"), k.pop("w"), st, **k)[0] for k in [dict(d) for d in args]], flags)
        else:
            for d in args:
                d = dict(d)
                ops.gemm(d.pop("a"), d.pop("w"), st, **d)
        ops.check_status(st)
        return x, h, qkv, sa, sm

    for got, want, name in zip(run(True), run(False), ("x", "h", "qkv", "stats_a", "stats_m")):
        assert torch.equal(got, want), f"{name}: chained GEMMs differ from separate launches ({(got.float() - want.float()).abs().max().item():.4g})"
