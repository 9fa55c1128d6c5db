"""tcgen05 GEMM and its fused epilogues against fp32 torch references of the same bf16 inputs (GPU).

Tolerance: the kernel accumulates in fp32 and rounds to bf16, so it agrees with the fp32 reference to one bf16 rounding
(2^-8 relative), twice where an epilogue rounds before a non-linearity and a tie falls the other way:
|got - want| <= 2^-6 * |want| + 2^-7 * rms(want)."""
import pytest
import torch

gpu = pytest.mark.gpu


def _check(got, want, what):
    got, want = got.float(), want.float()
    tol = 2.0 ** -6 * want.abs() + 2.0 ** -7 * want.pow(2).mean().sqrt()
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
    bias = torch.randn(n, device="cuda") * 0.1
    res = _rand(m, n, seed=6)
    st = ops.new_status("cuda")
    acc = a.float() @ w.float().t()
    rb = lambda x: x.to(torch.bfloat16).float()
    _check(ops.gemm(a, w, st, bias=bias), acc + bias, "bias")
    _check(ops.gemm(a, w, st, bias=bias, epi=_C.EPI_GELU),
           torch.nn.functional.gelu(rb(acc + bias), approximate="tanh"), "bias + gelu")
    _check(ops.gemm(a, w, st, bias=bias, residual=res), res.float() + rb(acc + bias), "bias + residual")
    _check(ops.gemm(a, w, st, residual=res), res.float() + rb(acc), "residual")
    g, u = rb(acc[:, 0::2]), rb(acc[:, 1::2])
    _check(ops.gemm(a, w, st, epi=_C.EPI_SWIGLU), rb(torch.nn.functional.silu(g)) * u, "swiglu")
    ops.check_status(st)


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
