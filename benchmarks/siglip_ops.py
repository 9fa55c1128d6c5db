"""Per-kernel timings of one SigLIP ViT-B/16 layer at batch B (default 64) on the GPU: each op repeated inside one CUDA
graph, so the figure includes the launch-to-launch gap a forward pass sees.  `python benchmarks/siglip_ops.py [B]`."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ittai_b200 import ops, _C
def us(fn, iters=50):
    for _ in range(5): fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters): fn()
    g.replay(); torch.cuda.synchronize()
    s.record(); g.replay(); e.record(); torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e3
B, S, D, H = (int(sys.argv[1]) if len(sys.argv) > 1 else 64), 196, 768, 12
M = B * S
st = ops.new_status('cuda')
x = torch.randn(M, D, device='cuda').bfloat16(); y = torch.empty_like(x)
gw = torch.randn(D, device='cuda'); gb = torch.randn(D, device='cuda')
print('layernorm  %.1f us' % us(lambda: ops.layernorm_rows(x, gw, gb, 1e-6, out=y)))
qkv = torch.randn(M, 3 * D, device='cuda').bfloat16(); o = torch.empty(M, D, device='cuda', dtype=torch.bfloat16)
seqs = torch.tensor([[b * S, S, b * S, S] for b in range(B)], dtype=torch.int32, device='cuda')
att = lambda: ops.attention(qkv, qkv[:, D:], qkv[:, 2 * D:], o, seqs, n_heads=H, group=1, head_dim=64, causal=False, max_q_len=S,
                            q_strides=(3 * D, 64), k_strides=(3 * D, 64, 0), v_strides=(3 * D, 64, 0), o_strides=(D, 64), max_kv_len=S,
                            q_rows_total=M, kv_rows_total=M, status=st)
print('attention  %.1f us' % us(att))
for (n, k, epi, res) in [(2304, 768, 0, False), (768, 768, 0, True), (3072, 768, 1, False), (768, 3072, 0, True)]:
    a = torch.randn(M, k, device='cuda').bfloat16(); w = (torch.randn(n, k, device='cuda') * 0.05).bfloat16()
    b = torch.randn(n, device='cuda'); r = torch.randn(M, n, device='cuda').bfloat16() if res else None
    out = torch.empty(M, n, device='cuda', dtype=torch.bfloat16)
    t = us(lambda: ops.gemm(a, w, st, bias=b, residual=r, epi=epi, out=out), 20)
    print('gemm N=%d K=%d epi=%d res=%d  %.1f us  %.0f TF' % (n, k, epi, res, t, 2.0 * M * n * k / t / 1e6))
ops.check_status(st)
