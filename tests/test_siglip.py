"""SigLIP ViT-B/16 path: oracle pinned by the golden fixture (CPU), CUDA engine against the oracle (GPU).

Gate (BASELINE north star): pooled-embedding cosine >= 0.9995 against the reference's eager path."""
import pytest
import torch
import torch.nn.functional as F

from oracle import siglip_hf as hf
from oracle import siglip_ref as ref

gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def vit():
    return hf.build_hf(seed=2)


def _golden(golden_dir):
    return torch.load(f"{golden_dir}/siglip_b16.pt", weights_only=True)


def test_restatement_matches_golden(vit, golden_dir):
    g = _golden(golden_dir)
    px = hf.pixels(4, seed=3)
    pooled, last = ref.SiglipRef(vit).forward(px)
    assert F.cosine_similarity(pooled, g["pooled_bf16"].float(), dim=-1).min() >= 0.9995
    assert F.cosine_similarity(pooled, g["pooled_fp32"].float(), dim=-1).min() >= 0.9995
    assert F.cosine_similarity(last[0, ::49].flatten(), g["last_hidden_fp32_img0"].float().flatten(), dim=0) >= 0.9995


def test_hf_rebuild_reproduces_golden(vit, golden_dir):
    g = _golden(golden_dir)
    with torch.no_grad():
        out = vit(pixel_values=hf.pixels(4, seed=3).to(torch.bfloat16)).pooler_output
    assert F.cosine_similarity(out.float(), g["pooled_bf16"].float(), dim=-1).min() >= 0.99999


@gpu
@pytest.mark.parametrize("B", [1, 4])
def test_engine_matches_golden_and_oracle(vit, golden_dir, B):
    from ittai_b200.siglip.kernel import Engine
    g = _golden(golden_dir)
    px = hf.pixels(4, seed=3)[:B]
    vm = hf.build_hf(seed=2, device="cuda")
    eng = Engine(vm, B)
    out = eng.forward({"pixel_values": px}).float().cpu()
    eng.check()
    assert F.cosine_similarity(out, g["pooled_bf16"].float()[:B], dim=-1).min() >= 0.9995
    assert F.cosine_similarity(out, g["pooled_fp32"].float()[:B], dim=-1).min() >= 0.9995
    want, _ = ref.SiglipRef(vit).forward(px)
    assert F.cosine_similarity(out, want, dim=-1).min() >= 0.9995
    assert (out - want).abs().max() <= 0.05 * want.abs().max()
    # a second call replays the captured graph and returns the same values
    assert torch.equal(eng.forward({"pixel_values": px}).float().cpu(), out)


@gpu
def test_engine_batch64_against_eager_on_device():
    """BASELINE config 3 at batch 64: the checker is the eager tower run on the same GPU."""
    from ittai_b200.siglip.kernel import Siglip2Embedder
    vm = hf.build_hf(seed=2, device="cuda")
    px = hf.pixels(64, seed=3)
    with torch.no_grad():
        want = vm(pixel_values=px.cuda().to(torch.bfloat16)).pooler_output.float().cpu()
    emb = Siglip2Embedder(vm, batch_size=64)
    out = emb.embed(px).float().cpu()
    emb.engine.check()
    cos = F.cosine_similarity(out, want, dim=-1)
    print("siglip B=64 min cos", cos.min().item())
    assert cos.min() >= 0.9995
    # ragged tail: 70 images -> one full batch and one padded batch
    px70 = torch.cat([px, px[:6]])
    out70 = emb.embed(px70).float().cpu()
    assert out70.shape == (70, 768) and torch.equal(out70[:64], out) and torch.equal(out70[64:], out[:6])


# ---- SigLIP2 NaFlex (variable resolution) at the base geometry ---------------------------------------------------------
NAFLEX_SHAPES = [(16, 16), (12, 20), (8, 8), (10, 25), (1, 1), (16, 15)]


def test_naflex_position_rows_match_the_eager_module():
    """The resized, padded position rows (CPU, fp32) are exactly what the eager embedding module computes."""
    from transformers.models.siglip2.modeling_siglip2 import Siglip2VisionEmbeddings
    from ittai_b200.siglip.kernel import resize_positions
    grid = torch.randn(16, 16, 24, generator=torch.Generator().manual_seed(0))
    want = Siglip2VisionEmbeddings.resize_positional_embeddings(grid, torch.tensor(NAFLEX_SHAPES), max_length=256)
    got = resize_positions(grid, NAFLEX_SHAPES, 256)
    assert torch.equal(got, want)
    with pytest.raises(ValueError):
        resize_positions(grid, [(17, 16)], 256)


@gpu
def test_naflex_engine_against_eager_on_device():
    """Ragged batch (full grid, wide, small, single-patch images) through the NaFlex path: Linear patch embedding, position
    rows resized per image, keys limited to each image's own rows in the encoder and in the pooling head."""
    from ittai_b200.siglip.kernel import Siglip2Embedder
    vm = hf.build_hf_naflex(seed=2, device="cuda")
    inp = hf.naflex_inputs(NAFLEX_SHAPES, seed=3)
    with torch.no_grad():
        want = vm(pixel_values=inp["pixel_values"].cuda().to(torch.bfloat16), pixel_attention_mask=inp["pixel_attention_mask"].cuda(),
                  spatial_shapes=inp["spatial_shapes"].cuda()).pooler_output.float().cpu()
        want32 = hf.build_hf_naflex(seed=2, dtype=torch.float32)(**inp).pooler_output
    emb = Siglip2Embedder(vm, batch_size=len(NAFLEX_SHAPES))
    out = emb.embed(inp).float().cpu()
    emb.engine.check()
    cos, cos32 = F.cosine_similarity(out, want, dim=-1), F.cosine_similarity(out, want32, dim=-1)
    print("naflex min cos vs bf16 eager", cos.min().item(), "vs fp32 eager", cos32.min().item())
    assert cos.min() >= 0.9995 and cos32.min() >= 0.9995
    # other shapes through the same engine (the graph is replayed; only the records and the position rows change)
    inp2 = hf.naflex_inputs(NAFLEX_SHAPES[::-1], seed=5)
    with torch.no_grad():
        want2 = vm(pixel_values=inp2["pixel_values"].cuda().to(torch.bfloat16), pixel_attention_mask=inp2["pixel_attention_mask"].cuda(),
                   spatial_shapes=inp2["spatial_shapes"].cuda()).pooler_output.float().cpu()
    out2 = emb.embed(inp2).float().cpu()
    assert F.cosine_similarity(out2, want2, dim=-1).min() >= 0.9995
    with pytest.raises(ValueError):
        bad = dict(inp)
        bad["pixel_attention_mask"] = torch.ones_like(inp["pixel_attention_mask"])
        emb.embed(bad)


# ---- so400m geometry (width 1152, 16 heads of 72, MLP 4304, patch 14): the kernels on zero-padded weights -----------------
def _so400m(naflex: bool, n_layers: int = 2, device="cpu", dtype=torch.bfloat16, seed: int = 5):
    return hf.build_hf_so400m(naflex, n_layers=n_layers, device=device, dtype=dtype, seed=seed)


def test_geometry_dispatch():
    from ittai_b200.siglip.kernel import fits_fast_path
    assert fits_fast_path(hf.build_hf(n_layers=1).config)
    assert not fits_fast_path(_so400m(False, n_layers=1).config) and not fits_fast_path(_so400m(True, n_layers=1).config)


@gpu
@pytest.mark.parametrize("naflex", [False, True])
def test_so400m_geometry_against_eager(naflex):
    """The benchmark default of the reference (`siglip2-so400m-patch14-384`, benchmarks/siglip.py:7) at two layers, and the
    same widths as a NaFlex tower: pooled embeddings against the eager tower on the same GPU (bf16) and on the CPU (fp32)."""
    from ittai_b200.siglip.kernel import Siglip2Embedder
    from ittai_b200.siglip.padded import PaddedEngine
    vm = _so400m(naflex, device="cuda")
    if naflex:
        inp = hf.naflex_inputs([(16, 16), (9, 21), (3, 5)], seed=8)
        kw = dict(pixel_values=inp["pixel_values"].cuda().to(torch.bfloat16), pixel_attention_mask=inp["pixel_attention_mask"].cuda(),
                  spatial_shapes=inp["spatial_shapes"].cuda())
        B = 3
    else:
        B = 2
        inp = {"pixel_values": torch.randn(B, 3, 384, 384, generator=torch.Generator().manual_seed(8))}
        kw = dict(pixel_values=inp["pixel_values"].cuda().to(torch.bfloat16))
    with torch.no_grad():
        want = vm(**kw).pooler_output.float().cpu()
        want32 = _so400m(naflex, dtype=torch.float32)(**inp).pooler_output
    emb = Siglip2Embedder(vm, batch_size=B)
    assert isinstance(emb.engine, PaddedEngine) and emb.engine.hdp == 128 and emb.engine.Dp == 1280 and emb.engine.Fp == 4352
    out = emb.embed(inp if naflex else inp["pixel_values"]).float().cpu()
    emb.engine.check()
    cos, cos32 = F.cosine_similarity(out, want, dim=-1), F.cosine_similarity(out, want32, dim=-1)
    print("so400m", "naflex" if naflex else "patch14-384", "min cos vs bf16 eager", cos.min().item(), "vs fp32 eager", cos32.min().item())
    assert out.shape == (B, 1152) and cos.min() >= 0.9995 and cos32.min() >= 0.9995
    assert torch.equal(emb.embed(inp if naflex else inp["pixel_values"]).float().cpu(), out)       # graph replay
    # the same tower with the separate LayerNorm pass, and with one GEMM per launch: same embeddings within the gate, and
    # chained vs unchained bit-identical
    from ittai_b200.siglip.kernel import Engine
    for kw in (dict(fold_ln=False), dict(chain=False)):
        alt = Siglip2Embedder(vm, batch_size=B, engine=Engine(vm, B, **kw))
        got = alt.embed(inp if naflex else inp["pixel_values"]).float().cpu()
        alt.engine.check()
        assert F.cosine_similarity(got, want, dim=-1).min() >= 0.9995
        if "chain" in kw and emb.engine.chain:
            assert torch.equal(got, out)


@gpu
def test_embed_from_host_memory_overlaps_copies_and_matches_device_inputs():
    """``embed`` on pixels in (pinned) host memory stages batch k + 1 on a copy stream while batch k is in the encoder; the
    embeddings equal those of the same pixels handed over on the device, batch by batch, short last batch included."""
    from ittai_b200.siglip.kernel import Siglip2Embedder
    vm = hf.build_hf(seed=2, device="cuda")
    emb = Siglip2Embedder(vm, batch_size=8)
    px = hf.pixels(8 * 3 + 5, seed=11)
    on_device = emb.embed(px.cuda())
    from_host = emb.embed(px.pin_memory())
    from_pageable = emb.embed(px.clone())
    assert on_device.shape == (29, 768)
    assert torch.equal(on_device, from_host) and torch.equal(on_device, from_pageable)
    hosts = emb.embed_batches([px[:8].pin_memory(), px[8:16].pin_memory()], to_host=True)
    torch.cuda.synchronize()
    assert all(h.is_pinned() for h in hosts) and torch.equal(torch.cat(hosts).cuda(), on_device[:16])
