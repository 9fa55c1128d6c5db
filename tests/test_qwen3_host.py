"""Host-side logic of the Qwen3 decode engine: weight packing, RoPE table, byte accounting (CPU only)."""
import torch

from ittai_b200.qwen3 import config as cfg
from ittai_b200.qwen3.decoder import pack_weights, rope_table
from oracle import qwen3_ref as ref


def test_constants_match_reference_names():
    assert (cfg.D, cfg.DQ, cfg.DKV, cfg.DQKV, cfg.DGU, cfg.FF, cfg.L, cfg.G) == (1024, 2048, 1024, 4096, 6144, 3072, 28, 2)
    assert abs(cfg.SCALE_LOG2 - 128 ** -0.5 * 1.4426950408889634) < 1e-12


def test_bytes_per_token():
    assert cfg.decode_bytes_per_token(4096) == 1_661_978_624
    assert cfg.decode_bytes_per_token(8192) - cfg.decode_bytes_per_token(4096) == 4096 * 114_688


def test_pack_weights_layout(tiny_hf):
    model, dims = tiny_hf
    sd = model.state_dict()
    w = pack_weights(sd, dims.n_layers, "cpu")
    l = 1
    p = f"model.layers.{l}."
    assert torch.equal(w["wqkv"][l, :2048], sd[p + "self_attn.q_proj.weight"])
    assert torch.equal(w["wqkv"][l, 2048:3072], sd[p + "self_attn.k_proj.weight"])
    assert torch.equal(w["wqkv"][l, 3072:], sd[p + "self_attn.v_proj.weight"])
    assert torch.equal(w["wgu"][l, 0::2], sd[p + "mlp.gate_proj.weight"])
    assert torch.equal(w["wgu"][l, 1::2], sd[p + "mlp.up_proj.weight"])
    assert torch.equal(w["wd"][l], sd[p + "mlp.down_proj.weight"])
    assert torch.equal(w["embed"], sd["model.embed_tokens.weight"])
    assert w["qn"].shape == (dims.n_layers, 128) and w["fin_w"].shape == (1024,)


def test_rope_table_matches_eager_rotary(tiny_hf):
    model, dims = tiny_hf
    t = rope_table(96, "cpu")
    cos, sin = model.model.rotary_emb(torch.zeros(1, dtype=torch.bfloat16), torch.arange(96)[None])
    assert torch.equal(t[:, :64], cos[0, :, :64]) and torch.equal(t[:, 64:], sin[0, :, :64])
    c, s = ref.rope_table(96, dims)
    assert torch.equal(t[:, :64].float(), c) and torch.equal(t[:, 64:].float(), s)


def test_embedder_batches_respect_both_limits():
    """The batching rule of ``Qwen3Embedder.embed``: runs of consecutive sequences under max_seqs and max_tokens."""
    from ittai_b200.qwen3.model import Qwen3Embedder
    import pytest
    e = Qwen3Embedder.__new__(Qwen3Embedder)
    e.max_seqs, e.max_tokens = 3, 10
    lens = [4, 4, 4, 1, 1, 1, 1, 10, 9, 1]
    runs = list(e._batches(lens))
    assert runs == [(0, 2), (2, 3), (5, 2), (7, 1), (8, 2)]
    assert sum(n for _, n in runs) == len(lens) and all(sum(lens[a:a + n]) <= 10 and n <= 3 for a, n in runs)
    assert list(e._batches([])) == []
    with pytest.raises(ValueError):
        list(e._batches([3, 11]))
