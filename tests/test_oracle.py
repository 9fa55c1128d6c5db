"""The CPU restatement against the Hugging Face golden fixtures (no GPU)."""
import torch
import torch.nn.functional as F

from oracle import qwen3_hf as hf
from oracle import qwen3_ref as ref


def _load(golden_dir, name):
    return torch.load(f"{golden_dir}/{name}", weights_only=True)


def test_golden_meta(golden_dir):
    g = _load(golden_dir, "qwen3_tiny.pt")
    assert g["meta"]["attn"] == "sdpa" and g["meta"]["dtype"] == "bf16"
    assert g["logits"].shape == (8, hf.TINY.vocab)


def test_hf_rebuild_reproduces_golden(golden_dir, tiny_hf):
    """Same seed, same image -> same weights -> same ids and logits as the committed fixture."""
    g = _load(golden_dir, "qwen3_tiny.pt")
    model, dims = tiny_hf
    assert torch.equal(hf.prompt_ids(16, 0, dims.vocab), g["prompt"])
    picks, logits, _ = hf.greedy(model, g["prompt"], 8)
    assert torch.equal(picks, g["ids"])
    assert (logits.float() - g["logits"].float()).abs().max() <= 1e-2


def test_restatement_matches_hf_tiny(golden_dir, tiny_hf):
    g = _load(golden_dir, "qwen3_tiny.pt")
    model, dims = tiny_hf
    R = ref.Qwen3Ref(model.state_dict(), dims, 64)
    picks, logits = R.greedy(g["prompt"], 8, forced=g["ids"])
    gl = g["logits"].float()
    assert torch.equal(picks, g["ids"])
    assert (logits - gl).abs().max() <= 3e-2                       # bf16 logits max-abs gate
    assert F.cosine_similarity(logits, gl, dim=-1).min() >= 0.9995  # cosine gate
    # layer-1 keys: same placement, values equal up to bf16 rounding noise of layer 0's attention
    k = R.k[1, :, :R.len]
    gk = g["k_layer1"].float()[:, :R.len]
    assert k.shape == gk.shape and (k - gk).abs().max() <= 0.0625


def test_restatement_layer0_cache_bit_exact(tiny_hf):
    """Before any attention output feeds back, K/V rounding points are identical: >= 99.9 % of bf16 values equal."""
    from transformers import DynamicCache
    model, dims = tiny_hf
    ids = hf.prompt_ids(16, 0, dims.vocab)
    c = DynamicCache(config=model.config)
    with torch.no_grad():
        model(input_ids=ids[None], past_key_values=c, use_cache=True)
    R = ref.Qwen3Ref(model.state_dict(), dims, 32)
    R.forward(ids)
    k, v = hf.cache_kv(c, 0)
    assert (R.k[0, :, :16] == k[0].float()).float().mean() >= 0.999
    assert (R.v[0, :, :16] == v[0].float()).float().mean() >= 0.999


def test_full_model_fixture_shape(golden_dir):
    g = _load(golden_dir, "qwen3_full_c1.pt")
    assert g["ids"].shape == (64,) and g["prompt"].shape == (32,)
    # the greedy id is a top-1 logit (exact bf16 ties exist, so it need not be topk's first pick)
    hit = g["top_indices"].long() == g["ids"][:, None]
    assert hit.any(1).all()
    assert torch.equal((g["top_values"].float() * hit).sum(1), g["top_values"][:, 0].float())
    assert torch.equal(hf.prompt_ids(32, 0), g["prompt"])
