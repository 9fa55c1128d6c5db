"""Hugging Face eager Qwen3 as the checker (test infrastructure, never the product path).

The reference validates its kernels against ``AutoModel(...)`` outputs
(reference ``src/ittai/qwen3/model.py:32-37``); the decode loop, KV cache, tied lm_head and argmax
exist only in ``transformers``' ``Qwen3ForCausalLM``, which is therefore the oracle for them.
Everything is built offline from a config with seeded random initialisation.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Qwen3Dims:
    """Qwen3-0.6B geometry (reference ``src/ittai/qwen3/config.py:1``); layers and vocab may shrink for tests."""
    n_layers: int = 28
    vocab: int = 151936
    hidden: int = 1024
    n_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 128
    inter: int = 3072
    eps: float = 1e-6
    theta: float = 1e6


FULL = Qwen3Dims()
TINY = Qwen3Dims(n_layers=2, vocab=2048)


def build_hf(dims: Qwen3Dims = FULL, seed: int = 0, dtype=torch.bfloat16, device="cpu", attn="sdpa"):
    """Random-init ``Qwen3ForCausalLM`` (normal std 0.02, tied head), seeded on the CPU generator."""
    from transformers import Qwen3Config, Qwen3ForCausalLM

    cfg = Qwen3Config(
        vocab_size=dims.vocab, hidden_size=dims.hidden, intermediate_size=dims.inter,
        num_hidden_layers=dims.n_layers, num_attention_heads=dims.n_heads,
        num_key_value_heads=dims.n_kv_heads, head_dim=dims.head_dim, rms_norm_eps=dims.eps,
        rope_theta=dims.theta, max_position_embeddings=40960, tie_word_embeddings=True,
        attention_bias=False, use_sliding_window=False, initializer_range=0.02,
    )
    cfg._attn_implementation = attn
    torch.manual_seed(seed)
    model = Qwen3ForCausalLM(cfg)
    inv_freq = model.model.rotary_emb.inv_freq.clone()
    model = model.to(dtype).eval()
    # ``from_pretrained(dtype=bf16)`` (how the reference loads) leaves the rotary inverse frequencies in fp32,
    # whereas ``module.to(bf16)`` would round that buffer too; put the fp32 values back.
    model.model.rotary_emb.inv_freq = inv_freq
    if device != "cpu":
        model = model.to(device)
    return model


def prompt_ids(n: int, seed: int, vocab: int = FULL.vocab) -> torch.Tensor:
    """``n`` token ids uniform over [0, vocab) from a seeded CPU generator."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g, dtype=torch.int64)


@torch.no_grad()
def greedy(model, ids: torch.Tensor, n_steps: int, forced: torch.Tensor | None = None):
    """Prefill ``ids`` then ``n_steps`` greedy steps.

    Returns (next_ids[n_steps], logits[n_steps, V] bf16, cache).  ``next_ids[0]`` is the argmax
    after the prompt.  With ``forced`` the fed-back ids are taken from it (teacher forcing) while
    the returned ids remain the model's own argmax.
    """
    from transformers import DynamicCache

    dev = next(model.parameters()).device
    cache = DynamicCache(config=model.config)
    out = model(input_ids=ids[None].to(dev), past_key_values=cache, use_cache=True)
    logits = [out.logits[0, -1]]
    picks = [int(logits[-1].argmax())]
    for s in range(1, n_steps):
        feed = picks[-1] if forced is None else int(forced[s - 1])
        out = model(input_ids=torch.tensor([[feed]], device=dev), past_key_values=cache, use_cache=True)
        logits.append(out.logits[0, -1])
        picks.append(int(logits[-1].argmax()))
    return torch.tensor(picks, dtype=torch.int64), torch.stack(logits).cpu(), cache


def cache_kv(cache, layer: int):
    """(K, V) of one layer as [B, n_kv, len, head_dim] tensors, across transformers versions."""
    if hasattr(cache, "layers"):
        lyr = cache.layers[layer]
        return lyr.keys, lyr.values
    return cache.key_cache[layer], cache.value_cache[layer]


@torch.no_grad()
def time_decode_cpu(dims: Qwen3Dims, kv_len: int, n_steps: int, seed: int = 0, threads: int | None = None):
    """Time HF eager batch-1 decode on host cores at a given KV length.

    The cache is filled with N(0,1) bf16 keys/values directly (a decode step's cost depends on the
    cache length, not its contents), which bounds the sample: no CPU prefill of ``kv_len`` tokens.
    Returns dict(tok_s, ms_per_tok, threads, steps, kv_len).
    """
    from transformers import DynamicCache

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    model = build_hf(dims, seed)
    cache = DynamicCache(config=model.config)
    g = torch.Generator().manual_seed(seed + 1)
    for l in range(dims.n_layers):
        k = torch.randn(1, dims.n_kv_heads, kv_len, dims.head_dim, generator=g).to(torch.bfloat16)
        v = torch.randn(1, dims.n_kv_heads, kv_len, dims.head_dim, generator=g).to(torch.bfloat16)
        cache.update(k, v, l)
    tok = torch.tensor([[1]])
    pos = kv_len
    for w in range(2):  # warm-up
        o = model(input_ids=tok, past_key_values=cache, use_cache=True)
        tok = o.logits[:, -1].argmax(-1, keepdim=True)
    t0 = time.perf_counter()
    for s in range(n_steps):
        o = model(input_ids=tok, past_key_values=cache, use_cache=True)
        tok = o.logits[:, -1].argmax(-1, keepdim=True)
    dt = time.perf_counter() - t0
    return dict(tok_s=n_steps / dt, ms_per_tok=dt / n_steps * 1e3, threads=threads, steps=n_steps, kv_len=kv_len)
