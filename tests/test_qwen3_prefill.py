"""Qwen3 tensor-core prefill: the embedding Engine (drop-in surface) and the decoder's dense prompt path (GPU)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import qwen3_hf as hf
from oracle import qwen3_ref as ref

gpu = pytest.mark.gpu


def test_packing_metadata():
    from ittai_b200.qwen3 import rope_perm
    from ittai_b200.qwen3.engine import packing
    pos, seq, slot, seqs, T = packing([3, 1, 4])
    assert T == 8 and pos.tolist() == [0, 1, 2, 0, 0, 1, 2, 3] and slot.tolist() == list(range(8)) and not seq.any()
    assert seqs.tolist() == [[0, 3, 0, 3], [3, 1, 3, 1], [4, 4, 4, 4]]
    p = rope_perm(2)
    assert p[:4].tolist() == [0, 64, 1, 65] and p[128:130].tolist() == [128, 192]


@gpu
def test_engine_embeddings_match_oracle(tiny_hf):
    """Varlen batch through Engine.forward: L2-normalised last-token embedding vs the restatement and the eager model
    (the reference's own gate is min cosine > 0.999: src/ittai/qwen3/model.py:63-68)."""
    from ittai_b200.qwen3 import Qwen3Embedder
    model, dims = tiny_hf
    lens = [1, 37, 128, 129, 200, 64]
    ids = [hf.prompt_ids(n, seed=10 + i, vocab=dims.vocab).tolist() for i, n in enumerate(lens)]
    emb = Qwen3Embedder(model, max_tokens=1024, max_seqs=8)
    out = emb.embed(ids).cpu()
    emb.engine.check()
    assert out.shape == (len(lens), 1024) and torch.allclose(out.norm(dim=-1), torch.ones(len(lens)), atol=1e-4)
    for i, s in enumerate(ids):
        R = ref.Qwen3Ref(model.state_dict(), dims, 256)
        R.forward(torch.tensor(s))
        assert F.cosine_similarity(out[i], R.embed_pool(), dim=0) >= 0.9995, f"sequence {i} (length {lens[i]})"
    # same batch again: the cached graph replays; a different packing captures a new one
    assert torch.equal(emb.embed(ids).cpu(), out)
    out2 = emb.embed(ids[::-1]).cpu()
    assert F.cosine_similarity(out2.flip(0), out, dim=-1).min() >= 0.99999
    assert emb.validate(ids[:3]) > 0.999
    # the same engine with every RMSNorm as a pass of its own (the eager modules' rounding points) instead of folded into
    # the GEMMs: both clear the gate, and they agree with each other far inside it
    from ittai_b200.qwen3.engine import Engine
    assert emb.engine.core.fold_norm
    plain = Engine(model.state_dict(), 1024, 8, fold_norm=False)
    out3 = plain.forward(ids).cpu()
    plain.check()
    assert not plain.core.fold_norm and F.cosine_similarity(out3, out, dim=-1).min() >= 0.9999
    for i, s in enumerate(ids):
        R = ref.Qwen3Ref(model.state_dict(), dims, 256)
        R.forward(torch.tensor(s))
        assert F.cosine_similarity(out3[i], R.embed_pool(), dim=0) >= 0.9995


@gpu
def test_decoder_dense_prefill_matches_stepwise(tiny_hf):
    """Filling the cache with the tensor-core prefill gives the same continuation as feeding the prompt token by token."""
    from ittai_b200.qwen3 import Qwen3Decoder
    model, dims = tiny_hf
    prompt = hf.prompt_ids(150, seed=21, vocab=dims.vocab)
    d = Qwen3Decoder(model, max_batch=1, kv_capacity=256)
    first_a = int(d.prefill(prompt, tensor_cores=False)[0])
    la, ka = d.logits[0].float().cpu(), d.kcache[:, 0, :, :150].float().cpu()
    rest_a = d.decode(8).cpu()
    d.reset()
    first_b = int(d.prefill(prompt, tensor_cores=True)[0])
    lb, kb = d.logits[0].float().cpu(), d.kcache[:, 0, :, :150].float().cpu()
    rest_b = d.decode(8).cpu()
    assert d.pos.tolist() == [158]
    assert F.cosine_similarity(la, lb, dim=0) >= 0.9999 and (la - lb).abs().max() <= 3e-2
    assert F.cosine_similarity(ka.flatten(), kb.flatten(), dim=0) >= 0.9999
    assert first_a == first_b and torch.equal(rest_a, rest_b)


@gpu
def test_decoder_dense_prefill_batch2_and_append(tiny_hf):
    from ittai_b200.qwen3 import Qwen3Decoder
    model, dims = tiny_hf
    p = torch.stack([hf.prompt_ids(70, seed=31, vocab=dims.vocab), hf.prompt_ids(70, seed=32, vocab=dims.vocab)])
    d2 = Qwen3Decoder(model, max_batch=2, kv_capacity=128)
    d2.prefill(p[:, :40], tensor_cores=True)          # 39 dense + 1 stepped
    d2.prefill(p[:, 40:], tensor_cores=True)          # appended behind a non-empty cache: causal offset
    l2 = d2.logits.float().cpu()
    d1 = Qwen3Decoder(model, max_batch=1, kv_capacity=128)
    for b in range(2):
        d1.reset()
        d1.prefill(p[b], tensor_cores=False)
        assert F.cosine_similarity(l2[b], d1.logits[0].float().cpu(), dim=0) >= 0.9999
