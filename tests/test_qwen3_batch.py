"""Batch-4 and batch-8 decode (BASELINE config 4 shape at a small size): sequences with their own caches, dense prefill
then greedy steps, against independent batch-1 runs of the same sequences (GPU).  The batched kernels run their GEMV
phases on tensor-core tiles, batch 1 on the fp32 pipes: the ids must agree all the same."""
import pytest
import torch
import torch.nn.functional as F

from oracle import qwen3_hf as hf

gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("batch", [8, 4])
def test_batch_matches_batch1(tiny_hf, batch):
    from ittai_b200.qwen3 import Qwen3Decoder
    model, dims = tiny_hf
    prompts = torch.stack([hf.prompt_ids(48, seed=50 + b, vocab=dims.vocab) for b in range(batch)])
    d8 = Qwen3Decoder(model, max_batch=batch, kv_capacity=96)
    first8 = d8.prefill(prompts).cpu()                     # 47 tokens on the tensor cores, the last one stepped
    rest8 = d8.decode(6).cpu()
    l8 = d8.logits.float().cpu()
    assert d8.pos.tolist() == [54] * batch
    d1 = Qwen3Decoder(model, max_batch=1, kv_capacity=96)
    for b in (0, 3, batch - 1):
        d1.reset()
        first1 = d1.prefill(prompts[b]).cpu()
        rest1 = d1.decode(6).cpu()
        cos = F.cosine_similarity(l8[b], d1.logits[0].float().cpu(), dim=0).item()
        assert cos >= 0.9999, f"sequence {b}: logits cosine {cos}"
        assert int(first8[b]) == int(first1[0]) and torch.equal(rest8[b], rest1[0]), f"sequence {b}: ids differ"
