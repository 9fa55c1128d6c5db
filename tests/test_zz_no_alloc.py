"""The allocation-free decode entry point (``ittai_qwen3_decode_launch_static``) against the regular one (GPU).

Hosts that cannot allocate device memory at call time (all GPU memory pre-assigned to a pool, no device allocator in
the host runtime, or no tolerance for cudaMalloc's device-wide synchronisation) call this variant: its scratch is an
array built into the library.  The test drives both entry points through the C ABI on the same model and prompt and
expects the same tokens and logits, twice in a row because the built-in array keeps the previous call's contents.
Collected last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

from oracle import qwen3_hf as hf

gpu = pytest.mark.gpu


@gpu
def test_static_scratch_decode_matches_workspace_decode(tiny_hf):
    from ittai_b200 import _C
    from ittai_b200.qwen3 import Qwen3Decoder
    model, dims = tiny_hf
    prompt = hf.prompt_ids(20, seed=41, vocab=dims.vocab)
    d = Qwen3Decoder(model, max_batch=1, kv_capacity=64)

    d.reset()
    first = d.prefill(prompt, tensor_cores=False).clone()
    want_ids = d.decode(6).cpu()
    want_logits = d.logits[0].float().cpu()

    for attempt in range(2):                      # second round starts from the first round's leftovers in the array
        d.reset()
        d.prefill(prompt, tensor_cores=False)
        d.next_id.copy_(first)
        got_ids = d.decode_static(6).cpu()
        got_logits = d.logits[0].float().cpu()
        assert torch.equal(got_ids, want_ids), f"round {attempt}: ids differ"
        assert F.cosine_similarity(got_logits, want_logits, dim=0) >= 0.9999 and (got_logits - want_logits).abs().max() <= 3e-2
        assert d.pos.tolist() == [26]

    # batch 2 fits the built-in array as well; anything larger is refused without launching
    d2 = Qwen3Decoder(model, max_batch=2, kv_capacity=64)
    p2 = torch.stack([prompt, hf.prompt_ids(20, seed=42, vocab=dims.vocab)])
    d2.prefill(p2, tensor_cores=False)
    a = d2.decode(4).cpu()
    d2.reset()
    d2.prefill(p2, tensor_cores=False)
    assert torch.equal(d2.decode_static(4).cpu(), a)
    big = _C.Qwen3Decode()
    big.batch = 4
    assert _C.lib().ittai_qwen3_decode_launch_static(C.byref(big), None) == -1
    assert b"built-in scratch" in _C.lib().ittai_last_error()
