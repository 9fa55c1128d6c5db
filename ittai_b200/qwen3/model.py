"""``Qwen3Embedder``: the reference's user-facing wrapper (reference ``src/ittai/qwen3/model.py:13-90``) over the B200 engine.

Differences forced by running offline: the first argument may be a Hugging Face Qwen3 module (or its state dict) instead
of a hub id, ``embed`` also takes ready-made token-id lists, and there is no autotune pass (one sm_100a kernel set, no
configuration grid); the reference's validation gate (minimum cosine > 0.999 against the eager model,
``model.py:63-68``) is available as ``validate``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .engine import Engine


class Qwen3Embedder:
    CANDIDATES = ({"fused_rope": True}, {"fused_rope": False})

    def __init__(self, model_id="Qwen/Qwen3-Embedding-0.6B", max_tokens=8192, max_seqs=256, device="cuda", tune=None):
        self.tok = None
        if isinstance(model_id, str):
            from transformers import AutoModel, AutoTokenizer
            self.tok = AutoTokenizer.from_pretrained(model_id, padding_side="left")
            self.model = AutoModel.from_pretrained(model_id, dtype=torch.bfloat16, device_map=device).eval()
        else:
            self.model = model_id
        self.sd = self.model if isinstance(self.model, dict) else self.model.state_dict()
        self.max_tokens, self.max_seqs, self.device, self.model_id = max_tokens, max_seqs, device, model_id
        # a hub id is tuned like the reference tunes (model.py:25); an in-memory module only on request
        tune = isinstance(model_id, str) if tune is None else tune
        self.engine = Engine(self.sd, max_tokens, max_seqs, device=device, **(self._tune() if tune else {}))

    def _tune(self, path=None) -> dict:
        """Fastest engine configuration that agrees with the eager module (minimum cosine above 0.999), remembered per
        GPU, model and size in the tuning cache: the reference's ``_tune`` (``model.py:50-77``) over this build's switches.
        The probe batch is 32 sequences of seeded random ids of mixed lengths (no tokenizer is needed)."""
        from .. import tuning
        if isinstance(self.model, dict):
            raise RuntimeError("tuning validates against the eager module: pass the module, not a state dict")
        g = torch.Generator().manual_seed(11)
        vocab = self.sd[[k for k in self.sd if k.endswith("embed_tokens.weight")][0]].shape[0]
        lens = [min(self.max_tokens // 32, n) for n in (24, 9, 240, 3)] * 8
        ids = [torch.randint(0, vocab, (max(n, 1),), generator=g).tolist() for n in lens]
        dev = next(self.model.parameters()).device
        body = self.model.model if hasattr(self.model, "lm_head") else self.model
        with torch.no_grad():
            ref = torch.stack([F.normalize(body(input_ids=torch.tensor([s], device=dev)).last_hidden_state[0, -1].float(), dim=-1) for s in ids])

        def time_ms(engine, iters=10):
            for _ in range(3):
                engine.forward(ids)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                engine.forward(ids)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / iters

        name = self.model_id if isinstance(self.model_id, str) else type(self.model).__name__
        key = f"{torch.cuda.get_device_name()}|{name}|{self.max_tokens}"
        return tuning.choose(key, self.CANDIDATES, lambda c: Engine(self.sd, self.max_tokens, self.max_seqs, device=self.device, **c),
                             lambda e: F.cosine_similarity(e.forward(ids).float().to(ref.device), ref, dim=-1).min().item(), time_ms, path=path)

    def _ids(self, texts, max_length):
        if len(texts) and not isinstance(texts[0], str):
            return [list(map(int, t))[:max_length] for t in texts]
        if self.tok is None:
            raise RuntimeError("no tokenizer loaded: pass lists of token ids")
        return [self.tok(t, truncation=True, max_length=max_length)["input_ids"] for t in texts]

    def _batches(self, lengths):
        """Cuts the sequences, in order, into runs that fit one forward: at most ``max_seqs`` sequences and ``max_tokens``
        tokens each (the batching rule of the reference's ``embed``, ``model.py:79-90``).  Yields (first, count)."""
        first, tokens = 0, 0
        for i, n in enumerate(lengths):
            if n > self.max_tokens:
                raise ValueError(f"sequence {i} has {n} tokens, more than max_tokens={self.max_tokens}")
            if i - first == self.max_seqs or tokens + n > self.max_tokens:
                yield first, i - first
                first, tokens = i, 0
            tokens += n
        if len(lengths) > first:
            yield first, len(lengths) - first

    @torch.no_grad()
    def embed(self, texts, max_length=2048):
        """fp32 ``[N, 1024]`` embeddings; every batch's result is cloned out of the engine's persistent buffer."""
        ids = self._ids(texts, max_length)
        parts = [self.engine.forward(ids[a:a + n]).clone() for a, n in self._batches([len(s) for s in ids])]
        return torch.cat(parts) if parts else torch.zeros(0, 1024)

    @torch.no_grad()
    def validate(self, ids, threshold=0.999):
        """Minimum cosine of the engine's embeddings against the eager module's last-token pooling; raises below ``threshold``."""
        if isinstance(self.model, dict):
            raise RuntimeError("validation needs the eager module, not a state dict")
        dev = next(self.model.parameters()).device
        body = self.model.model if hasattr(self.model, "lm_head") else self.model
        ref = []
        for s in ids:
            hs = body(input_ids=torch.tensor([s], device=dev)).last_hidden_state
            ref.append(F.normalize(hs[0, -1].float(), dim=-1))
        cos = F.cosine_similarity(self.embed(ids).to(dev), torch.stack(ref), dim=-1).min().item()
        if cos <= threshold:
            raise RuntimeError(f"engine output fails validation: min cosine {cos:.5f} <= {threshold}")
        return cos
