"""Host request loop around the batch decode kernel: continuous batching over the fixed sequence slots of one
``Qwen3Decoder``.  The reference has no decode loop at all (it embeds; ``src/ittai/qwen3/model.py:79-90`` batches
independent prompts), so this is the serving-side counterpart of its ``embed`` batching for generation.

Every iteration admits waiting requests into free slots (their prompts, minus the last token, go through the tensor-core
prefill into the slot's own cache region; the last token becomes the slot's next input), runs ``chunk`` greedy steps of
the whole batch as ONE persistent launch, and retires requests that reached their token budget or produced their stop
id.  A slot's cache is one contiguous region of ``kv_capacity`` rows: there is no paging, a request longer than the
capacity is refused at submission.  Idle slots decode a dummy token at position 0 (the kernel's batch is fixed); their
output is dropped and their position is reset every iteration.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field


@dataclass
class Request:
    rid: int
    prompt: list
    max_new_tokens: int
    stop_id: int | None = None
    tokens: list = field(default_factory=list)
    slot: int | None = None

    @property
    def done(self) -> bool:
        return len(self.tokens) >= self.max_new_tokens or (self.stop_id is not None and self.stop_id in self.tokens)


class DecodeServer:
    """``DecodeServer(decoder, chunk=8)``: ``submit`` prompts, then ``step()`` (one admission + ``chunk`` decode steps) or
    ``run()`` until everything submitted has finished.  Results: ``{request id: generated ids}``."""

    def __init__(self, decoder, chunk: int = 8):
        self.dec, self.chunk = decoder, int(chunk)
        self.waiting: deque = deque()
        self.slots: list = [None] * decoder.B
        self.finished: dict = {}
        self._next = 0
        decoder.reset()

    def submit(self, prompt_ids, max_new_tokens: int, stop_id: int | None = None) -> int:
        prompt = [int(t) for t in prompt_ids]
        if not prompt or max_new_tokens < 1:
            raise ValueError("a request needs at least one prompt token and one token to generate")
        # the last generated token is never fed back, so the cache holds at most prompt + max_new_tokens - 1 rows; chunks
        # run to their end, which may overshoot a budget by up to chunk - 1 steps
        if len(prompt) + max_new_tokens - 1 + self.chunk - 1 > self.dec.cap:
            raise ValueError(f"request needs {len(prompt) + max_new_tokens - 1 + self.chunk - 1} cache rows, capacity is {self.dec.cap}")
        r = Request(self._next, prompt, int(max_new_tokens), stop_id)
        self._next += 1
        self.waiting.append(r)
        return r.rid

    @property
    def busy(self) -> bool:
        return bool(self.waiting) or any(s is not None for s in self.slots)

    def _admit(self) -> None:
        fresh = {}
        for b in range(self.dec.B):
            if self.slots[b] is None and self.waiting:
                r = self.waiting.popleft()
                r.slot, self.slots[b] = b, r
                self.dec.set_length(b, 0)
                fresh[b] = r
        if fresh:
            self.dec.prefill_slots({b: r.prompt[:-1] for b, r in fresh.items()})
        for b in range(self.dec.B):
            r = self.slots[b]
            if r is None:                         # idle slot: one dummy token at position 0, output dropped
                self.dec.set_length(b, 0)
                self.dec.next_id[b] = 0
            elif b in fresh:
                self.dec.next_id[b] = r.prompt[-1]

    def step(self) -> list:
        """One iteration; returns the ids of the requests that finished in it."""
        self._admit()
        if not any(s is not None for s in self.slots):
            return []
        out = self.dec.decode(self.chunk).cpu()               # [B, chunk]; next_id keeps every slot's last token
        retired = []
        for b, r in enumerate(self.slots):
            if r is None:
                continue
            for t in out[b].tolist():
                if r.done:
                    break
                r.tokens.append(t)
            if r.done:
                if r.stop_id is not None and r.stop_id in r.tokens:
                    r.tokens = r.tokens[:r.tokens.index(r.stop_id) + 1]
                self.finished[r.rid] = r.tokens[:r.max_new_tokens]
                self.slots[b] = None
                retired.append(r.rid)
        return retired

    def run(self) -> dict:
        while self.busy:
            self.step()
        return self.finished
