"""Host engine of the Qwen3-0.6B KV-cache decode loop.

The reference's ``Engine`` (reference ``src/ittai/qwen3/engine.py:87-187``) packs weights, owns every
device buffer as a torch tensor and launches one persistent kernel per forward; this class keeps that
shape for the decode loop the reference does not have: torch owns the buffers, the C-ABI library
borrows raw pointers and the current stream, and one cooperative launch runs ``n_steps`` tokens with
the argmax fed back on the device.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _C
from .config import D, DGU, DQ, DQKV, EPS, FF, HD, NKV, THETA


def _strip(sd: dict) -> dict:
    """Drop the ``model.`` prefix as the reference does (``src/ittai/qwen3/engine.py:91``)."""
    return {k.removeprefix("model."): v for k, v in sd.items()}


def pack_weights(sd: dict, n_layers: int, device) -> dict:
    """Layer-stacked bf16 matrices in the layout ``include/ittai_b200.h`` documents.

    Differences from the reference's packing (``src/ittai/qwen3/engine.py:100-117``): the norm gains are
    kept as separate bf16 vectors instead of being folded into the weights, and Q/K rows stay in the
    half-split RoPE order (no ``rope_perm``), so the cache holds keys exactly as the eager model does.
    Gate and up rows are interleaved as there (``:110-111``).
    """
    sd = _strip(sd)
    bf = lambda t: t.detach().to(torch.bfloat16).contiguous().to(device)
    wqkv, wo, wgu, wd, ln1, ln2, qn, kn = ([] for _ in range(8))
    for l in range(n_layers):
        p = f"layers.{l}."
        wqkv.append(torch.cat([sd[p + f"self_attn.{n}_proj.weight"] for n in "qkv"]))
        wo.append(sd[p + "self_attn.o_proj.weight"])
        wgu.append(torch.stack([sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]], 1).reshape(DGU, D))
        wd.append(sd[p + "mlp.down_proj.weight"])
        ln1.append(sd[p + "input_layernorm.weight"])
        ln2.append(sd[p + "post_attention_layernorm.weight"])
        qn.append(sd[p + "self_attn.q_norm.weight"])
        kn.append(sd[p + "self_attn.k_norm.weight"])
    out = dict(wqkv=bf(torch.stack(wqkv)), wo=bf(torch.stack(wo)), wgu=bf(torch.stack(wgu)), wd=bf(torch.stack(wd)),
               ln1=bf(torch.stack(ln1)), ln2=bf(torch.stack(ln2)), qn=bf(torch.stack(qn)), kn=bf(torch.stack(kn)),
               fin_w=bf(sd["norm.weight"]), embed=bf(sd["embed_tokens.weight"]))
    assert out["wqkv"].shape == (n_layers, DQKV, D) and out["wo"].shape == (n_layers, D, DQ)
    assert out["wgu"].shape == (n_layers, DGU, D) and out["wd"].shape == (n_layers, D, FF)
    return out


def rope_table(kv_cap: int, device, theta: float = THETA) -> torch.Tensor:
    """bf16 [kv_cap, 128]: cos of the 64 pair angles, then sin; angle = pos * theta**(-2i/128) in fp32.

    Same angles as the reference's table (``src/ittai/qwen3/engine.py:118-122``), rounded to bf16 because the
    eager rotary module hands bf16 cos/sin to bf16 queries and keys.
    """
    inv = 1.0 / (theta ** (torch.arange(0, HD, 2, dtype=torch.int64).to(torch.float32) / HD))
    ang = torch.arange(kv_cap, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.sin()], 1).to(torch.bfloat16).contiguous().to(device)


class Qwen3Decoder:
    """Greedy batch decode with an in-place bf16 KV cache ``[L, B, 8, kv_capacity, 128]``.

    ``sd_or_model``: a Hugging Face Qwen3 module or its ``state_dict`` (no hub access is needed).
    ``.prefill(ids)`` feeds a prompt, ``.decode(n)`` runs n greedy steps, ``.logits`` holds the bf16 logits of
    the last step, ``.kcache`` / ``.vcache`` are the cache tensors.
    """

    def __init__(self, sd_or_model, max_batch: int = 1, kv_capacity: int = 8192, device="cuda"):
        sd = sd_or_model if isinstance(sd_or_model, dict) else sd_or_model.state_dict()
        sd = _strip(sd)
        if max_batch not in (1, 2, 4, 8):
            raise ValueError("max_batch must be 1, 2, 4 or 8")
        self.dev = torch.device(device)
        self.lib = _C.lib()
        n_sms = C.c_int()
        _C.check(self.lib.ittai_device_check(self.dev.index or 0, C.byref(n_sms)))
        self.n_sms = n_sms.value
        self.L = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
        self.V = sd["embed_tokens.weight"].shape[0]
        self.B, self.cap = max_batch, kv_capacity
        self.w = pack_weights(sd, self.L, self.dev)
        self.rope = rope_table(kv_capacity, self.dev)
        z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt, device=self.dev)
        self.kcache = z(self.L, self.B, NKV, self.cap, HD)
        self.vcache = z(self.L, self.B, NKV, self.cap, HD)
        self.pos = z(self.B, dt=torch.int32)
        self.next_id = z(self.B, dt=torch.int32)
        self.logits = z(self.B, self.V)
        self.status = z(_C.STATUS_WORDS, dt=torch.int32)
        nbytes = C.c_size_t()
        _C.check(self.lib.ittai_qwen3_decode_workspace_bytes(self.B, C.byref(nbytes)))
        self.workspace = z(nbytes.value + 256, dt=torch.uint8)
        self._ws_ptr = (self.workspace.data_ptr() + 255) // 256 * 256
        self.flags = 0
        self.spin_limit = 0                  # 0 = library default
        self.lengths = [0] * self.B          # host mirror of `pos`, for capacity checks without a device read
        self._unchecked = 0                  # steps launched whose status has not been read yet
        self._keep = None
        self._phase_clk = None
        self._core = None                    # dense prefill buffers, created at the first long prompt

    # ---- plumbing -------------------------------------------------------------------------------
    def _params(self, n_steps, n_forced, forced, out_ids, step_ns, write_logits=True) -> _C.Qwen3Decode:
        p = _C.Qwen3Decode()
        p.n_layers, p.vocab, p.kv_cap, p.batch = self.L, self.V, self.cap, self.B
        p.n_steps, p.n_forced, p.eps, p.write_logits, p.flags = n_steps, n_forced, EPS, int(write_logits), self.flags
        p.spin_limit = self.spin_limit
        for k, t in self.w.items():
            setattr(p, k, t.data_ptr())
        p.rope, p.kcache, p.vcache = self.rope.data_ptr(), self.kcache.data_ptr(), self.vcache.data_ptr()
        p.pos, p.next_id = self.pos.data_ptr(), self.next_id.data_ptr()
        p.forced = forced.data_ptr() if forced is not None else None
        p.out_ids, p.logits = out_ids.data_ptr(), self.logits.data_ptr()
        p.workspace, p.status = self._ws_ptr, self.status.data_ptr()
        p.step_ns = step_ns.data_ptr() if step_ns is not None else None
        p.phase_clk = self._phase_clk.data_ptr() if self._phase_clk is not None else None
        return p

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)

    def check_status(self) -> None:
        """Synchronise and raise if a bounded device wait ran out during the last launch.

        A launch that aborts leaves the device positions where they were (the kernel advances ``pos`` only when every
        step completed), so the host mirror ``lengths`` is advanced here, after the verdict, and re-read from the device
        when a launch failed: a later prefill or decode then works on consistent positions."""
        try:
            _C.decode_status(self.status.cpu().tolist())
        except _C.IttaiError:
            self._unchecked = 0
            self.lengths = self.pos.cpu().tolist()
            raise
        self.lengths = [n + self._unchecked for n in self.lengths]
        self._unchecked = 0

    def reset(self) -> None:
        self.pos.zero_()
        self.lengths = [0] * self.B
        self._unchecked = 0

    def rewind(self, length: int) -> None:
        """Set every sequence's cache length to ``length``: rows from there on stay in memory but are no longer attended
        and will be overwritten (benchmarks replay the same decode steps from one prefilled state)."""
        if not 0 <= length <= self.cap:
            raise ValueError(f"length {length} outside 0..{self.cap}")
        self.pos.fill_(length)
        self.lengths = [length] * self.B
        self._unchecked = 0

    def prefill_cache(self, ids) -> None:
        """Append prompts ``ids`` ([B, n] ints) to the caches with the tensor-core prefill only: no logits, no first id
        (``prefill`` adds the decode step that yields them)."""
        ids = torch.as_tensor(ids, dtype=torch.int32)
        self._prefill_dense(ids[None] if ids.dim() == 1 else ids)

    def _launch(self, n_steps, forced=None, timed=False, check=True):
        if max(self.lengths) + self._unchecked + n_steps > self.cap:
            raise ValueError(f"KV capacity {self.cap} exceeded: {max(self.lengths) + self._unchecked} cached + {n_steps} steps")
        n_forced = 0 if forced is None else forced.shape[0]
        out_ids = torch.empty(n_steps, self.B, dtype=torch.int32, device=self.dev)
        step_ns = torch.zeros(n_steps, dtype=torch.int64, device=self.dev) if timed else None
        p = self._params(n_steps, n_forced, forced, out_ids, step_ns)
        self._keep = (p, forced, out_ids, step_ns)
        _C.check(self.lib.ittai_qwen3_decode_launch(C.byref(p), self._stream()))
        self._unchecked += n_steps
        if check:
            self.check_status()
        return out_ids, step_ns

    # ---- public API -----------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids, tensor_cores: bool | None = None) -> torch.Tensor:
        """Feed prompts ``ids`` ([B, T] ints, equal lengths) into the cache; returns the first greedy id per sequence.

        Long prompts go through the tensor-core prefill (tcgen05 GEMMs + flash attention over all tokens at once) for
        every token but the last; the last token, or a short prompt as a whole, is fed through the decode kernel with
        its ids forced (lm_head only on the final one), which also yields the logits and the first generated id.
        ``tensor_cores`` forces one path (default: tensor cores from 32 prompt tokens on).
        """
        ids = torch.as_tensor(ids, dtype=torch.int32)
        if ids.dim() == 1:
            ids = ids[None]
        assert ids.shape[0] == self.B, "one prompt per sequence of the batch"
        T = ids.shape[1]
        if tensor_cores is None:
            tensor_cores = T >= 32
        if tensor_cores and T > 1:
            self._prefill_dense(ids[:, :T - 1])
            ids = ids[:, T - 1:]
        forced = ids.t().contiguous().to(self.dev, non_blocking=True)       # [T, B]
        out, _ = self._launch(forced.shape[0], forced=forced)
        return out[-1]

    def prefill_slots(self, prompts: dict) -> None:
        """Append token ids to the caches of SOME sequences of the batch, each with its own length: ``prompts`` maps a
        sequence index to a 1-D id list.  The other sequences' caches and positions stay as they are.  Tensor-core
        prefill, tokens of all named sequences packed into one activation matrix (the varlen packing of the reference's
        engine, ``src/ittai/qwen3/engine.py:20,149-150``); no logits are produced."""
        from .engine import PrefillCore
        if self._unchecked:
            self.check_status()
        todo = {int(b): torch.as_tensor(t, dtype=torch.int32).reshape(-1) for b, t in prompts.items() if len(t) > 0}
        if not todo:
            return
        for b, t in todo.items():
            if not 0 <= b < self.B:
                raise ValueError(f"sequence {b} outside 0..{self.B - 1}")
            if int(t.min()) < 0 or int(t.max()) >= self.V:
                raise ValueError(f"token id outside [0, {self.V})")
            if self.lengths[b] + len(t) > self.cap:
                raise ValueError(f"KV capacity {self.cap} exceeded: {self.lengths[b]} cached + {len(t)} prompt tokens")
        total = sum(len(t) for t in todo.values())
        if self._core is None or self._core.M < total:
            self._core = PrefillCore(self.w, self.L, max(total, 256), self.dev)
        i32 = lambda x: torch.as_tensor(x, dtype=torch.int32).to(self.dev, non_blocking=True)
        tokens, pos, seq, seqs, row = [], [], [], [], 0
        for b in range(self.B):                       # one record per sequence of the batch: the record index names the cache
            n = len(todo[b]) if b in todo else 0
            seqs.append([row, n, 0, self.lengths[b] + n])
            if n:
                tokens.append(todo[b])
                pos.append(torch.arange(self.lengths[b], self.lengths[b] + n, dtype=torch.int32))
                seq.append(torch.full((n,), b, dtype=torch.int32))
                row += n
        pos_d = i32(torch.cat(pos))
        self._core.status.zero_()
        self._core.run(total, i32(torch.cat(tokens)), pos_d, i32(torch.cat(seq)), pos_d, i32(seqs), max(len(t) for t in todo.values()),
                       self.rope, lambda l: (self.kcache[l], self.vcache[l]), self.cap, (HD, self.cap * HD, NKV * self.cap * HD))
        for b, t in todo.items():
            self.lengths[b] += len(t)
        self.pos.copy_(i32(self.lengths))
        from .. import ops
        ops.check_status(self._core.status)

    def set_length(self, b: int, length: int) -> None:
        """Set ONE sequence's cache length (0 frees the slot for a new request)."""
        if not 0 <= length <= self.cap:
            raise ValueError(f"length {length} outside 0..{self.cap}")
        if self._unchecked:
            self.check_status()
        self.lengths[b] = length
        self.pos[b] = length

    def _prefill_dense(self, ids: torch.Tensor) -> None:
        """Append ``ids`` ([B, n]) to every sequence's cache with the dense prefill kernels."""
        from .engine import PrefillCore
        B, n = ids.shape
        if self._unchecked:
            self.check_status()
        if int(ids.min()) < 0 or int(ids.max()) >= self.V:
            raise ValueError(f"token id outside [0, {self.V})")
        if max(self.lengths) + n > self.cap:
            raise ValueError(f"KV capacity {self.cap} exceeded: {max(self.lengths)} cached + {n} prompt tokens")
        if self._core is None or self._core.M < B * n:
            self._core = PrefillCore(self.w, self.L, max(B * n, 256), self.dev)
        i32 = lambda x: torch.as_tensor(x, dtype=torch.int32).to(self.dev, non_blocking=True)
        base = torch.tensor(self.lengths, dtype=torch.int32)
        pos = (base[:, None] + torch.arange(n, dtype=torch.int32)[None, :]).reshape(-1)
        seq = torch.arange(B, dtype=torch.int32)[:, None].expand(B, n).reshape(-1)
        seqs = torch.tensor([[b * n, n, 0, self.lengths[b] + n] for b in range(B)], dtype=torch.int32)
        pos_d = i32(pos)
        cap = self.cap
        self._core.status.zero_()
        self._core.run(B * n, i32(ids.reshape(-1)), pos_d, i32(seq), pos_d, i32(seqs), n, self.rope,
                       lambda l: (self.kcache[l], self.vcache[l]), cap, (HD, cap * HD, NKV * cap * HD))
        self.pos += n
        self.lengths = [x + n for x in self.lengths]
        from .. import ops
        ops.check_status(self._core.status)

    @torch.no_grad()
    def decode(self, n_steps: int, timed: bool = False, check: bool = True):
        """Run ``n_steps`` greedy steps from ``next_id``; returns int32 ``[B, n_steps]`` (device tensor).

        With ``timed`` also returns the device ``globaltimer`` stamp (ns) taken at the end of every step.
        """
        out, ns = self._launch(n_steps, timed=timed, check=check)
        return (out.t(), ns) if timed else out.t()

    @torch.no_grad()
    def decode_static(self, n_steps: int) -> torch.Tensor:
        """``decode`` through ``ittai_qwen3_decode_launch_static``: the kernel's scratch is the library's built-in
        device array instead of this object's workspace tensor (for hosts that cannot allocate device memory; batch
        at most 2).  Returns int32 ``[B, n_steps]``.  Calls that overlap on the GPU share that one array and race."""
        if max(self.lengths) + n_steps > self.cap:
            raise ValueError(f"KV capacity {self.cap} exceeded: {max(self.lengths)} cached + {n_steps} steps")
        out_ids = torch.empty(n_steps, self.B, dtype=torch.int32, device=self.dev)
        p = self._params(n_steps, 0, None, out_ids, None)
        p.workspace = None
        self._keep = (p, out_ids)
        _C.check(self.lib.ittai_qwen3_decode_launch_static(C.byref(p), self._stream()))
        self._unchecked += n_steps
        self.check_status()
        return out_ids.t()

    @torch.no_grad()
    def decode_profiled(self, n_steps: int) -> torch.Tensor:
        """Decode ``n_steps`` tokens recording CTA 0's SM cycle counter for every phase.

        Returns int64 ``[n_steps, 5*L+1, 2]``: cycles at (inputs of the phase complete, phase finished)."""
        self._phase_clk = torch.zeros(n_steps, 5 * self.L + 1, 2, dtype=torch.int64, device=self.dev)
        try:
            self._launch(n_steps)
        finally:
            clk, self._phase_clk = self._phase_clk, None
        return clk

    @torch.no_grad()
    def decode_forced(self, ids) -> torch.Tensor:
        """Teacher forcing: feed ``ids`` ([B, T]) one per step but run the head on every step.

        Returns the model's own argmax ``[B, T]``; ``.logits`` holds the last step's logits.
        """
        ids = torch.as_tensor(ids, dtype=torch.int32)
        if ids.dim() == 1:
            ids = ids[None]
        outs = []
        for t in range(ids.shape[1]):
            self.next_id.copy_(ids[:, t].to(self.dev))
            outs.append(self.decode(1)[:, 0].clone())
        return torch.stack(outs, 1)

    @torch.no_grad()
    def run_phase(self, phase: int, layer: int) -> None:
        """Launch one phase of one layer as its own kernel (unit tests, per-phase profiles)."""
        out_ids = torch.empty(1, self.B, dtype=torch.int32, device=self.dev)
        p = self._params(1, 0, None, out_ids, None)
        self._keep = (p, out_ids)
        _C.check(self.lib.ittai_qwen3_phase_launch(C.byref(p), phase, layer, self._stream()))
        self.check_status()

    # The vectors one phase hands to the next live in the workspace as flagged words.  h and hmid use 64-bit words:
    # two bf16 values in the low half, the tag of the producing (step, layer) in the high half.  qkv, attn and act use
    # 128-bit words of three 32-bit payloads + tag: four bf16 values per word for qkv and attn (the third payload is
    # unused), six for act.  These helpers let tests and profiles read a phase's output and
    # plant a phase's input; a phase launch runs at step 0, where layer l's tag is l + 1.
    _FLAGGED = (("h", D), ("qkv", DQKV), ("attn", DQ), ("hmid", D), ("act", FF))
    _WIDE = {"qkv": 4, "attn": 4, "act": 6}       # bf16 values per 128-bit word

    def _flagged_words(self, name: str) -> torch.Tensor:
        """int64 view of buffer ``name``: ``[B, n/2]`` for 64-bit words, ``[B, 512, 2]`` (low, high half) for 128-bit ones."""
        off = self._ws_ptr - self.workspace.data_ptr()
        up = lambda n: (n + 255) // 256 * 256
        o = off + up(64 * 4)
        for nm, n in self._FLAGGED:
            nb = self.B * (n // 2) * 8
            if nm == name:
                if nm in self._WIDE:
                    words = n // self._WIDE[nm]
                    return self.workspace[o:o + self.B * words * 16].view(torch.int64).view(self.B, words, 2)
                return self.workspace[o:o + nb].view(torch.int64).view(self.B, n // 2)
            o += up(nb)
        raise KeyError(name)

    def read_buf(self, name: str) -> torch.Tensor:
        """bf16 ``[B, n]`` payload of the flagged buffer ``name`` (h, qkv, attn, hmid, act)."""
        w = self._flagged_words(name)
        if name in self._WIDE:
            lo, hi = w[..., 0], w[..., 1]
            vals = [lo & 0xFFFF, (lo >> 16) & 0xFFFF, (lo >> 32) & 0xFFFF, (lo >> 48) & 0xFFFF, hi & 0xFFFF, (hi >> 16) & 0xFFFF]
            pair = torch.stack(vals[:self._WIDE[name]], -1)
        else:
            pair = torch.stack([w & 0xFFFF, (w >> 16) & 0xFFFF], -1)
        return pair.to(torch.int32).to(torch.int16).view(torch.bfloat16).reshape(self.B, -1)

    def write_buf(self, name: str, values: torch.Tensor, layer: int) -> None:
        """Plant ``values`` ([B, n] or [n]) in flagged buffer ``name`` with the tag of (step 0, ``layer``)."""
        per = self._WIDE.get(name, 2)
        v = values.to(torch.bfloat16).reshape(self.B, -1, per).to(self.dev).view(torch.int16).to(torch.int64) & 0xFFFF
        tag = (layer + 1) << 32
        if name in self._WIDE:
            lo = v[..., 0] | (v[..., 1] << 16) | (v[..., 2] << 32) | (v[..., 3] << 48)
            hi = (v[..., 4] | (v[..., 5] << 16) if per == 6 else torch.zeros_like(lo)) | tag
            self._flagged_words(name).copy_(torch.stack([lo, hi], -1))
        else:
            self._flagged_words(name).copy_(v[..., 0] | (v[..., 1] << 16) | tag)

    @torch.no_grad()
    def generate(self, prompt_host: torch.Tensor, n_steps: int) -> torch.Tensor:
        """End to end from host memory: copy the prompt ids in, prefill, decode, copy the ids out (host tensor [B, n_steps])."""
        self.reset()
        first = self.prefill(prompt_host)
        rest = self.decode(n_steps - 1) if n_steps > 1 else None
        out = first[:, None] if rest is None else torch.cat([first[:, None], rest], 1)
        return out.cpu()
