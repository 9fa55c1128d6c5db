"""Write the golden fixtures in this directory from the Hugging Face eager modules.

Run from the repository root:  python tests/golden/make_golden.py [qwen3_tiny|qwen3_full|siglip|qwen3_tasks ...]
(``qwen3_tasks`` needs ITTAI_REFERENCE=<checkout of the reference>; the others need only ``transformers``.)

The reference ships no fixtures; these are outputs of the ``transformers`` modules it validates
against (reference ``src/ittai/qwen3/model.py:32-37``, ``src/ittai/siglip/kernel.py:701-702``),
built offline from seeded random initialisation.  Weights are not stored: the fixtures are only
meaningful together with the torch / transformers versions recorded inside them, which regenerate
the same weights from the same seed.
"""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
HERE = os.path.dirname(os.path.abspath(__file__))


def _versions():
    import transformers
    return dict(torch=str(torch.__version__), transformers=transformers.__version__, threads=torch.get_num_threads())


def qwen3_tiny():
    from oracle import qwen3_hf as hf
    dims = hf.TINY
    m = hf.build_hf(dims, seed=0)
    ids = hf.prompt_ids(16, seed=0, vocab=dims.vocab)
    picks, logits, cache = hf.greedy(m, ids, 8)
    k1, v1 = hf.cache_kv(cache, 1)
    torch.save(dict(meta=dict(_versions(), dims=dims.__dict__, seed=0, prompt_seed=0, attn="sdpa", dtype="bf16"),
                    prompt=ids, ids=picks, logits=logits, k_layer1=k1[0].clone(), v_layer1=v1[0].clone()),
               os.path.join(HERE, "qwen3_tiny.pt"))
    print("qwen3_tiny", picks.tolist())


def _distance(logits, picks, free, ref_logits, ref_ids, top_i):
    """How far one run of the oracle is from the pinned one, in the units the parity tests use."""
    a, b = logits.float(), ref_logits.float()
    sa, sb = a[:, ::1009], b[:, ::1009]
    same = 0
    while same < len(ref_ids) and int(free[same]) == int(ref_ids[same]):
        same += 1
    return dict(strided_max_abs=(sa - sb).abs().max().item(),
                strided_min_cos=torch.nn.functional.cosine_similarity(sa, sb, dim=-1).min().item(),
                full_max_abs=(a - b).abs().max().item(),
                strided_rms=(sa - sb).pow(2).mean().sqrt().item(), full_rms=(a - b).pow(2).mean().sqrt().item(),
                full_min_cos=torch.nn.functional.cosine_similarity(a, b, dim=-1).min().item(),
                top8_max_abs=(torch.gather(a, 1, top_i) - torch.gather(b, 1, top_i)).abs().max().item(),
                argmax_agree=int((picks == ref_ids).sum()), free_running_prefix_equal=same)


def qwen3_full():
    """BASELINE config 1: full 28-layer model, 32-id prompt seed 0, 64 greedy steps on CPU.

    Besides the pinned run (bf16, sdpa attention) the fixture records how far the oracle's own variants are from it
    on the same weights and ids: bf16 with the eager attention backend, and fp32.  Each variant is teacher-forced on
    the pinned ids (every step judged on its own) and also run freely.  The parity tests use these distances as the
    noise floor of the comparison instead of a hand-picked constant.
    """
    from oracle import qwen3_hf as hf
    dims = hf.FULL
    m = hf.build_hf(dims, seed=0)
    ids = hf.prompt_ids(32, seed=0)
    picks, logits, cache = hf.greedy(m, ids, 64)
    top_v, top_i = logits.float().topk(8, dim=-1)
    k0, v0 = hf.cache_kv(cache, dims.n_layers - 1)
    floor = {}
    for name, kw in (("bf16_eager_attention", dict(attn="eager")), ("fp32_sdpa", dict(dtype=torch.float32))):
        mv = hf.build_hf(dims, seed=0, **kw)
        p_tf, l_tf, _ = hf.greedy(mv, ids, 64, forced=picks)
        p_free, _, _ = hf.greedy(mv, ids, 64)
        floor[name] = _distance(l_tf, p_tf, p_free, logits, picks, top_i)
        print(name, floor[name])
        del mv
    torch.save(dict(meta=dict(_versions(), dims=dims.__dict__, seed=0, prompt_seed=0, attn="sdpa", dtype="bf16"),
                    prompt=ids, ids=picks, top_values=top_v.to(torch.bfloat16), top_indices=top_i.to(torch.int32),
                    strided_logits=logits[:, ::1009].clone(), logit_norm=logits.float().norm(dim=-1),
                    k_last_layer_head0=k0[0, 0].clone(), variant_distance=floor),
               os.path.join(HERE, "qwen3_full_c1.pt"))
    print("qwen3_full", picks.tolist())


def siglip():
    """BASELINE config 3 at batch 1 and the first 4 images of the batch-64 stream (seed 3)."""
    from oracle import siglip_hf as hf
    m = hf.build_hf(seed=2)
    px = hf.pixels(4, seed=3)
    with torch.no_grad():
        out = m(pixel_values=px.to(torch.bfloat16))
        out32 = m.float()(pixel_values=px)
    torch.save(dict(meta=dict(_versions(), seed=2, pixel_seed=3, dtype="bf16"),
                    pooled_bf16=out.pooler_output.clone(), pooled_fp32=out32.pooler_output.clone(),
                    last_hidden_fp32_img0=out32.last_hidden_state[0, ::49].clone()),
               os.path.join(HERE, "siglip_b16.pt"))
    print("siglip", out32.pooler_output[0, :4])


TASK_CASES = {          # name -> (seqlens, MB_alloc, Bmax, n_tiles, spt, kv block, group_m)
    "single_short": ([37], 1, 1, (32, 8, 48, 8), 1, 64, 8),
    "ragged": ([300, 5, 129, 1, 64], 4, 8, (32, 8, 48, 8), 1, 64, 8),
    "straddling_sm90": ([100, 100, 100, 100, 100], 8, 8, (16, 4, 24, 4), 2, 128, 16),
    "one_block_each": ([128, 128, 128], 3, 4, (32, 8, 48, 8), 1, 64, 2),
    "long": ([1000, 1048], 16, 2, (16, 4, 24, 4), 2, 128, 8),
}


def qwen3_tasks():
    """Task lists of the reference's own ``build_tasks`` for a handful of packings.

    The reference's engine module cannot be imported here (its kernels need a newer CuTe DSL than this image has), but
    ``build_tasks`` is plain numpy: the function's source is taken out of ``src/ittai/qwen3/engine.py`` with ``ast`` and
    executed against the reference's own ``config.py``.  Stored: every case's T, the SHA-256 of its task and expect arrays,
    and the arrays themselves for the smaller cases."""
    import ast
    import hashlib
    import numpy as np
    root = os.environ.get("ITTAI_REFERENCE")
    if not root or not os.path.isdir(os.path.join(root, "src", "ittai")):
        raise SystemExit("set ITTAI_REFERENCE to a checkout of the reference (the directory that holds src/ittai)")
    ns = {"np": np}
    exec(compile(open(os.path.join(root, "src/ittai/qwen3/config.py")).read(), "config.py", "exec"), ns)
    src = open(os.path.join(root, "src/ittai/qwen3/engine.py")).read()
    fn = [n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "build_tasks"][0]
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "engine.py", "exec"), ns)
    out = {}
    for name, (lens, mb, bmax, tiles, spt, kvb, gm) in TASK_CASES.items():
        tasks, expect, T = ns["build_tasks"](lens, mb, bmax, ns["L"] + 1, tiles, spt, kvb, gm)
        out[name + "__T"] = np.int64(T)
        out[name + "__sha"] = np.frombuffer(hashlib.sha256(tasks.astype(np.int32).tobytes() + expect.astype(np.int32).tobytes()).digest(), dtype=np.uint8)
        if len(tasks) < 20000:
            out[name + "__tasks"], out[name + "__expect"] = tasks.astype(np.int32), expect.astype(np.int32)
        print(name, tasks.shape, expect.shape, T)
    np.savez_compressed(os.path.join(HERE, "qwen3_tasks.npz"), **out)


if __name__ == "__main__":
    which = sys.argv[1:] or ["qwen3_tiny", "qwen3_full", "siglip", "qwen3_tasks"]
    for w in which:
        globals()[w]()
