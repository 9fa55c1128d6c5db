"""Choosing between kernel configurations at construction time, with the choice remembered in a JSON file.

The reference times a grid of tile / stage / warp settings per GPU, rejects every candidate whose output strays from the
eager model (minimum cosine not above 0.999) and caches the fastest under a key of GPU name, model and size
(reference ``src/ittai/qwen3/model.py:50-77``, ``src/ittai/siglip/kernel.py:690-713``).  This build has one sm_100a kernel
set, so the candidates are the few real switches the engines have (LayerNorm folded into the GEMMs or not, QK-norm + RoPE
inside the QKV epilogue or as its own pass); the procedure is the reference's.
"""
from __future__ import annotations

import json
import os

CACHE_PATH = os.environ.get("ITTAI_TUNE_CACHE", os.path.join(os.path.dirname(os.path.abspath(__file__)), "tune_cache.json"))


def load_cache(path: str = None) -> dict:
    path = path or CACHE_PATH
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


def store_choice(key: str, choice: dict, path: str = None) -> None:
    path = path or CACHE_PATH
    cache = load_cache(path)
    cache[key] = choice
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(cache, f, indent=1, sort_keys=True)
    os.replace(tmp, path)


def choose(key: str, candidates, build, agreement, time_ms, threshold: float = 0.999, path: str = None, log=print) -> dict:
    """The cached choice for ``key``, or the fastest candidate that validates.

    ``build(cfg)`` makes an engine, ``agreement(engine)`` returns its minimum cosine against the eager model,
    ``time_ms(engine)`` its time per forward.  A candidate that raises or whose agreement is not above ``threshold`` is
    reported and skipped; if none is left the call fails, as the reference's does (``model.py:73-74``)."""
    cache = load_cache(path)
    if key in cache:
        return cache[key]
    timed = []
    for cfg in candidates:
        try:
            engine = build(cfg)
            cos = float(agreement(engine))
            if cos > threshold:
                ms = float(time_ms(engine))
                timed.append((ms, cfg))
                log(f"{cfg}: cos={cos:.5f} ok {ms:.3f} ms")
            else:
                log(f"{cfg}: cos={cos:.5f} MISMATCH")
            del engine
        except Exception as ex:      # a candidate that cannot be built or run is not a reason to stop the search
            log(f"{cfg}: failed ({type(ex).__name__}: {ex})")
    if not timed:
        raise RuntimeError("no kernel configuration passed validation (see the messages above)")
    best = min(timed, key=lambda t: t[0])[1]
    store_choice(key, best, path)
    return best
