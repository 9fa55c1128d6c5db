"""Qwen3-0.6B path: the reference's constant names plus the decode engine
(reference ``src/ittai/qwen3/__init__.py:1-6`` star-exports its constants the same way)."""
from .config import *  # noqa: F401,F403
from .decoder import Qwen3Decoder, pack_weights, rope_table

__all__ = ["Qwen3Decoder"]
