"""Qwen3-0.6B path: the reference's names (``src/ittai/qwen3/__init__.py:1-6`` star-exports its constants and lists
``Engine, build_tasks, rope_perm, Qwen3Embedder``) plus the KV-cache decode engine the reference does not have."""
from .config import *  # noqa: F401,F403
from .decoder import Qwen3Decoder, pack_weights, rope_table
from .engine import Engine, PrefillCore, build_tasks, rope_perm
from .model import Qwen3Embedder
from .serving import DecodeServer, Request

__all__ = ["Qwen3Embedder", "Qwen3Decoder", "DecodeServer"]
