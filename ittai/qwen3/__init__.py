"""``ittai.qwen3``: the names the reference package exports (``src/ittai/qwen3/__init__.py:1-6``), served by
``ittai_b200.qwen3``.  The reference's kernel classes (``MegaBase``, ``MegaSm80``, ``MegaSm90``, ``acc_mn_view``) are
CuTe-DSL code generators with no counterpart in a prebuilt CUDA library and are not provided."""
from ittai_b200.qwen3.config import *  # noqa: F401,F403
from ittai_b200.qwen3 import Engine, PrefillCore, Qwen3Decoder, Qwen3Embedder, build_tasks, pack_weights, rope_perm, rope_table  # noqa: F401

__all__ = ["Qwen3Embedder"]
