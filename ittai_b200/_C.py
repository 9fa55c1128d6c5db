"""ctypes binding of ``libittai_b200.so`` (the C ABI of ``include/ittai_b200.h``).

The reference compiles its kernels at construction time (reference ``src/ittai/qwen3/engine.py:141``);
here the library is prebuilt and only loaded.  A missing library is an error, never a fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libittai_b200.so")

ABI_VERSION = 1
MAX_BATCH = 8
STATUS_WORDS = 8
F_TEST_DROP_CTA = 2
PH_QKV, PH_ATTN, PH_OPROJ, PH_GU, PH_DOWN, PH_HEAD = range(6)

# every symbol include/ittai_b200.h declares
EXPORTS = (
    "ittai_version", "ittai_last_error", "ittai_device_check", "ittai_decode_status",
    "ittai_qwen3_decode_workspace_bytes", "ittai_qwen3_decode_launch", "ittai_qwen3_phase_launch",
    "ittai_qwen3_decode_launch_static",
    "ittai_gemm_bf16_launch", "ittai_gemm_chain_launch", "ittai_attention_launch", "ittai_rmsnorm_rows", "ittai_layernorm_rows", "ittai_row_stats",
    "ittai_qwen3_qk_rope_scatter", "ittai_siglip_im2col", "ittai_embed_rows", "ittai_qwen3_final_pool",
)
EPI_NONE, EPI_GELU, EPI_SWIGLU, EPI_QKROPE = range(4)


class IttaiError(RuntimeError):
    pass


class Qwen3Decode(C.Structure):
    """Mirror of ``struct IttaiQwen3Decode``."""
    _fields_ = [
        ("n_layers", C.c_int32), ("vocab", C.c_int32), ("kv_cap", C.c_int32), ("batch", C.c_int32),
        ("n_steps", C.c_int32), ("n_forced", C.c_int32), ("eps", C.c_float), ("write_logits", C.c_int32),
        ("flags", C.c_int32), ("spin_limit", C.c_int32),
        ("wqkv", C.c_void_p), ("wo", C.c_void_p), ("wgu", C.c_void_p), ("wd", C.c_void_p),
        ("ln1", C.c_void_p), ("ln2", C.c_void_p), ("qn", C.c_void_p), ("kn", C.c_void_p),
        ("fin_w", C.c_void_p), ("embed", C.c_void_p), ("rope", C.c_void_p),
        ("kcache", C.c_void_p), ("vcache", C.c_void_p), ("pos", C.c_void_p), ("next_id", C.c_void_p),
        ("forced", C.c_void_p), ("out_ids", C.c_void_p), ("logits", C.c_void_p),
        ("workspace", C.c_void_p), ("status", C.c_void_p), ("step_ns", C.c_void_p), ("phase_clk", C.c_void_p),
    ]


class QkRope(C.Structure):
    """Mirror of ``struct IttaiQkRope``."""
    _fields_ = [
        ("qn", C.c_void_p), ("kn", C.c_void_p), ("rope", C.c_void_p), ("pos", C.c_void_p), ("seq", C.c_void_p),
        ("slot", C.c_void_p), ("kcache_layer", C.c_void_p), ("vcache_layer", C.c_void_p), ("kv_cap", C.c_int32), ("eps", C.c_float),
    ]


class Gemm(C.Structure):
    """Mirror of ``struct IttaiGemm``."""
    _fields_ = [
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("epi", C.c_int32),
        ("ld_a", C.c_int32), ("ld_w", C.c_int32), ("ld_out", C.c_int32), ("ld_res", C.c_int32),
        ("a", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p),
        ("out", C.c_void_p), ("status", C.c_void_p), ("row_stats", C.c_void_p), ("col_sums", C.c_void_p),
        ("stats_out", C.c_void_p), ("stats_parts", C.c_int32), ("stats_eps", C.c_float), ("stats_k", C.c_int32), ("stats_rms", C.c_int32), ("qk_rope", C.POINTER(QkRope)),
    ]


class Attention(C.Structure):
    """Mirror of ``struct IttaiAttention``."""
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("q_row", C.c_int64), ("q_head", C.c_int64), ("k_row", C.c_int64), ("k_head", C.c_int64), ("k_seq", C.c_int64),
        ("v_row", C.c_int64), ("v_head", C.c_int64), ("v_seq", C.c_int64), ("o_row", C.c_int64), ("o_head", C.c_int64),
        ("seqs", C.c_void_p),
        ("n_seqs", C.c_int32), ("n_heads", C.c_int32), ("group", C.c_int32), ("head_dim", C.c_int32),
        ("causal", C.c_int32), ("max_q_len", C.c_int32), ("max_kv_len", C.c_int32), ("q_rows_total", C.c_int32),
        ("kv_rows_total", C.c_int32), ("reserved0", C.c_int32), ("status", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; raise if it is missing or of another ABI version."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise IttaiError(f"{LIB_PATH} is missing: build it with `python -m ittai_b200.build` (there is no fallback path)")
    L = C.CDLL(LIB_PATH)
    L.ittai_version.restype = C.c_int
    L.ittai_last_error.restype = C.c_char_p
    L.ittai_device_check.argtypes = [C.c_int, C.POINTER(C.c_int)]
    L.ittai_decode_status.argtypes = [C.POINTER(C.c_uint32), C.c_char_p, C.c_size_t]
    L.ittai_qwen3_decode_workspace_bytes.argtypes = [C.c_int, C.POINTER(C.c_size_t)]
    L.ittai_qwen3_decode_launch.argtypes = [C.POINTER(Qwen3Decode), C.c_void_p]
    L.ittai_qwen3_phase_launch.argtypes = [C.POINTER(Qwen3Decode), C.c_int, C.c_int, C.c_void_p]
    L.ittai_qwen3_decode_launch_static.argtypes = [C.POINTER(Qwen3Decode), C.c_void_p]
    L.ittai_gemm_bf16_launch.argtypes = [C.POINTER(Gemm), C.c_void_p]
    L.ittai_gemm_chain_launch.argtypes = [C.POINTER(Gemm), C.c_int32, C.c_void_p, C.c_void_p]
    L.ittai_attention_launch.argtypes = [C.POINTER(Attention), C.c_void_p]
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    L.ittai_rmsnorm_rows.argtypes = [vp, i32, vp, vp, i32, i32, f32, vp]
    L.ittai_layernorm_rows.argtypes = [vp, i32, vp, vp, vp, i32, i32, i32, f32, vp]
    L.ittai_row_stats.argtypes = [vp, i32, vp, i32, i32, f32, vp]
    L.ittai_qwen3_qk_rope_scatter.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, vp]
    L.ittai_siglip_im2col.argtypes = [vp, vp, i32, i32, i32, i32, i32, vp]
    L.ittai_embed_rows.argtypes = [vp, vp, vp, i32, i32, vp]
    L.ittai_qwen3_final_pool.argtypes = [vp, vp, vp, vp, i32, f32, vp]
    if L.ittai_version() != ABI_VERSION:
        raise IttaiError(f"library ABI {L.ittai_version()} != binding ABI {ABI_VERSION}; rebuild")
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != 0:
        raise IttaiError(f"ittai_b200 call failed ({rc}): {lib().ittai_last_error().decode()}")


def decode_status(words) -> None:
    """Raise if a host copy of the device status words reports a failed wait."""
    arr = (C.c_uint32 * STATUS_WORDS)(*[int(w) & 0xFFFFFFFF for w in words])
    msg = C.create_string_buffer(256)
    if lib().ittai_decode_status(arr, msg, 256) != 0:
        raise IttaiError(msg.value.decode())
