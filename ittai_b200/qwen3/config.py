"""Qwen3-0.6B geometry and op vocabulary, under the names the reference exports
(reference ``src/ittai/qwen3/config.py:1-20``; its benchmark imports ``D, DQ, DQKV, DGU, FF, L``).

``VOCAB`` is the 151936-row table of Qwen3-0.6B; the reference's constant (151669, the embedding
checkpoint's tokenizer size) is never read by its code, the table height always comes from the weights.
"""
D, NH, NKV, HD, FF, L, VOCAB, EPS, THETA = 1024, 16, 8, 128, 3072, 28, 151936, 1e-6, 1e6
DQ, DKV = NH * HD, NKV * HD
DQKV, DGU = DQ + 2 * DKV, 2 * FF
K_OFF, V_OFF = DQ, DQ + DKV
G = NH // NKV
LOG2E = 1.4426950408889634
SCALE_LOG2 = HD ** -0.5 * LOG2E

# decode phases in execution order (ids of include/ittai_b200.h: ITTAI_PH_*)
PH_QKV, PH_ATTN, PH_OPROJ, PH_GU, PH_DOWN, PH_HEAD = range(6)
PHASE_NAMES = ("qkv", "attn", "oproj", "gu", "down", "head")


def decode_bytes_per_token(kv_len: int, n_layers: int = L, vocab: int = VOCAB) -> int:
    """Algorithmic HBM bytes one batch-1 decoded token must move at cache length ``kv_len``:
    every weight once (tied lm_head included), the whole KV cache once, the appended K/V row, one embedding row."""
    layer = 2 * (DQKV * D + D * DQ + DGU * D + D * FF)
    gains = 2 * (n_layers * (2 * D + 2 * HD) + D)
    weights = n_layers * layer + 2 * vocab * D + gains
    kv_row = n_layers * 2 * NKV * HD * 2
    return weights + kv_row * kv_len + kv_row + 2 * D

# The op table of the prefill task list, under the reference's names (reference ``src/ittai/qwen3/config.py:8-20``):
# op ids, dependency-flag slots, words per task record, rows per GEMM block / attention query block, and for every GEMM
# its width N, depth K, the slot it waits on, the slot it arrives on (``dl`` layers further), the norm statistics it
# consumes / produces and its epilogue kind.
OP_QKV, OP_OPROJ, OP_GU, OP_DOWN, OP_EMB, OP_ATTN, OP_FINAL = range(7)
NGEMM = 4
SLOT_X, SLOT_QKV, SLOT_ATTN, SLOT_XMID, SLOT_H, SLOT_SEQ = range(6)
NSLOT = 5
LN1, LN2 = 0, 1
TW = 8
BM, QB = 128, 64
SPEC = {
    OP_QKV: {"N": DQKV, "K": D, "dep": SLOT_X, "out": SLOT_QKV, "dl": 0, "s_in": LN1, "s_out": None, "kind": "qkv"},
    OP_OPROJ: {"N": D, "K": DQ, "dep": SLOT_ATTN, "out": SLOT_XMID, "dl": 0, "s_in": None, "s_out": LN2, "kind": "res"},
    OP_GU: {"N": DGU, "K": D, "dep": SLOT_XMID, "out": SLOT_H, "dl": 0, "s_in": LN2, "s_out": None, "kind": "gu"},
    OP_DOWN: {"N": D, "K": FF, "dep": SLOT_H, "out": SLOT_X, "dl": 1, "s_in": None, "s_out": LN1, "kind": "res"},
}
# The reference searches these tile / stage grids per GPU (``config.py:22-27``); there is one sm_100a kernel set here, so
# the table only names it.  Kept because callers import the name.
CONFIGS = {"sm100": [{"tile_m": 256, "tile_n": 256, "stages": 5, "cta_pair": True}]}
