"""The reference's import name (CPU): its two benchmark scripts start with these import lines (reference
``benchmarks/qwen3.py:4`` and ``benchmarks/siglip.py:5``); they have to resolve against this repository unchanged."""
import subprocess
import sys
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_IMPORT_LINES = (
    "from ittai.qwen3 import Qwen3Embedder, D, DQ, DQKV, DGU, FF, L",
    "from ittai.siglip.kernel import Siglip2Embedder",
)


def test_reference_import_lines_resolve():
    ns = {}
    for line in REFERENCE_IMPORT_LINES:
        exec(line, ns)
    import ittai_b200.qwen3 as q
    import ittai_b200.siglip.kernel as k
    assert ns["Qwen3Embedder"] is q.Qwen3Embedder and ns["Siglip2Embedder"] is k.Siglip2Embedder
    assert (ns["D"], ns["DQ"], ns["DQKV"], ns["DGU"], ns["FF"], ns["L"]) == (1024, 2048, 4096, 6144, 3072, 28)


def test_star_exports_of_the_reference_package():
    """``src/ittai/qwen3/__init__.py:1-6`` star-exports its constants and names Engine, build_tasks, rope_perm."""
    import ittai.qwen3 as iq
    for name in ("SPEC", "CONFIGS", "SLOT_X", "SLOT_QKV", "SLOT_ATTN", "SLOT_XMID", "SLOT_H", "SLOT_SEQ", "NSLOT", "NGEMM", "TW",
                 "BM", "QB", "LN1", "LN2", "OP_QKV", "OP_FINAL", "K_OFF", "V_OFF", "G", "SCALE_LOG2", "Engine", "build_tasks",
                 "rope_perm", "Qwen3Embedder"):
        assert hasattr(iq, name), name
    assert iq.SPEC[iq.OP_DOWN]["dl"] == 1 and iq.SPEC[iq.OP_QKV]["kind"] == "qkv"
    import ittai.siglip.kernel as ik
    assert callable(ik.fold_ln) and callable(ik.gemm_tasks) and ik.gemm_tasks(0, 1, 3, 2, 2) == [
        (0, 1, 0, 0), (0, 1, 1, 0), (0, 1, 0, 1), (0, 1, 1, 1), (0, 1, 2, 0), (0, 1, 2, 1)]


def test_import_in_a_fresh_interpreter():
    code = "; ".join(REFERENCE_IMPORT_LINES) + "; import ittai; ittai.main()"
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
