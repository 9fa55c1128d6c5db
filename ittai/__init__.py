"""Import name of the reference library (``teraflop-ai/ittai``) over the B200 build: ``from ittai.qwen3 import ...`` and
``from ittai.siglip.kernel import ...`` resolve to ``ittai_b200``, so the reference's scripts run with their import lines
unchanged (reference ``benchmarks/qwen3.py:4``, ``benchmarks/siglip.py:5``).  Re-exports only; no code lives here."""
from ittai_b200 import __version__  # noqa: F401


def main() -> None:
    """Console entry point of the reference package (``src/ittai/__init__.py:1-2``)."""
    print("ittai on B200 (sm_100a): import ittai.qwen3 or ittai.siglip.kernel")
