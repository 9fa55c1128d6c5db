"""``ittai.siglip.kernel``: ``Siglip2Embedder``, ``Engine`` and ``fold_ln`` of the reference module
(``src/ittai/siglip/kernel.py:523-723``), served by ``ittai_b200.siglip.kernel``."""
from ittai_b200.siglip.kernel import *  # noqa: F401,F403
from ittai_b200.siglip.kernel import Engine, Siglip2Embedder  # noqa: F401
