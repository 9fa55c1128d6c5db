"""ittai_b200: B200 (sm_100a) kernels behind the Python model API of the ittai megakernel library.

Python and PyTorch own weights, tensors and streams; all device work goes through the C-ABI shared
library ``libittai_b200.so`` declared in ``include/ittai_b200.h``.  There is no CPU or eager fallback:
importing an engine without the built library raises.
"""
__version__ = "0.1.0"
