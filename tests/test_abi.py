"""The C-ABI library loads and exports every symbol the public header declares (no compute, no GPU)."""
import ctypes
import os
import re

from ittai_b200 import _C, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for f in os.listdir(os.path.join(ROOT, "include")):
        if f.endswith(".h"):
            src = open(os.path.join(ROOT, "include", f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names += re.findall(r"^\s*(?:const\s+)?(?:int|char\s*\*|void|size_t)\s*\*?\s*(ittai_\w+)\s*\(", src, flags=re.M)
    return sorted(set(names))


def test_header_and_binding_agree():
    assert _declared() == sorted(_C.EXPORTS)


def test_library_exports_every_declared_symbol():
    build.build()
    lib = ctypes.CDLL(_C.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), name
    assert _C.lib().ittai_version() == _C.ABI_VERSION


def test_argument_errors_need_no_gpu():
    L = _C.lib()
    n = ctypes.c_size_t()
    assert L.ittai_qwen3_decode_workspace_bytes(1, ctypes.byref(n)) == 0 and n.value > 0
    assert L.ittai_qwen3_decode_workspace_bytes(9, ctypes.byref(n)) == -1
    assert b"batch" in L.ittai_last_error()
    p = _C.Qwen3Decode()
    p.batch = 3
    assert L.ittai_qwen3_decode_launch(ctypes.byref(p), None) == -1
    assert L.ittai_qwen3_phase_launch(ctypes.byref(p), 9, 0, None) == -1


def test_status_decoding():
    _C.decode_status([0] * 8)
    try:
        _C.decode_status([1, 5, 7, 100, 148, 0, 0, 0])
        raise AssertionError("expected IttaiError")
    except _C.IttaiError as e:
        assert "barrier" in str(e) and "b=7" in str(e)
