"""The ctypes signatures in ksa_b200/ops/_lib.py must match the C prototypes of the kernel library."""
import ctypes
import glob
import os
import re

from ksa_b200.ops._lib import _SIGNATURES

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ksa_b200", "csrc")


def _kind_c(arg: str) -> str:
    if "*" in arg:
        return "P"
    if "long long" in arg:
        return "L"
    if "float" in arg:
        return "F"
    if "unsigned" in arg:
        return "U"
    return "I"


def _kind_py(t) -> str:
    return {ctypes.c_void_p: "P", ctypes.c_int: "I", ctypes.c_longlong: "L", ctypes.c_float: "F",
            ctypes.c_uint: "U"}[t]


def test_signatures_match_prototypes():
    src = "".join(open(f).read() for f in glob.glob(os.path.join(CSRC, "*.cu")))
    seen = 0
    for m in re.finditer(r"KSA_API int (ksa_\w+)\(([^)]*)\)\s*\{", src):
        name = m.group(1)
        if name not in _SIGNATURES:
            continue
        args = [a.strip() for a in m.group(2).split(",") if a.strip()]
        c_sig = "".join(_kind_c(a) for a in args)
        py_sig = "".join(_kind_py(t) for t in _SIGNATURES[name])
        assert c_sig == py_sig, f"{name}: C prototype {c_sig} != ctypes {py_sig}"
        seen += 1
    assert seen >= 15
