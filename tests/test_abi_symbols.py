"""CPU: the C-ABI library builds, loads and exports every symbol include/tm_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if not fn.endswith(".h"):
            continue   # include/compat holds header shims that only call what tm_b200.h declares
        src = open(os.path.join(ROOT, "include", fn)).read()
        names |= set(re.findall(r"TM_API\s+[\w\s\*]+?\b(tm_\w+)\s*\(", src))
    return names


def test_library_builds_and_exports_all_declared_symbols():
    from lmdeploy_b200 import build
    path = build.build()
    lib = ctypes.CDLL(path)
    declared = _declared()
    assert len(declared) >= 10
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"


def test_python_binding_covers_header():
    from lmdeploy_b200 import lib as l
    assert set(l.SIGNATURES) == _declared()
    assert l.status_string(0) == "ok"
    assert l.lib.tm_gemm_s4_f16_workspace_bytes(4096, 1, 4096) > 0
    assert l.lib.tm_gemm_s4_f16_workspace_bytes(4096, 1, 100) == 0
