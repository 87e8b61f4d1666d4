"""CPU tests of the C-ABI boundary: the library builds, loads and exports every symbol the header declares."""
import ctypes as C
import os
import re

from ruai_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ruai_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ruai_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _lib.load()
    declared = header_symbols()
    assert declared, "no declarations found in include/ruai_b200.h"
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in the header but not exported"
    assert set(declared) == set(_lib.symbols()), set(declared) ^ set(_lib.symbols())


def test_version_and_device_probe_do_not_need_a_gpu():
    L = _lib.load()
    assert b"sm_100a" in L.ruai_version()
    assert L.ruai_device_count() >= 0


def test_no_cpu_fallback():
    """Without a device the library refuses to create a context and says why."""
    L = _lib.load()
    if L.ruai_device_count() > 0:
        return
    h = C.c_void_p()
    rc = L.ruai_ctx_create(0, None, C.byref(h))
    assert rc == _lib.ERR_CUDA and not h.value
    assert b"no CPU fallback" in L.ruai_last_error(None)


def test_product_does_not_import_the_oracle():
    """The checker is test infrastructure: nothing under ruai_b200/ may reference it."""
    pkg = os.path.join(ROOT, "ruai_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "import oracle" not in text and "from oracle" not in text and "oracle/" not in text, f
