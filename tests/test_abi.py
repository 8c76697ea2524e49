"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(mb[a-z]?_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    import mace_b200
    from mace_b200 import capi
    lib = mace_b200.lib()
    decl = declared_symbols()
    assert len(decl) >= 20
    for name in sorted(decl):
        assert hasattr(lib, name), "library does not export %s" % name
        assert name in capi.PROTOTYPES, "no ctypes prototype for %s" % name
    for name in capi.PROTOTYPES:
        assert name in decl, "%s is bound but not declared in include/" % name


def test_no_cpu_fallback_without_a_device():
    """mb_init must fail (not fall back) when there is no CUDA device."""
    import mace_b200
    lib = mace_b200.lib()
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    h = ctypes.c_void_p()
    assert lib.mb_init(0, ctypes.byref(h)) == 4  # MACE_RUNTIME_ERROR
    assert not h.value


def test_product_does_not_import_the_oracle():
    """Nothing under mace_b200/ may reference oracle/ (the oracle is test infrastructure)."""
    pkg = os.path.join(ROOT, "mace_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cc", ".h", ".cpp")) or fn == "Makefile":
                text = open(os.path.join(dirpath, fn), errors="ignore").read()
                assert "pyoracle" not in text and "oracle/" not in text and "liboracle" not in text, \
                    "%s references the oracle" % os.path.join(dirpath, fn)
