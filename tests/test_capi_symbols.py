"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""

import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "mfqb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mfqb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from tyloquant_b200 import _capi
    lib = ctypes.CDLL(_capi.LIB_PATH)
    names = _declared()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # and the binding covers them all
    unbound = [n for n in names if n not in _capi._SIGNATURES]
    assert not unbound, unbound
    assert lib.mfqb_version() >= 100
