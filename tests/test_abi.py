"""CPU checks of the C-ABI library: it loads, exports every symbol the header declares, and
refuses to compute without a device (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "endia_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(endia_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    from endia_b200 import _lib
    syms = declared_symbols()
    assert len(syms) >= 30
    for s in syms:
        assert hasattr(_lib.lib, s), "library does not export %s" % s
        assert s in _lib.SIGNATURES, "python binding lacks a prototype for %s" % s
    for s in _lib.SIGNATURES:
        assert s in syms, "binding declares %s which the header does not" % s


def test_version_and_error_string():
    from endia_b200 import _lib
    assert _lib.lib.endia_b200_version() == 1000
    assert isinstance(_lib.lib.endia_b200_last_error(), bytes)


def test_struct_layout_matches_header():
    from endia_b200 import _lib
    assert C.sizeof(_lib.Tensor) == 8 + 64 + 64 + 8 + 4 + 4
    assert _lib.Tensor.offset.offset == 136
    assert C.sizeof(_lib.Epilogue) == 96


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from endia_b200 import _lib
    import endia_b200 as nd
    with pytest.raises(_lib.EndiaError) as ei:
        nd.Array([2, 3])
    assert ei.value.status == _lib.ENODEV
    # the raw entry points refuse as well
    assert _lib.lib.endia_b200_init(0) == _lib.ENODEV
    assert _lib.lib.endia_b200_fill(None, 4, 0, 1.0, 0.0, None) == _lib.ENODEV
    assert b"no CPU fallback" in _lib.lib.endia_b200_last_error()


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "endia_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, "%s mentions the oracle" % os.path.join(dirpath, f)
