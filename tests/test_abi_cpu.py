"""CPU checks of the C-ABI boundary: the shared library loads without a GPU and exports every entry
point that include/*.h declares (no compute calls here)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared(header):
    src = open(os.path.join(ROOT, "include", header)).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(stafb?_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def lib():
    from alphanesgpu_b200 import build
    path = build.build()
    return ctypes.CDLL(path)


@pytest.mark.parametrize("header", ["stafb.h", "staf.h"])
def test_every_declared_symbol_is_exported(lib, header):
    names = _declared(header)
    assert len(names) >= 5
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_error_strings_and_argument_checks_without_gpu(lib):
    lib.stafb_strerror.restype = ctypes.c_char_p
    assert b"radial" in lib.stafb_strerror(1)
    assert b"angular" in lib.stafb_strerror(2)
    # invalid arguments are rejected before any CUDA call
    h = ctypes.c_void_p()
    assert lib.stafb_create(ctypes.byref(h), 7, ctypes.c_double(4.5), ctypes.c_double(2.25), ctypes.c_double(4.5),
                            60, 1770, 96, 1) == 5
    assert lib.stafb_create(ctypes.byref(h), 0, ctypes.c_double(4.5), ctypes.c_double(2.25), ctypes.c_double(5.0),
                            60, 1770, 96, 1) == 5  # angular cutoff larger than the radial one
    assert lib.stafb_init_force_radial(60) == 0 and lib.stafb_init_grad_force_tripl(1770) == 0
    assert lib.staf_compute(None, 1, 0, None, None, None, None, None, 0, None, None, None) == -1


def test_package_refuses_to_run_without_the_library(monkeypatch):
    import alphanesgpu_b200._lib as L
    monkeypatch.setattr(L, "_LIB", None)
    monkeypatch.setattr(L, "LIB_PATH", os.path.join(ROOT, "does_not_exist.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        L.lib()
