"""CPU-only checks of the C-ABI library: it loads, exports every symbol the
header declares, and fails loudly (never silently falls back) without a GPU."""
import ctypes as C
import os
import re

import pytest

import npeff_ref_b200
from npeff_ref_b200 import _lib
from npeff_ref_b200._lib import Params, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = ""
    for name in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if name.endswith(".h"):
            text += open(os.path.join(ROOT, "include", name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dnpeff_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 25
    handle = C.CDLL(_lib.lib_path())
    for name in names:
        assert hasattr(handle, name), name
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_abi_version():
    assert lib().dnpeff_abi_version() == 1


def test_bad_params_rejected_without_touching_a_device():
    h = C.c_void_p()
    p = Params(0, 1e-8, 1, 0.0, 0, 1, 0)
    assert lib().dnpeff_create(C.byref(p), 0, None, C.byref(h)) == -1
    assert b"rank" in lib().dnpeff_last_error()
    p = Params(4, 1e-8, 1, 0.0, 2, 2, 0)
    assert lib().dnpeff_create(C.byref(p), 0, None, C.byref(h)) == -1


def _no_gpu():
    import torch
    return not torch.cuda.is_available()


@pytest.mark.skipif(not _no_gpu(), reason="checks the behaviour on a machine without a GPU")
def test_no_cpu_fallback_without_gpu():
    with pytest.raises(npeff_ref_b200.DnpeffError) as ei:
        npeff_ref_b200.MuNmf(npeff_ref_b200.MuNmfParams(rank=4))
    assert ei.value.code == -2


def test_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "npeff_ref_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().lower(), f
