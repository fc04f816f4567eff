"""CPU-side checks of the drop-in boundary: the library loads and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "puter_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(cuda_[a-z0-9_]+)\s*\(", text))
    for g in re.findall(r"PUTER_DECLARE_GATED\((\w+)\)", text):
        if g != "name":
            names.add(f"cuda_dispatch_{g}")
            names.add(f"cuda_dispatch_{g}_packed")
    names.discard("cuda_dispatch_")
    return sorted(n for n in names if not n.endswith("_"))


@pytest.fixture(scope="module")
def lib():
    from puter_b200.csrc import build as b

    return ctypes.CDLL(b.build())


def test_every_declared_symbol_is_exported(lib):
    declared = _declared_symbols()
    assert len(declared) > 40
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_matches_header():
    from puter_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    _lib.load()


def test_status_helpers_need_no_gpu():
    from puter_b200 import _lib

    lib = _lib.load()
    st = _lib.CUDAStatus()
    lib.cuda_status_set(ctypes.byref(st), -6, b"unknown dtype")
    assert st.code == -6 and st.message == b"unknown dtype"
    lib.cuda_status_clear(ctypes.byref(st))
    assert st.code == 0 and st.message == b""


def test_no_device_fails_loudly_without_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import puter_b200

    with pytest.raises(puter_b200.DeviceError) as e:
        puter_b200.Device()
    assert e.value.code == -1 and "no CPU fallback" in e.value.message


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "puter_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src and "puter_oracle" not in src, f
