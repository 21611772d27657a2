"""The C-ABI library loads without a GPU and exports exactly what include/mtb200.h declares."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "mtb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mtb200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from minitensor_b200 import build, _lib
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    from minitensor_b200 import _lib
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in mtb200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header disagree"


def test_version_and_error_string(lib):
    assert lib.mtb200_version() == 100
    assert isinstance(lib.mtb200_last_error(), bytes)


def test_create_fails_cleanly_without_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    h = ctypes.c_void_p()
    rc = lib.mtb200_create(0, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert b"CUDA" in lib.mtb200_last_error() or b"device" in lib.mtb200_last_error()


def test_null_handle_is_rejected_not_dereferenced(lib):
    assert lib.mtb200_sync(None) == 1
    assert lib.mtb200_colsum(None, 0, 1, 1, None, None) == 1
    assert b"null handle" in lib.mtb200_last_error()


def test_python_layer_has_no_fallback():
    """Without a device the operator layer must raise, never compute on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from minitensor_b200.backend import Backend
    with pytest.raises(RuntimeError):
        Backend(0)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "minitensor_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src and "liboracle" not in src, f
