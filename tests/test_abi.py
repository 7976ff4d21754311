"""CPU tests of the boundary: the built library loads and exports exactly what the
header declares, and argument validation returns the documented status codes
(no kernel is launched: validation happens before any CUDA call)."""
import ctypes
import os
import re

import pytest

from jaxrwkv_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(b200wkv\w*)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported_and_bound(lib):
    decl = declared_symbols()
    assert decl, "no declarations found"
    for name in decl:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert decl == set(_lib.PROTOTYPES), (decl ^ set(_lib.PROTOTYPES))


def test_status_strings(lib):
    assert lib.b200wkv_strerror(0) == b"ok"
    for code in range(-8, 0):
        assert lib.b200wkv_strerror(code) not in (b"ok", b"unknown status")
    assert lib.b200wkv_abi_version() >= 2


def test_argument_validation_without_gpu(lib):
    one = ctypes.c_void_p(16)  # never dereferenced: validation fails first
    args = [one] * 9 + [one, one, None, 0, 0]
    assert lib.b200wkv7_fwd(None, 7, 1, 16, 1, 64, *args) == -1          # dtype
    assert lib.b200wkv7_fwd(None, 0, 1, 16, 1, 32, *args) == -2          # head size
    assert lib.b200wkv7_fwd(None, 0, 0, 16, 1, 64, *args) == -2          # B < 1
    assert lib.b200wkv7_fwd(None, 0, 1, 0, 1, 64, *args) == -2           # T < 1
    bad = [None] + [one] * 8 + [one, one, None, 0, 0]
    assert lib.b200wkv7_fwd(None, 0, 1, 16, 1, 64, *bad) == -3           # NULL operand
    small = [one] * 9 + [one, one, one, 8, 0]
    assert lib.b200wkv7_fwd(None, 0, 1, 16, 1, 64, *small) == -4         # residual too small
    bargs = [one] * 9 + [one, one, None, 0] + [one] * 7 + [0]
    assert lib.b200wkv7_bwd(None, 1, 1, 16, 1, 64, *bargs) == -3         # bwd needs the residual
    assert lib.b200wkv7_residual_bytes(1, 1, 16, 1, 64) > 0
    assert lib.b200wkv7_residual_bytes(1, 1, 16, 1, 63) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(_lib.B200WKVError, match="no CPU or PyTorch fallback"):
        _lib.load()
