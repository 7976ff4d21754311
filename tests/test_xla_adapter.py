"""CPU checks of the XLA boundary sources.  JAX and its FFI headers are not installed where this suite
runs, so the adapter cannot be built for real; what can be checked is that it is valid C++ whose handler
signatures match their bindings (type-checked against tests/stubs/xla/ffi/api/ffi.h, a stand-in that
spells the part of the FFI API the adapter uses), that it exports every symbol jaxrwkv registers, and
that the JAX-side modules at least compile and name targets the adapter defines."""
import os
import py_compile
import re
import shutil
import subprocess

import pytest

from jaxrwkv_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ADAPTER = os.path.join(ROOT, "jaxrwkv_b200", "csrc", "xla_ffi_adapter.cc")
XLA_DIR = os.path.join(ROOT, "jaxrwkv_b200", "xla")


def handler_symbols():
    return set(re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\((\w+),", open(ADAPTER).read()))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_adapter_type_checks_against_the_ffi_stand_in():
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    subprocess.check_call(["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-I", os.path.join(ROOT, "tests", "stubs"),
                           "-I", cuda_inc, ADAPTER])


def test_adapter_defines_the_handlers_jaxrwkv_registers():
    syms = handler_symbols()
    for name in ("WKV7FwdF32", "WKV7FwdBF16", "WKV7BwdF32", "WKV7BwdBF16",      # src/jaxrwkv/rwkv7.py:461-465
                 "WKV4FwdF32", "WKV4FwdBF16", "WKV4BwdF32", "WKV4BwdBF16"):     # src/jaxrwkv/rwkv4.py:396-400
        assert name in syms


def test_jax_modules_compile_and_name_existing_handlers():
    for fn in os.listdir(XLA_DIR):
        if fn.endswith(".py"):
            py_compile.compile(os.path.join(XLA_DIR, fn), doraise=True)
    text = open(os.path.join(XLA_DIR, "_ffi.py")).read()
    stems = set(re.findall(r'f"(\w+)\{_sym\}"', text))
    assert stems, "no handler names found in _ffi.py"
    syms = handler_symbols()
    for stem in stems:
        assert stem + "F32" in syms and stem + "BF16" in syms, stem


def test_adapter_build_is_skipped_cleanly_without_jax():
    if build.xla_ffi_include_dir() is None:
        assert build.build_xla_adapter() is None
