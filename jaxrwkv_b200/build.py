"""Build libb200wkv.so in-tree with nvcc for sm_100a:  python -m jaxrwkv_b200.build [--force] [-v]

Every ``csrc/*.cu`` is compiled to an object file of its own (in parallel, only when it or a header
is newer than the object) and the objects are linked into ``lib/libb200wkv.so``.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
OUT = os.path.join(LIBDIR, "libb200wkv.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def _obj(src):
    return os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(p) > t for p in deps)


def needs_build():
    return _stale(OUT, sources() + headers())


def build(force=False, verbose=False):
    if not force and not needs_build():
        return OUT
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    hdrs = headers()
    todo = [s for s in sources() if force or _stale(_obj(s), [s] + hdrs)]

    def compile_one(src):
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", _obj(src), src]
        print(" ".join(cmd), file=sys.stderr)
        subprocess.check_call(cmd)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(compile_one, todo))
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", OUT] + [_obj(s) for s in sources()]
    print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)
    return OUT


XLA_SRC = os.path.join(CSRC, "xla_ffi_adapter.cc")
XLA_OUT = os.path.join(LIBDIR, "libb200wkv_xla.so")


def xla_ffi_include_dir():
    """Directory of the XLA FFI headers (xla/ffi/api/ffi.h), or None where JAX is not installed."""
    try:
        import jax.ffi
        d = jax.ffi.include_dir()
    except Exception:
        return None
    return d if os.path.exists(os.path.join(d, "xla", "ffi", "api", "ffi.h")) else None


def build_xla_adapter(force=False):
    """Compile csrc/xla_ffi_adapter.cc into lib/libb200wkv_xla.so (the handlers jax.ffi registers).  Returns
    the path, or None when the XLA FFI headers are not installed - the C ABI library does not need them."""
    inc = xla_ffi_include_dir()
    if inc is None:
        return None
    build()
    if not force and not _stale(XLA_OUT, [XLA_SRC, OUT] + headers()):
        return XLA_OUT
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", "-shared", "-fPIC", "-I", inc, "-I", cuda_inc, "-o", XLA_OUT,
           XLA_SRC, "-L", LIBDIR, "-lb200wkv", "-Wl,-rpath,$ORIGIN"]
    print(" ".join(cmd), file=sys.stderr)
    subprocess.check_call(cmd)
    return XLA_OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    if build_xla_adapter(force="--force" in sys.argv) is None:
        print("XLA FFI headers not found (jax is not installed): libb200wkv_xla.so not built", file=sys.stderr)
