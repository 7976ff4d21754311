"""JAX / XLA side of the operators: the modules a jaxrwkv maintainer drops in for the FFI glue of
``src/jaxrwkv/rwkv7.py:349-473`` and ``src/jaxrwkv/rwkv4.py:305-406``.

Importing this package needs ``jax`` (and, for the ``CudaRWKV`` classes, ``jaxrwkv`` itself); the rest
of ``jaxrwkv_b200`` does not.  The handlers come from ``lib/libb200wkv_xla.so``, which
``python -m jaxrwkv_b200.build`` produces from ``csrc/xla_ffi_adapter.cc`` when the XLA FFI headers
are installed (``jax.ffi.include_dir()``).

    from jaxrwkv_b200.xla import rwkv7      # rwkv7.CudaRWKV, rwkv7.wkv7_cuda
"""
