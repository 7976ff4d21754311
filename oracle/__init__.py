"""CPU restatement of the jaxrwkv WKV state recurrences (test infrastructure only).

This package is the *checker*: it is imported by the test-suite, by the smoke
entry point and by the CPU-baseline leg of the benchmark, and by nothing in the
shipped operator path.  Every function cites the jaxrwkv source lines it
restates (paths are relative to the jaxrwkv project root).

Pinning: jaxrwkv ships no golden vectors and JAX is not installable in the
build image, so the restatement is pinned against fixtures produced by
executing the reference's own ``inner_loop`` source (Base / Scan /
AssociativeScan classes of rwkv4/5/5_2/6/7) under a small NumPy stand-in for
the handful of ``jax`` / ``jax.numpy`` calls those functions make
(``tests/golden/make_golden.py``).  Parity against the external
``jaxrwkvkernel`` CUDA package that the reference's own ``CudaRWKV`` loads is
unpinned: that package is not part of the reference tree.
"""
from .wkv7 import (wkv7_base, wkv7_assoc, wkv7_base_batched, wkv7_assoc_batched,
                   wkv7_bwd, wkv7_bwd_batched, quirk_mask)
from .wkv6 import (wkv6_base, wkv6_assoc, wkv6_base_batched, wkv6_bwd, wkv6_bwd_batched)
from .wkv4 import (wkv4_base, wkv4_assoc, wkv4_base_batched)
from .scan import associative_scan
from .inputs import make_wkv7_inputs, make_wkv6_inputs, make_wkv4_inputs
