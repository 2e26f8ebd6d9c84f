"""Routes the attention ops to the library's diagnostic entry points (include/infer_b200_selftest.h).

Only the test suite uses this module.  Inside ``with variant(...)`` the ops of ``infer_b200.ops``
keep their signatures and checks but launch

* the decode kernels with a chosen number of kv heads per tile,
* the mma.sync cross-check kernel for prefill (``prefill_kernel=1``),
* or any of the product kernels with a short wait limit and a producer that arms no copy
  (``stall_producer=1``), which makes every bounded wait run out so that the status-word path
  can be checked without faulting or hanging the GPU.
"""
from __future__ import annotations

from contextlib import contextmanager

from . import ops


@contextmanager
def variant(decode_heads_per_tile: int = 0, prefill_kernel: int = 0, wait_limit: int = 0, stall_producer: int = 0):
    saved = ops._call_decode, ops._call_prefill, ops._call_dense

    def decode(lib, *args):
        return lib.infer_selftest_paged_decode(*args, decode_heads_per_tile, wait_limit, stall_producer)

    def prefill(lib, *args):
        return lib.infer_selftest_paged_prefill(*args, prefill_kernel, wait_limit, stall_producer)

    def dense(lib, *args):
        return lib.infer_selftest_flash_attn_prefill(*args, prefill_kernel)

    ops._call_decode, ops._call_prefill, ops._call_dense = decode, prefill, dense
    try:
        yield
    finally:
        ops._call_decode, ops._call_prefill, ops._call_dense = saved
