"""infer_paged_decode_noalloc: the decode entry point for callers that cannot hand the library
any scratch memory - an engine whose KV pools already own all free device memory, or a host
runtime that reaches the C ABI through a thin shim and only holds borrowed device pointers.
Its scratch is a 2 MiB array inside the library's device image, shared by every call.

The test goes through the C ABI directly and compares with the regular entry point (which gets
a caller-provided workspace) on two calls in a row with different shapes, so the second call
runs on whatever the first one left in the shared array.  It is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close
from infer_b200 import _lib, ops, workloads

pytestmark = pytest.mark.gpu


def _noalloc(w, dev):
    """Append with the regular op, decode through infer_paged_decode_noalloc."""
    lib = _lib.load()
    kc, vc = w.k_cache.to(dev), w.v_cache.to(dev)
    q = w.q.to(dev)
    cl, bt = w.context_lens_tensor().to(dev), w.block_tables_tensor().to(dev)
    ops.store_kvcache(w.k.to(dev), w.v.to(dev), kc, vc, w.slot_mapping.to(dev))
    want = ops.paged_attn_decode(q, kc, vc, cl, bt, w.scale)
    pool = ops.pool_of(kc, vc)
    out = torch.zeros_like(q)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.infer_paged_decode_noalloc(pool.handle, C.c_void_p(out.data_ptr()), C.c_void_p(q.data_ptr()),
                                        C.c_void_p(cl.data_ptr()), C.c_void_p(bt.data_ptr()), bt.stride(0),
                                        w.batch, w.n_q_heads, w.scale, stream)
    assert rc == 0, lib.infer_strerror(rc).decode()
    torch.cuda.synchronize()
    # a NULL workspace asks for the status word of the built-in array: no bounded wait ran out
    assert lib.infer_paged_decode_status(None, stream) == 0
    return out, want


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    first = workloads.config1(batch=12, lo=200, hi=3000)     # long contexts: many split sequences
    got, want = _noalloc(first, dev)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "no-alloc decode, first call")
    second = workloads.config0()                             # other head counts, shorter contexts
    got, want = _noalloc(second, dev)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "no-alloc decode, second call on the used scratch")


def test_noalloc_e4m3_pool_fits_by_taking_fewer_heads_per_tile():
    """An e4m3 pool with 8 KV heads and 4 query heads each: the partial-result slots of four heads
    per tile (the default) need more than the built-in 2 MiB, so the entry point has to fall back
    to fewer heads per tile instead of refusing the call."""
    dev = torch.device("cuda", 0)
    lib = _lib.load()
    w = workloads.config1(batch=12, lo=200, hi=3000, device=dev)
    nb, hkv = w.num_blocks, w.n_kv_heads
    k8 = torch.zeros(nb, 256, hkv, 128, dtype=torch.uint8, device=dev)
    v8 = torch.zeros_like(k8)
    ks, vs = torch.zeros(nb, hkv, device=dev), torch.zeros(nb, hkv, device=dev)
    slots = torch.arange(nb * 256, dtype=torch.int32, device=dev)
    ops.store_kvcache(w.k_cache.view(-1, hkv, 128), w.v_cache.view(-1, hkv, 128), k8, v8, slots, ks, vs)
    cl, bt = w.context_lens_tensor().to(dev), w.block_tables_tensor().to(dev)
    want = ops.paged_attn_decode(w.q, k8, v8, cl, bt, w.scale, k_scale=ks, v_scale=vs)
    pool = ops.pool_of(k8, v8, ks, vs)
    out = torch.zeros_like(w.q)
    rc = lib.infer_paged_decode_noalloc(pool.handle, C.c_void_p(out.data_ptr()), C.c_void_p(w.q.data_ptr()),
                                        C.c_void_p(cl.data_ptr()), C.c_void_p(bt.data_ptr()), bt.stride(0),
                                        w.batch, w.n_q_heads, w.scale, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.infer_strerror(rc).decode()
    torch.cuda.synchronize()
    # same kernel with a different tile width: the same bytes in a different summation order
    assert_close(out, want, 2e-2, 1e-2, "no-alloc e4m3 decode vs regular entry point")


def test_noalloc_rejects_what_does_not_fit():
    dev = torch.device("cuda", 0)
    lib = _lib.load()
    kc = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16, device=dev)
    pool = ops.pool_of(kc, kc)
    batch = 2049                                             # beyond the 2048-row prefix table
    q = torch.zeros(batch, 16, 128, dtype=torch.bfloat16, device=dev)
    out = torch.full_like(q, 3.0)
    cl = torch.ones(batch, dtype=torch.int32, device=dev)
    bt = torch.zeros(batch, 1, dtype=torch.int32, device=dev)
    rc = lib.infer_paged_decode_noalloc(pool.handle, C.c_void_p(out.data_ptr()), C.c_void_p(q.data_ptr()),
                                        C.c_void_p(cl.data_ptr()), C.c_void_p(bt.data_ptr()), 1, batch, 16, 0.1, None)
    assert rc == _lib.ERR_TOO_LARGE
    assert b"built-in scratch" in lib.infer_strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 3.0).all())                         # nothing was launched
