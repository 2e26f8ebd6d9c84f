"""The device-side error path, exercised without faulting or hanging the GPU: the self-test entry
points run the product kernels with a producer that arms no copy and a wait limit of a few
thousand polls, so every bounded wait runs out within microseconds, the kernels set their status
word and return, and the host reads INFER_ERR_DEVICE exactly once.  The context stays usable: the
same call without the stall gives the right answer afterwards."""
import ctypes as C

import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close, to_dev
from infer_b200 import _lib, ops, selftest, workloads
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "e4m3"])
def test_decode_wait_runs_out_and_is_reported_once(fp8, monkeypatch):
    lib = _lib.load()
    monkeypatch.setattr(ops, "_CHECK", False)                 # the status word is read by hand below
    w = workloads.config1(batch=6, lo=300, hi=2000)
    d = to_dev(w)
    if fp8:
        kc = torch.zeros(w.num_blocks, 256, w.n_kv_heads, 128, dtype=torch.uint8, device="cuda")
        vc = torch.zeros_like(kc)
        ks = torch.zeros(w.num_blocks, w.n_kv_heads, device="cuda")
        vs = torch.zeros_like(ks)
        slots = torch.arange(w.num_blocks * 256, dtype=torch.int32, device="cuda")
        ops.store_kvcache(d["k_cache"].view(-1, w.n_kv_heads, 128), d["v_cache"].view(-1, w.n_kv_heads, 128), kc, vc,
                          slots, ks, vs)
        pools = dict(k_scale=ks, v_scale=vs)
    else:
        kc, vc, pools = d["k_cache"], d["v_cache"], {}
    pool = ops.pool_of(kc, vc, pools.get("k_scale"), pools.get("v_scale"))
    ws = torch.zeros(pool.decode_workspace_bytes(w.batch, w.n_q_heads), dtype=torch.uint8, device="cuda")
    good = ops.paged_attn_decode(d["q"], kc, vc, d["context_lens"], d["block_tables"], w.scale, workspace=ws, **pools)
    torch.cuda.synchronize()
    assert lib.infer_paged_decode_status(C.c_void_p(ws.data_ptr()), _stream()) == _lib.OK

    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    with selftest.variant(wait_limit=4096, stall_producer=1):
        ops.paged_attn_decode(d["q"], kc, vc, d["context_lens"], d["block_tables"], w.scale, workspace=ws, **pools)
    t1.record()
    torch.cuda.synchronize()                                   # returns: nothing hangs, nothing faults
    assert t0.elapsed_time(t1) < 1000.0                        # milliseconds, not the default second-long limit per wait
    assert lib.infer_paged_decode_status(C.c_void_p(ws.data_ptr()), _stream()) == _lib.ERR_DEVICE
    assert lib.infer_paged_decode_status(C.c_void_p(ws.data_ptr()), _stream()) == _lib.OK     # reported once, then cleared
    torch.cuda.synchronize()
    assert int(ws[:4096 + 64].view(torch.int32).abs().sum()) == 0      # status word and tickets are back at zero

    again = ops.paged_attn_decode(d["q"], kc, vc, d["context_lens"], d["block_tables"], w.scale, workspace=ws, **pools)
    torch.cuda.synchronize()
    assert torch.equal(again, good)


def test_poisoned_status_word_raises_in_the_python_shim(monkeypatch):
    """Host-side injection: the magic word is written into the scratch header from the host; with
    status checking on, the next call's check raises and clears it."""
    monkeypatch.setattr(ops, "_CHECK", True)
    w = workloads.config0()
    d = to_dev(w)
    pool = ops.pool_of(d["k_cache"], d["v_cache"])
    ws = torch.zeros(pool.decode_workspace_bytes(w.batch, w.n_q_heads), dtype=torch.uint8, device="cuda")
    args = (d["q"], d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale)
    ops.paged_attn_decode(*args, workspace=ws)
    ws[:4].copy_(torch.tensor([0x5AFE0003], dtype=torch.int32).view(torch.uint8))
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        ops.paged_attn_decode(*args, workspace=ws)
    got = ops.paged_attn_decode(*args, workspace=ws)          # cleared: fine again
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    want = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "after a cleared status word")


def test_prefill_wait_runs_out_and_is_reported_once(monkeypatch):
    lib = _lib.load()
    monkeypatch.setattr(ops, "_CHECK", False)
    w = workloads.config2(n_seqs=2, max_prefix=500, chunk=300)
    d = to_dev(w)
    cu_q, cu_k = (t.cuda() for t in w.cu_seqlens())
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    args = (d["q"], d["k_cache"], d["v_cache"], cu_q, cu_k, max(w.new_lens), max(w.context_lens), w.scale, d["block_tables"])
    good = ops.paged_attn_prefill(*args)
    torch.cuda.synchronize()
    assert lib.infer_prefill_status(_stream()) == _lib.OK
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    with selftest.variant(wait_limit=4096, stall_producer=1):
        ops.paged_attn_prefill(*args)
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 1000.0
    assert lib.infer_prefill_status(_stream()) == _lib.ERR_DEVICE
    assert lib.infer_prefill_status(_stream()) == _lib.OK
    again = ops.paged_attn_prefill(*args)                       # tensor memory was freed, the kernel runs again
    torch.cuda.synchronize()
    assert torch.equal(again, good)
