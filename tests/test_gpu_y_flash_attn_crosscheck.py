"""Secondary cross-check against the third-party library the reference calls for attention
(flash_attn, infer/ops/attention.py:3,110-121), when that library runs on this GPU.  The
primary checker is the CPU oracle; these tests skip if flash_attn cannot be used."""
import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close, to_dev
from infer_b200 import ops, workloads

pytestmark = pytest.mark.gpu


def test_flash_attn_cross_check_if_available(monkeypatch):
    """Secondary check against the library the reference itself calls
    (flash_attn_with_kvcache, infer/ops/attention.py:118-120) when it runs on this GPU."""
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as e:                              # pragma: no cover
        pytest.skip(f"flash_attn not importable: {e}")
    w = workloads.config0()
    d = to_dev(w)
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    got = ops.paged_attn_decode(d["q"], d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale)
    try:
        ref = flash_attn_with_kvcache(d["q"].unsqueeze(1), d["k_cache"], d["v_cache"], cache_seqlens=d["context_lens"],
                                      block_table=d["block_tables"].clamp_min(0), softmax_scale=w.scale, causal=True)
        torch.cuda.synchronize()
    except Exception as e:                              # pragma: no cover
        pytest.skip(f"flash_attn does not run on this GPU: {type(e).__name__}: {str(e)[:120]}")
    assert_close(got, ref.squeeze(1), ATOL_BF16, RTOL_BF16, "vs flash_attn_with_kvcache")


def test_flash_attn_varlen_cross_check_if_available():
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception as e:                              # pragma: no cover
        pytest.skip(f"flash_attn not importable: {e}")
    w = workloads.config2(n_seqs=3, max_prefix=600, chunk=200)
    d = to_dev(w)
    cu_q, cu_k = (t.cuda() for t in w.cu_seqlens())
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    got = ops.paged_attn_prefill(d["q"], d["k_cache"], d["v_cache"], cu_q, cu_k, max(w.new_lens), max(w.context_lens),
                                 w.scale, d["block_tables"])
    try:
        ref = flash_attn_varlen_func(d["q"], d["k_cache"], d["v_cache"], max_seqlen_q=max(w.new_lens), cu_seqlens_q=cu_q,
                                     max_seqlen_k=max(w.context_lens), cu_seqlens_k=cu_k, softmax_scale=w.scale,
                                     causal=True, block_table=d["block_tables"].clamp_min(0))
        torch.cuda.synchronize()
    except Exception as e:                              # pragma: no cover
        pytest.skip(f"flash_attn does not run on this GPU: {type(e).__name__}: {str(e)[:120]}")
    assert_close(got, ref, ATOL_BF16, RTOL_BF16, "vs flash_attn_varlen_func")
