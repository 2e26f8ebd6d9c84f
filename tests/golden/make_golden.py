"""Generates the golden fixtures in this directory by running the REFERENCE's own code on CPU.

Usage (only where the reference checkout exists; the fixtures are committed):

    python tests/golden/make_golden.py /path/to/Graylatzhou-Infer

What is executed from the reference tree, unmodified:
  * infer/ops/attention.py  store_kvcache / store_kvcache_kernel, under TRITON_INTERPRET=1
    (the Triton interpreter runs the kernel on CPU tensors);
  * infer/engine/block_mannager.py BlockManager, infer/engine/sequence.py Sequence;
  * infer/engine/model_runner.py ModelRunner.prepare_block_tables / prepare_prefill /
    prepare_decode, called unbound on a stand-in object that only carries ``block_size``.
The reference's compiled extension (``infer_ops``) cannot be built without a GPU toolchain
setup, so the module name is stubbed; ``Tensor.cuda`` and ``pin_memory=`` are made no-ops.
The attention expectations use ``torch.nn.functional.scaled_dot_product_attention``, the
expected-value function of the reference's attention test (test/op.py:278-281).

Large tensors are not stored: inputs are regenerated from the seeds recorded here and
guarded by SHA-256 digests; outputs are stored in full when small, as digests otherwise.
"""
import hashlib
import json
import os
import sys
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def bits(t: torch.Tensor):
    return t.contiguous().view(torch.int16).numpy()


def import_reference(root: str):
    sys.path.insert(0, root)
    stub = types.ModuleType("infer_ops")
    for name in ["flash_attn_prefill", "add", "rms_norm", "matmul", "embedding", "rope", "silu", "softmax",
                 "rms_norm_vllm", "rms_norm_fused", "silu_and_mul"]:
        setattr(stub, name, None)
    sys.modules["infer_ops"] = stub
    torch.Tensor.cuda = lambda self, *a, **k: self
    real_tensor = torch.tensor

    def tensor(*a, **k):
        k.pop("pin_memory", None)
        return real_tensor(*a, **k)

    torch.tensor = tensor
    from infer.engine.block_mannager import BlockManager
    from infer.engine.model_runner import ModelRunner
    from infer.engine.sequence import Sequence
    from infer.ops.attention import store_kvcache
    from infer.sampling_params import SamplingParams
    from infer.context import get_context
    return BlockManager, ModelRunner, Sequence, SamplingParams, store_kvcache, get_context


def golden_allocator(BlockManager, ModelRunner, Sequence, SamplingParams, get_context):
    """A scripted engine life: shared prefixes, growth across page boundaries, frees and
    page re-use.  Records page lists, cache hits, reference counts and the step metadata the
    reference builds from them."""
    rng = np.random.default_rng(77)
    sp = SamplingParams()
    mgr = BlockManager(24, 256)
    runner = types.SimpleNamespace(block_size=256)
    runner.prepare_block_tables = lambda seqs: ModelRunner.prepare_block_tables(runner, seqs)
    common = rng.integers(0, 1000, size=600).tolist()
    prompts = [
        common + rng.integers(0, 1000, size=100).tolist(),     # 700 tokens
        common[:512] + rng.integers(0, 1000, size=255).tolist(),  # shares 2 pages, ends 1 short of a page
        rng.integers(0, 1000, size=256).tolist(),                 # exactly one page
        common + rng.integers(0, 1000, size=424).tolist(),     # 1024 tokens, shares 2 pages
    ]
    events = []
    seqs = []

    def snap(tag, extra=None):
        events.append({
            "tag": tag,
            "tables": [list(s.block_table) for s in seqs],
            "cached": [s.num_cached_tokens for s in seqs],
            "lens": [len(s) for s in seqs],
            "ref_counts": [b.ref_count for b in mgr.blocks],
            "free": list(mgr.free_block_ids),
            **(extra or {}),
        })

    def ctx_dump():
        c = get_context()
        out = {}
        for k in ("cu_seqlens_q", "cu_seqlens_k", "slot_mapping", "context_lens", "block_tables"):
            v = getattr(c, k)
            out[k] = None if v is None else v.tolist()
        out["max_seqlen_q"], out["max_seqlen_k"], out["is_prefill"] = c.max_seqlen_q, c.max_seqlen_k, c.is_prefill
        return out

    for p in prompts:
        s = Sequence(p, sp)
        mgr.allocate(s)
        seqs.append(s)
    ModelRunner.prepare_prefill(runner, seqs)
    snap("prefill", {"context": ctx_dump()})
    # decode steps: sequence 1 crosses a page boundary on step 2, sequence 2 on step 1
    new_tokens = rng.integers(0, 1000, size=(3, len(seqs))).tolist()
    for step in range(3):
        for s, tok in zip(seqs, new_tokens[step]):
            s.append_token(int(tok))
            mgr.may_append(s)
        ModelRunner.prepare_decode(runner, seqs)
        snap(f"decode{step}", {"context": ctx_dump()})
    # free two sequences, then admit a new one that revives a sealed page by digest
    mgr.deallocate(seqs[0])
    mgr.deallocate(seqs[2])
    snap("freed")
    late = Sequence(common + [5, 6, 7], sp)
    mgr.allocate(late)
    seqs.append(late)
    ModelRunner.prepare_prefill(runner, [late])
    snap("late_prefill", {"context": ctx_dump()})
    return {"num_blocks": 24, "block_size": 256, "prompts": prompts, "new_tokens": new_tokens,
            "late_prompt": common + [5, 6, 7], "events": events}


def golden_append(store_kvcache):
    """The reference's store kernel on a strided key/value (column slices of a fused qkv
    row, as the model passes them) into zero pools."""
    g = torch.Generator().manual_seed(4242)
    n, hq, hkv, d = 37, 4, 2, 128
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).bfloat16()
    key = qkv[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
    value = qkv[:, (hq + hkv) * d:].view(n, hkv, d)
    num_blocks = 6
    k_cache = torch.zeros(num_blocks, 256, hkv, d, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    slots = torch.randperm(num_blocks * 256, generator=g)[:n].to(torch.int32)
    store_kvcache(key, value, k_cache, v_cache, slots)
    return {"seed": 4242, "n": n, "hq": hq, "hkv": hkv, "num_blocks": num_blocks,
            "qkv_digest": digest(qkv), "slots": slots.tolist(),
            "k_cache_digest": digest(k_cache), "v_cache_digest": digest(v_cache)}


def golden_attention():
    """SDPA expectations: the dense causal case of the reference's test (reduced head count),
    and single-query attention over ragged contexts (what paged decode must reproduce once
    the same keys are laid out in pages)."""
    g = torch.Generator().manual_seed(9001)
    out = {"seed": 9001}
    Q = torch.randn(1, 4, 64, 128, generator=g).bfloat16()
    K = torch.randn(1, 4, 64, 128, generator=g).bfloat16()
    V = torch.randn(1, 4, 64, 128, generator=g).bfloat16()
    O = torch.nn.functional.scaled_dot_product_attention(Q, K, V, is_causal=True)
    out["dense_inputs_digest"] = digest(torch.cat([Q, K, V]))
    np.save(HERE / "dense_causal_O.npy", bits(O))
    lens = [1, 255, 256, 257, 700]
    hq, hkv = 4, 2
    outs = []
    dig = hashlib.sha256()
    for n in lens:
        q = torch.randn(hq, 1, 128, generator=g).bfloat16()
        k = torch.randn(hkv, n, 128, generator=g).bfloat16()
        v = torch.randn(hkv, n, 128, generator=g).bfloat16()
        dig.update(digest(torch.cat([q.flatten(), k.flatten(), v.flatten()])).encode())
        o = torch.nn.functional.scaled_dot_product_attention(
            q.float(), k.float().repeat_interleave(hq // hkv, 0), v.float().repeat_interleave(hq // hkv, 0))
        outs.append(o[:, 0, :])
    out["decode_lens"], out["decode_hq"], out["decode_hkv"] = lens, hq, hkv
    out["decode_inputs_digest"] = dig.hexdigest()
    np.save(HERE / "decode_sdpa_O.npy", torch.stack(outs).numpy())
    return out


def golden_norm_rope():
    """Per-head RMSNorm followed by the NeoX rotary embedding, computed by the reference's own
    Python code: RMSNorm.rms_forward (infer/ops/norm.py:63-73, the function under its
    torch.compile decorator, run eagerly) and _apply_rotary_emb_torch (infer/ops/rope.py:46-64).
    The cos/sin cache is an input: it is built here with the reference's formula
    (infer/ops/rope.py:100-115) on the CPU."""
    from infer.ops.norm import RMSNorm
    from infer.ops.rope import _apply_rotary_emb_torch
    g = torch.Generator().manual_seed(31337)
    t, h, d = 7, 3, 128
    x = (torch.randn(t, h, d, generator=g) * 1.7).bfloat16()
    weight = (1.0 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    positions = torch.tensor([0, 1, 2, 100, 255, 257, 1023], dtype=torch.int64)
    inv_freq = 1.0 / (100000.0 ** (torch.arange(0, d, 2, dtype=torch.bfloat16) / d))
    freqs = torch.einsum("i,j -> ij", torch.arange(1024, dtype=torch.bfloat16), inv_freq)
    cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1)
    norm = RMSNorm(d)
    norm.weight.data.copy_(weight)
    eager = getattr(RMSNorm.rms_forward, "_torchdynamo_orig_callable", None)
    assert eager is not None, "cannot reach the undecorated rms_forward"
    with torch.no_grad():
        xn = eager(norm, x.clone())
        cos, sin = cache.index_select(0, positions).chunk(2, dim=-1)
        out = _apply_rotary_emb_torch(xn, cos, sin, True)
    np.save(HERE / "norm_rope_out.npy", bits(out))
    np.save(HERE / "norm_only_out.npy", bits(xn))
    return {"seed": 31337, "t": t, "h": h, "positions": positions.tolist(), "theta": 100000.0, "max_position": 1024,
            "eps": 1e-6, "inputs_digest": digest(torch.cat([x.flatten(), weight])), "cache_digest": digest(cache)}


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of Graylatzhou/Infer>")
    root = sys.argv[1]
    BlockManager, ModelRunner, Sequence, SamplingParams, store_kvcache, get_context = import_reference(root)
    result = {
        "norm_rope": golden_norm_rope(),
        "allocator": golden_allocator(BlockManager, ModelRunner, Sequence, SamplingParams, get_context),
        "append": golden_append(store_kvcache),
        "attention": golden_attention(),
        "versions": {"torch": torch.__version__, "numpy": np.__version__},
    }
    with open(HERE / "golden.json", "w") as f:
        json.dump(result, f)
    print("wrote", HERE / "golden.json")


if __name__ == "__main__":
    main()
