"""The path driven end to end the way the reference engine drives it (scheduler -> step metadata
-> model -> postprocess; decode through per-bucket CUDA graphs over static buffers), with a
synthetic-weight attention layer standing in for the model, whose weights are not available.

More than 700 decode steps grow four requests across page boundaries; one request finishes
and a later prompt re-uses its pages through the prefix cache; one request is preempted and
resumed.  Every step's append and attention are checked against the CPU oracle stepped the same
way: the oracle gets the same q/k/v rows and the same step metadata, keeps its own pools, and
must end up with bit-identical pools and attention outputs within the bf16 tolerance."""
import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close
from infer_b200.context import get_context, reset_context
from infer_b200.engine import AttentionLayerModel, Engine, LayerRunner
from oracle import paged_kv_oracle as oracle
from test_engine_cpu import scenario

pytestmark = pytest.mark.gpu


def _oracle_step(tap, ctx, n_rows, is_prefill, kc, vc, scale):
    q, k, v, o = (tap[name][:n_rows].cpu() for name in ("q", "k", "v", "o"))
    oracle.store_kvcache(k, v, kc, vc, ctx.slot_mapping.cpu())
    if is_prefill:
        want = oracle.paged_prefill(q, kc, vc, ctx.cu_seqlens_q.cpu(), ctx.cu_seqlens_k.cpu(), ctx.block_tables.cpu(), scale)
    else:
        want = oracle.paged_decode(q, kc, vc, ctx.context_lens.cpu(), ctx.block_tables.cpu(), scale)
    return o.view(want.shape), want


@pytest.mark.parametrize("eager,device_metadata", [(False, False), (True, False), (False, True)],
                         ids=["bucket-graphs", "eager", "bucket-graphs-device-metadata"])
def test_engine_loop_against_oracle(eager, device_metadata):
    torch.cuda.set_device(0)
    num_blocks, hq, hkv = 7, 16, 8
    sch, seqs, c_prompt = scenario(num_blocks)
    model = AttentionLayerModel(hidden=256, n_q_heads=hq, n_kv_heads=hkv, vocab=1000, max_position=2048, device="cuda")
    runner = LayerRunner(model, num_blocks, 256, max_num_seqs=8, max_model_len=1536, device="cuda", enforce_eager=eager,
                         device_metadata=device_metadata)
    assert eager or runner.graph_bs == [1, 2, 4, 8]
    runner.kv_cache.zero_()                               # the capture's warm-up steps wrote nothing (slot -1), but be explicit
    engine = Engine(runner, sch)
    kc = torch.zeros(num_blocks, 256, hkv, 128, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    decode_steps, prefills, late, buckets = 0, [], False, set()
    limit = 40 if eager else 10 ** 9                       # the eager variant only needs to show the same ops agree
    while not sch.is_finished() and engine.steps < limit:
        batch, is_prefill, _ = engine.step()
        ctx = get_context()
        n_rows = int(ctx.cu_seqlens_q[-1]) if is_prefill else len(batch)
        got, want = _oracle_step(runner.last_tap, ctx, n_rows, is_prefill, kc, vc, model.attn.scale)
        assert_close(got, want, ATOL_BF16, RTOL_BF16, f"step {engine.steps} ({'prefill' if is_prefill else 'decode'})")
        if is_prefill:
            prefills += [(len(s) - 1, s.num_cached_tokens) for s in batch]
        else:
            decode_steps += 1
            buckets.add(runner.last_bucket)
        reset_context()
        if engine.steps % 64 == 0 or sch.is_finished():
            torch.cuda.synchronize()
            assert torch.equal(runner.kv_cache[0].cpu().view(torch.int16), kc.view(torch.int16)), f"k pool differs at step {engine.steps}"
            assert torch.equal(runner.kv_cache[1].cpu().view(torch.int16), vc.view(torch.int16)), f"v pool differs at step {engine.steps}"
        if not late and seqs["C"].num_completion_tokens == 40:
            seqs["D"] = engine.add_request(c_prompt, 100)
            late = True
    if eager:
        return
    assert decode_steps >= 600 and sch.preemptions == 1
    assert (600, 512) in prefills and (300, 256) in prefills       # shared prefix, revived page
    assert prefills[-1][0] > 600 and prefills[-1][1] >= 512        # the preempted request resumed on its old pages
    assert 4 in buckets and buckets <= {1, 2, 4}                    # batches of 3 ran in the bucket of 4, padded rows skipped
    assert [s.num_completion_tokens for s in seqs.values()] == [700, 500, 40, 100]
