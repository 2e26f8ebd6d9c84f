"""The engine stand-in's scheduler over the native page allocator, without a GPU: admission,
prefix-cache hits, growth across page boundaries, a request finishing and its pages being
re-used by a later prompt that revives their digests, preemption and resume."""
import numpy as np

from infer_b200.engine import Scheduler
from infer_b200.sequence import Sequence


def scenario(num_blocks=7, seed=7):
    """Three requests at once (B shares A's first two pages), a fourth arriving when C has finished
    with C's prompt; the pool is one page short of what A and B need at their longest."""
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 1000, 600).tolist()
    b = a[:512] + rng.integers(0, 1000, 88).tolist()
    c = rng.integers(0, 1000, 300).tolist()
    sch = Scheduler(num_blocks, 256, max_num_seqs=8)
    seqs = {"A": Sequence(a, 700), "B": Sequence(b, 500), "C": Sequence(c, 40)}
    for s in seqs.values():
        sch.add(s)
    return sch, seqs, c


def test_scheduler_life_cycle_with_preemption_and_prefix_hits():
    sch, seqs, c_prompt = scenario()
    rng = np.random.default_rng(1)
    prefills, decode_steps, late = [], 0, False
    while not sch.is_finished():
        batch, is_prefill = sch.schedule()
        for s in batch:                                   # every scheduled request owns exactly the pages it needs
            assert len(s.block_table) == s.num_blocks
        if is_prefill:
            prefills += [(len(s), s.num_cached_tokens) for s in batch]
        else:
            decode_steps += 1
        sch.postprocess(batch, [int(rng.integers(0, 1000)) for _ in batch])
        if not late and seqs["C"].num_completion_tokens == 40:
            seqs["D"] = Sequence(c_prompt, 100)            # C's pages are free again; its first page's digest survives
            sch.add(seqs["D"])
            late = True
    assert prefills[:3] == [(600, 0), (600, 512), (300, 0)]       # B shares A's two full pages
    assert (300, 256) in prefills                                 # D revives C's sealed page
    assert sch.preemptions == 1
    resumed = prefills[-1]
    assert resumed[0] > 600 and resumed[1] >= 512                 # the preempted request comes back with its pages found again
    assert decode_steps >= 600
    assert [s.num_completion_tokens for s in seqs.values()] == [700, 500, 40, 100]
    assert sch.block_manager.num_free() == 7 and sum(sch.block_manager.ref_counts()) == 0
