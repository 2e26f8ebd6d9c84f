"""Device-side decode metadata (DecodeState.advance) against the host rebuild that mirrors the
reference's prepare_decode, over many steps that cross page boundaries."""
import pytest
import torch

from infer_b200 import BlockManager, Sequence, get_context, metadata

pytestmark = pytest.mark.gpu


def test_advance_tracks_prepare_decode_over_page_boundaries():
    bs = 256
    mgr = BlockManager(64, bs)
    prompts = [250, 255, 256, 511, 3, 700]
    seqs = [Sequence(list(range(n))) for n in prompts]
    for s in seqs:
        mgr.allocate(s)
    state = metadata.DecodeState(max_batch=8, max_pages=6, block_size=bs, device="cuda")   # 2 padding rows
    state.load(seqs)
    for step in range(270):
        for s in seqs:                                   # the engine appends the sampled token, then grows pages
            s.append_token(step)
            mgr.may_append(s)
        state.publish_new_pages(seqs)
        state.advance()
        torch.cuda.synchronize()
        _, positions = metadata.prepare_decode(seqs, bs)  # host rebuild (the reference's way)
        ref = get_context()
        n = len(seqs)
        assert state.context_lens[:n].cpu().tolist() == ref.context_lens.tolist(), step
        assert state.slot_mapping[:n].cpu().tolist() == ref.slot_mapping.tolist(), step
        assert state.positions[:n].cpu().tolist() == positions.tolist(), step
        width = ref.block_tables.shape[1]
        assert state.block_tables[:n, :width].cpu().tolist() == ref.block_tables.tolist(), step
        assert state.context_lens[n:].cpu().tolist() == [0, 0] and state.slot_mapping[n:].cpu().tolist() == [-1, -1]


def test_advance_marks_missing_page():
    state = metadata.DecodeState(max_batch=2, max_pages=2, block_size=256, device="cuda")
    s = Sequence(list(range(256)))
    s.block_table = [3]                                  # the allocator has not provided page 2 yet
    state.load([s])
    state.advance()
    torch.cuda.synchronize()
    assert state.context_lens.cpu().tolist() == [257, 0]
    assert state.slot_mapping.cpu().tolist() == [-1, -1]  # append will skip the row instead of writing anywhere
