"""KV-head sharding on real GPUs: every rank runs append + paged decode on its own heads,
outputs are all-gathered over NCCL (validation only) and compared with the CPU oracle of the
unsharded problem.  Needs at least two GPUs; skipped otherwise."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gpu_util import ATOL_BF16, RTOL_BF16

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from infer_b200 import ops, workloads
        from infer_b200.sharding import gather_heads
        from oracle import paged_kv_oracle as oracle
        w = workloads.config4(batch=24, cap=3000)               # group 8, shared prefix pages
        s = w.shard(rank, world)
        kc, vc = s.k_cache.to(dev), s.v_cache.to(dev)
        ops.store_kvcache(s.k.to(dev), s.v.to(dev), kc, vc, s.slot_mapping.to(dev))
        local = ops.paged_attn_decode(s.q.to(dev), kc, vc, s.context_lens_tensor().to(dev),
                                      s.block_tables_tensor().to(dev), s.scale)
        full = gather_heads(local)
        torch.cuda.synchronize()
        if rank == 0:
            rk, rv = w.k_cache.clone(), w.v_cache.clone()
            oracle.store_kvcache(w.k, w.v, rk, rv, w.slot_mapping)
            want = oracle.paged_decode(w.q, rk, rv, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
            err = (full.float().cpu() - want.float()).abs()
            result.put(bool((err <= ATOL_BF16 + RTOL_BF16 * want.float().abs()).all()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_head_sharded_decode_over_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = 29700 + os.getpid() % 200 + world
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    ok = result.get(timeout=240)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert ok
