"""Failure detection without a GPU: a rank that leaves between steps is reported by the
survivors within a time limit instead of blocking them inside a collective (gloo ranks on
CPU), and error codes of the library turn into exceptions that say what happened."""
import os
import socket
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from infer_b200 import _lib
from infer_b200.sharding import PeerMissing, StepRendezvous, checked_gather_heads


def _rank_main(rank, world, port, leave_after, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", port + 1, world, is_master=(rank == 0), timeout=timedelta(seconds=30))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    rdv = StepRendezvous(store, rank, world, timeout_s=2.0)
    local = torch.full((3, 2, 4), float(rank))
    try:
        for step in range(4):
            if rank == 1 and step == leave_after:
                # the rank leaves between steps: none of its collectives is in flight
                result.put(("left", rank, step))
                result.close()
                result.join_thread()                # the message is on its way before the process goes
                os._exit(0)
            t0 = time.monotonic()
            try:
                full = checked_gather_heads(local, rdv, step)
            except PeerMissing as e:
                result.put(("missing", rank, e.step, e.ranks, time.monotonic() - t0))
                return
            assert full.shape == (3, 2 * world, 4)
        result.put(("done", rank))
    finally:
        if rank == 0:
            time.sleep(0.2)


def _free_port_pair():
    while True:
        with socket.socket() as a:
            a.bind(("127.0.0.1", 0))
            port = a.getsockname()[1]
        with socket.socket() as b:
            try:
                b.bind(("127.0.0.1", port + 1))
            except OSError:
                continue
        return port


@pytest.mark.timeout(120)
def test_rank_that_leaves_between_steps_is_reported_not_waited_for():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port_pair()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, 2, result)) for r in range(2)]
    for p in procs:
        p.start()
    seen = [result.get(timeout=90), result.get(timeout=90)]
    for p in procs:
        p.join(30)
    kinds = {m[0]: m for m in seen}
    assert "left" in kinds and kinds["left"][1:] == (1, 2)
    assert "missing" in kinds, seen
    _, rank, step, ranks, waited = kinds["missing"]
    assert rank == 0 and step == 2 and ranks == [1]
    assert waited < 10.0                           # the 2 s limit, not the process group's


def test_rendezvous_passes_when_everyone_arrives():
    store = dist.HashStore()
    a, b = StepRendezvous(store, 0, 2, 1.0), StepRendezvous(store, 1, 2, 1.0)
    store.set("step0/rank1", b"1")                 # rank 1 got there first
    a.arrive(0)
    b.arrive(0)
    with pytest.raises(PeerMissing) as e:
        a.arrive(1)                                # nobody else reaches step 1
    assert e.value.ranks == [1] and e.value.step == 1


def test_device_error_code_becomes_an_exception():
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        _lib.check(_lib.ERR_DEVICE, "paged_attn_decode (device status)")
    with pytest.raises(RuntimeError, match="built-in scratch"):
        _lib.check(_lib.ERR_TOO_LARGE, "noalloc")
    _lib.check(_lib.OK, "fine")
