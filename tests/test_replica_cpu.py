"""CPU: the replica-parallel plumbing with two gloo ranks — sharding covers every unit once, results merge back in
input order, the timing reduction is the max over ranks, and a failing rank is reported instead of hanging the others."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from pimaicompiler_b200 import replica

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_and_merge_roundtrip():
    for n in (0, 1, 7, 128, 1024):
        for world in (1, 2, 3, 8):
            shards = [replica.shard_indices(n, r, world) for r in range(world)]
            assert sorted(i for sh in shards for i in sh) == list(range(n))
            assert max(len(s) for s in shards) - min(len(s) for s in shards) <= 1
            assert replica.merge_shards([[i * 10 for i in sh] for sh in shards], n) == [i * 10 for i in range(n)]
    with pytest.raises(ValueError):
        replica.shard_indices(4, 2, 2)
    with pytest.raises(ValueError):
        replica.merge_shards([[1], []], 3)


def _worker(rank, world, port, n_items, q):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from pimaicompiler_b200 import replica as rp
    r, w, l = rp.env_rank()
    rp.init_process_group(w, l, use_cuda=False)
    mine = rp.shard_indices(n_items, r, w)
    results = [[i, i * i] for i in mine]           # stands for the token list of utterance i
    rp.barrier(w)
    slowest = rp.max_over_ranks(1.0 + r, w)       # rank r "took" 1+r seconds
    total = rp.sum_over_ranks(len(mine), w)
    gathered = rp.gather_objects(results, w)
    merged = rp.merge_shards(gathered, n_items)
    q.put((r, slowest, total, merged))
    import torch.distributed as dist
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_time_and_gather():
    world, n_items = 2, 11
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_items, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r, slowest, total, merged in out:
        assert slowest == 2.0                       # max over ranks, not this rank's own time
        assert total == n_items
        assert merged == [[i, i * i] for i in range(n_items)]


def _failing_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        os._exit(3)                                 # a replica dies between steps, nothing in flight
    try:
        dist.barrier()
        dist.all_reduce(torch.zeros(1))
        q.put((rank, "no error"))
    except Exception as e:                          # the survivor learns of it through the short group timeout
        q.put((rank, "detected: " + type(e).__name__))


def test_a_dead_replica_is_detected_not_waited_for_forever():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    rank0, msg = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
    assert procs[1].exitcode == 3
    assert rank0 == 0 and msg.startswith("detected")
