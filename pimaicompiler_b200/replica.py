"""Replica-parallel plumbing: utterances / sentences are independent, so N GPUs run N replicas of the model and no
collective touches the data path.  torch.distributed is used for rendezvous, the barrier around the timed region and
the max-over-ranks of the device time only (NCCL on GPUs, gloo in the CPU tests).

The reference's multi-GPU mode has the same shape — one worker thread and one runtime per GPU, the batch chunked
over the GPUs and the outputs concatenated (runtime/python/pipeline_manager/pipeline_manager.cpp:27-53, 86-121) — but
collects results through a shared vector whose order depends on thread finish times; here every unit keeps its index.
"""
from __future__ import annotations

import os
from typing import List, Sequence, Tuple

import torch


def env_rank() -> Tuple[int, int, int]:
    """(rank, world_size, local_rank) from the torchrun environment; (0, 1, 0) when launched plainly."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def shard_indices(n_items: int, rank: int, world: int) -> List[int]:
    """Round-robin shard of range(n_items): unit i goes to rank i % world.  Every index appears exactly once over
    the ranks, and shard sizes differ by at most one."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("need 0 <= rank < world")
    return list(range(rank, n_items, world))


def merge_shards(shards: Sequence[Sequence], n_items: int) -> list:
    """Inverse of shard_indices: shards[r][k] is the result of unit r + k*world."""
    world = len(shards)
    out = [None] * n_items
    for r, sh in enumerate(shards):
        idx = shard_indices(n_items, r, world)
        if len(sh) != len(idx):
            raise ValueError(f"rank {r} returned {len(sh)} results for {len(idx)} units")
        for i, v in zip(idx, sh):
            out[i] = v
    return out


def init_process_group(world: int, local_rank: int, use_cuda: bool) -> None:
    if world <= 1:
        return
    import torch.distributed as dist
    if dist.is_initialized():
        return
    if use_cuda:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group("gloo")


def barrier(world: int) -> None:
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def _reduce(value: float, world: int, op_name: str) -> float:
    if world == 1:
        return float(value)
    import torch.distributed as dist
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=getattr(dist.ReduceOp, op_name))
    return float(t.item())


def max_over_ranks(value: float, world: int) -> float:
    """The slowest rank's time: what a multi-GPU throughput number must be computed from."""
    return _reduce(value, world, "MAX")


def sum_over_ranks(value: float, world: int) -> float:
    return _reduce(value, world, "SUM")


def gather_objects(obj, world: int) -> list:
    """Host-side gather of per-rank Python results (token lists); rank order."""
    if world == 1:
        return [obj]
    import torch.distributed as dist
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out
