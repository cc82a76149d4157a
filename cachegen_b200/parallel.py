"""Sharding of the codec's independent units across the GPUs of one box, one process per GPU.

Every (row, channel, sub-chunk) stream is independent, tables are per chunk and scales per (row,
token), so the codec has no exchange step: work is split by request, by token chunk or by layer and
each rank runs the single-GPU path on its share.  The only communication is the optional delivery of
decoded KV to the GPU that consumes it (`gather_layers`, NCCL over NVLink; gloo on CPU in the tests).
"""
from typing import List, Optional

import torch
import torch.distributed as dist


def partition(n_units: int, world: int, rank: int) -> range:
    """Contiguous, balanced share of `n_units` for `rank` (the first n_units % world ranks get one more)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def max_over_ranks(value: float, device="cpu", group=None) -> float:
    """The slowest rank's time: what a whole-job throughput must be computed from."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def all_agree_ok(ok: bool, device="cpu", group=None) -> bool:
    """True when every rank reports success (a rank that met a malformed blob says so before any
    collective on the data path is entered)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return bool(ok)
    t = torch.tensor([0 if ok else 1], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t.item()) == 0


def gather_layers(local: torch.Tensor, total_layers: int, root: int = 0, out: Optional[torch.Tensor] = None,
                  group=None) -> Optional[torch.Tensor]:
    """Delivers layer-sharded decoded KV to `root`.

    local: this rank's layers, [L_r, 2, T, H, D] ("vllm") or [L_r, 2, H, T, D], L_r = len(partition(
    total_layers, world, rank)), contiguous.  On `root` returns the full blob [total_layers, ...]
    (`out` when given); elsewhere returns None.  Layer-major layout makes every rank's share one
    contiguous slab of the result, so each transfer is a single send / receive.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    mine = partition(total_layers, world, rank)
    if local.shape[0] != len(mine) or not local.is_contiguous():
        raise RuntimeError("local slab must be contiguous and hold exactly this rank's layers")
    if world == 1:
        if out is not None:
            out.copy_(local)
            return out
        return local
    if rank == root:
        if out is None:
            out = torch.empty((total_layers,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        ops: List[dist.P2POp] = []
        for r in range(world):
            part = partition(total_layers, world, r)
            if len(part) == 0:
                continue
            if r == root:
                out[part.start:part.stop].copy_(local)
            else:
                ops.append(dist.P2POp(dist.irecv, out[part.start:part.stop], r, group))
        for req in (dist.batch_isend_irecv(ops) if ops else []):
            req.wait()
        return out
    if len(mine):
        for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, local, root, group)]):
            req.wait()
    return None
