"""The multi-rank host logic on CPU: two gloo ranks shard requests / layers, agree on the slowest
rank's time and deliver layer-sharded KV to rank 0."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cachegen_b200.parallel import all_agree_ok, gather_layers, max_over_ranks, partition


def test_partition_covers_every_unit_once():
    for n in (0, 1, 7, 8, 64, 80):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                part = partition(n, world, r)
                seen += list(part)
                assert len(part) in (n // world, n // world + 1)
            assert seen == list(range(n))
    assert list(partition(80, 8, 3)) == list(range(30, 40))  # 10 layers per GPU for the 80-layer model
    with pytest.raises(ValueError):
        partition(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, T, H, D = 5, 3, 2, 4
        full = torch.arange(L * 2 * T * H * D, dtype=torch.float32).reshape(L, 2, T, H, D).to(torch.float16)
        mine = partition(L, world, rank)
        local = full[mine.start:mine.stop].contiguous()
        got = gather_layers(local, L, root=0)
        ok = True
        if rank == 0:
            ok = got is not None and torch.equal(got, full)
        else:
            ok = got is None
        slowest = max_over_ranks(10.0 + rank)
        agree_all = all_agree_ok(True)
        agree_one_bad = all_agree_ok(rank != 1)
        results[rank] = (ok, slowest, agree_all, agree_one_bad, list(partition(64, world, rank)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_deliver():
    world = 2
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            ok, slowest, agree_all, agree_one_bad, part = results[rank]
            assert ok
            assert slowest == 11.0          # the max over ranks, on every rank
            assert agree_all is True
            assert agree_one_bad is False   # rank 1 reported a failure: nobody proceeds
            assert part == list(range(rank * 32, rank * 32 + 32))


def test_token_range_copy_refuses_other_layouts():
    """The two-dimensional copy only takes token ranges of contiguous [L, 2, T, H, D] tensors (checked
    before anything is enqueued)."""
    import pytest
    import torch
    from cachegen_b200.parallel import copy_token_range_async
    a = torch.zeros(3, 2, 16, 4, 8, dtype=torch.float16)
    b = torch.zeros(3, 2, 16, 4, 8, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        copy_token_range_async(a[:, :, 2:6], b[:, :, 2:7], None)              # shapes differ
    with pytest.raises(RuntimeError):
        copy_token_range_async(a[:, :, 2:6], b.float()[:, :, 2:6], None)      # types differ
    with pytest.raises(RuntimeError):
        copy_token_range_async(a.permute(0, 1, 3, 2, 4)[:, :, :, 2:6].permute(0, 1, 3, 2, 4)[..., ::2],
                               b[:, :, 2:6][..., ::2], None)                  # not a unit innermost stride
    with pytest.raises(RuntimeError):
        copy_token_range_async(a[:, :1, 2:6].expand(3, 2, 4, 4, 8), b[:, :, 2:6], None)   # rows not evenly spaced
