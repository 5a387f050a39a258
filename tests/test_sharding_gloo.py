"""The multi-GPU plumbing on CPU: two gloo ranks shard P, run a stand-in operator (the CPU
checker) on their slices, and the gathered result equals the single-process one."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_cover_p_in_order():
    from sharding import shard_range
    for P in (1, 2, 5, 48, 96):
        for world in (1, 2, 3, 4, 8):
            parts = [shard_range(P, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == P
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in parts]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, P, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "quasi-linear-kernel-attention_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import sorted_scan
    from sharding import sharded_call
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(P, 3, 40, generator=g), torch.randn(P, 3, 50, generator=g), torch.randn(P, 50, 4, generator=g)
    fn = lambda a, b, c: tuple(t.float() for t in sorted_scan.laplace_sum(a, b, c))
    local = sharded_call(fn, (q, k, v))
    full = sharded_call(fn, (q, k, v), gather=True)
    if rank == 0:
        want = fn(q, k, v)
        ret["ok"] = all(torch.allclose(a, b) for a, b in zip(full, want))
        ret["local_rows"] = 0 if local is None else local[0].shape[0]
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("P", [5, 1])
def test_two_rank_gather_matches_single_process(P):
    port = 29500 + (os.getpid() % 2000) + P
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, P, ret), nprocs=2, join=True)
        assert ret["ok"]
        assert ret["local_rows"] == (3 if P == 5 else 1)
