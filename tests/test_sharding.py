"""CPU: batch x heads sharding bookkeeping, including a 2-rank gloo run of the host logic."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernels_b200 import sharding
from oracle import streaming_attention_oracle as SO


def test_useful_pairs_agrees_with_oracle():
    for L, c, b in [(0, 4, 1), (1, 4, 1), (100, 7, 3), (256, 64, 8), (16384, 256, 2), (33, 40, 0)]:
        assert sharding.useful_pairs(L, c, b) == SO.useful_pairs(L, c, b)


@pytest.mark.parametrize("B,H,world", [(4, 32, 1), (4, 32, 8), (64, 32, 4), (3, 6, 4), (5, 1, 2), (2, 3, 8)])
def test_partition_covers_every_slice_once_and_balances(B, H, world):
    lens = SO.make_lens(B, 100, 800, seed=1).tolist()
    shards = sharding.partition(B, H, world, lens, T=800, context_size=64, back_contexts=2)
    seen = sorted(u for s in shards for u in s.units)
    assert seen == [(b, h) for b in range(B) for h in range(H)]
    total = sum(s.work for s in shards)
    assert total == H * sum(SO.useful_pairs(min(L, 800), 64, 2) for L in lens)
    if H % world == 0:
        assert len({s.work for s in shards}) == 1
    elif B * H >= 2 * world:
        biggest = max(SO.useful_pairs(min(L, 800), 64, 2) for L in lens)
        assert max(s.work for s in shards) - min(s.work for s in shards) <= biggest


def test_take_and_put_roundtrip():
    x = torch.arange(2 * 6 * 3 * 2, dtype=torch.float32).reshape(2, 6, 3, 2)
    for world in (2, 3, 4):
        full = torch.zeros_like(x)
        for s in sharding.partition(2, 6, world, None, T=3):
            loc = sharding.take_local(x, s)
            sharding.put_local(full, loc, s)
        assert torch.equal(full, x)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, H, T, D, c, back, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens = SO.make_lens(B, T // 2, T, seed=0)
        shard = sharding.partition(B, H, world, lens.tolist(), T=T, context_size=c, back_contexts=back)[rank]
        # each rank builds ONLY its own slices from the per-slice seeds and evaluates them with the
        # oracle (the CUDA operator has no CPU path); what is under test is the bookkeeping.
        outs = {}
        for (b, h) in shard.units:
            q, k, v, do = SO.make_slice(b, h, H, T, D, seed=0)
            o, *_ = SO.banded_fwd_bwd(q, k, v, do, c, back, int(lens[b]))
            outs[(b, h)] = o.float()
        work = torch.tensor([float(shard.work)])
        dist.all_reduce(work, op=dist.ReduceOp.MAX)  # the only cross-rank traffic: a scalar
        torch.save({"outs": outs, "max_work": work.item(), "units": shard.units}, os.path.join(out_dir, f"r{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_run_reassembles_single_rank_result(tmp_path):
    B, H, T, D, c, back = 2, 4, 48, 8, 8, 1
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), B, H, T, D, c, back, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    assert sorted(u for p in parts for u in p["units"]) == [(b, h) for b in range(B) for h in range(H)]
    lens = SO.make_lens(B, T // 2, T, seed=0)
    for p in parts:
        for (b, h), o in p["outs"].items():
            q, k, v, do = SO.make_slice(b, h, H, T, D, seed=0)
            ref, *_ = SO.banded_fwd_bwd(q, k, v, do, c, back, int(lens[b]))
            assert torch.equal(o, ref.float())
    assert parts[0]["max_work"] == parts[1]["max_work"]
