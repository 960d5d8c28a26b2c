"""CPU tests of the multi-rank logic (gloo, world size 2): shards are disjoint, cover the problem, equal the
matching slices of the unsharded inputs, and per-shard gradients (FP64 oracle) assemble to the unsharded ones."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rewy_b200.sharding import shard
from rewy_b200.synthetic import make_inputs, operator_inputs


def test_shards_partition_every_batch_head_pair():
    for B, H, world in ((8, 32, 1), (8, 32, 2), (8, 32, 8), (2, 8, 8), (1, 4, 4)):
        seen = set()
        for r in range(world):
            bs, hs = shard(B, H, world, r)
            pairs = {(b, h) for b in bs for h in hs}
            assert not (pairs & seen)
            seen |= pairs
        assert seen == {(b, h) for b in range(B) for h in range(H)}
    with pytest.raises(ValueError):
        shard(3, 4, 2, 0)


def test_shard_inputs_equal_slices_of_the_full_problem():
    full = make_inputs("kda", 2, 64, 4, seed=9)
    part = make_inputs("kda", 2, 64, 4, seed=9, batches=[1], heads=[2, 3])
    for n in ("q", "k", "v", "g", "do"):
        assert torch.equal(part[n], full[n][1:2, :, 2:4])
    assert torch.equal(part["beta"], full["beta"][1:2, :, 2:4])
    assert torch.equal(part["initial_state"], full["initial_state"][1:2, 2:4])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out, B=2, T=128, H=2):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import chunk_backward, chunk_forward
    bs, hs = shard(B, H, world, rank)
    xs = make_inputs("gdn2", B, T, H, seed=4, batches=bs, heads=hs)
    ins = {n: (x.double() if x is not None else None) for n, x in operator_inputs("gdn2", xs).items()}
    g = chunk_backward("gdn2", ins, chunk_forward("gdn2", ins), xs["do"], xs["dht"])
    # timing-style reduction the benchmark uses: max over ranks
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    gathered = [None] * world
    dist.all_gather_object(gathered, {n: g[n] for n in ("dq", "dk", "dv", "dg", "db", "dw")} | {"bs": bs, "hs": hs})
    if rank == 0:
        torch.save({"max": t.item(), "parts": gathered}, out)
    dist.destroy_process_group()


def test_two_rank_shards_assemble_to_the_unsharded_gradients(tmp_path):
    from oracle import chunk_backward, chunk_forward
    out = tmp_path / "gathered.pt"
    mp.spawn(_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    res = torch.load(out, weights_only=False)
    assert res["max"] == 2.0
    xs = make_inputs("gdn2", 2, 128, 2, seed=4)
    ins = {n: (x.double() if x is not None else None) for n, x in operator_inputs("gdn2", xs).items()}
    full = chunk_backward("gdn2", ins, chunk_forward("gdn2", ins), xs["do"], xs["dht"])
    for part in res["parts"]:
        b0, b1 = part["bs"][0], part["bs"][-1] + 1
        h0, h1 = part["hs"][0], part["hs"][-1] + 1
        for n in ("dq", "dk", "dv", "dg", "db", "dw"):
            assert torch.allclose(part[n], full[n][b0:b1, :, h0:h1], atol=1e-12), n


def test_head_split_shards_of_a_fixed_problem_assemble_to_the_unsharded_gradients(tmp_path):
    """Fixed-problem (strong scaling) partition with more ranks than batch elements: both ranks own the one batch
    element and half of its heads each; the per-rank gradients are the matching head slices of the full problem."""
    from oracle import chunk_backward, chunk_forward
    B, T, H = 1, 128, 4
    assert shard(B, H, 2, 0) == ([0], [0, 1]) and shard(B, H, 2, 1) == ([0], [2, 3])
    out = tmp_path / "gathered_heads.pt"
    mp.spawn(_worker, args=(2, _free_port(), str(out), B, T, H), nprocs=2, join=True)
    res = torch.load(out, weights_only=False)
    xs = make_inputs("gdn2", B, T, H, seed=4)
    ins = {n: (x.double() if x is not None else None) for n, x in operator_inputs("gdn2", xs).items()}
    full = chunk_backward("gdn2", ins, chunk_forward("gdn2", ins), xs["do"], xs["dht"])
    assert sorted(tuple(p["hs"]) for p in res["parts"]) == [(0, 1), (2, 3)]
    for part in res["parts"]:
        h0, h1 = part["hs"][0], part["hs"][-1] + 1
        for n in ("dq", "dk", "dv", "dg", "db", "dw"):
            assert torch.allclose(part[n], full[n][:, :, h0:h1], atol=1e-12), n
