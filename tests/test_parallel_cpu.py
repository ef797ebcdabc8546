"""Host-side logic of the column-sharded path on CPU: shard arithmetic, and a
world_size-2 gloo run in which every rank computes its shard with plain integer
torch ops (a stand-in for the GPU kernel, used by this test only), all-gathers,
and the reassembled result must equal the unsharded product."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rns_llm_b200.parallel import group_view, shard_rows, shard_tensor, unshard


def test_shard_rows_and_errors():
    assert shard_rows(12, 2, 0) == [slice(0, 6)]
    assert shard_rows(12, 2, 1) == [slice(6, 12)]
    assert shard_rows(12, 2, 1, groups=3) == [slice(2, 4), slice(6, 8), slice(10, 12)]
    with pytest.raises(ValueError):
        shard_rows(10, 4, 0)
    with pytest.raises(ValueError):
        shard_rows(12, 2, 2)


@pytest.mark.parametrize("world,groups", [(1, 1), (2, 1), (4, 1), (2, 3), (4, 3), (8, 3)])
def test_unshard_inverts_sharding(world, groups):
    n, m, k = 24 * groups, 5, 7
    torch.manual_seed(0)
    w = torch.randint(-9, 10, (n, k))
    x = torch.randint(-9, 10, (m, k))
    full = x @ w.t()
    gathered = torch.stack([x @ shard_tensor(w, world, r, groups).t() for r in range(world)])
    assert torch.equal(unshard(gathered, groups), full)
    per = n // groups
    for g in range(groups):
        part = group_view(gathered, groups, g)
        assert torch.equal(unshard(part.contiguous(), 1), full[:, g * per:(g + 1) * per])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(1234)                       # same full problem on every rank
        m, k, hidden = 6, 16, 8
        x = torch.randint(-127, 128, (m, k), dtype=torch.int32)
        w_qkv = torch.randint(-127, 128, (3 * hidden, k), dtype=torch.int32)
        w_out = torch.randint(-127, 128, (k, hidden), dtype=torch.int32)
        # layer 1: fused qkv, sharded inside each of q, k, v
        local = x @ shard_tensor(w_qkv, world, rank, groups=3).t()
        gathered = torch.empty((world, m, local.shape[1]), dtype=torch.int32)
        gathered[rank] = local
        dist.all_gather_into_tensor(gathered.view(world * m, -1), gathered[rank].clone())
        full_qkv = x @ w_qkv.t()
        ok = torch.equal(unshard(gathered, 3), full_qkv)
        # layer 2 consumes the q block straight from the gathered layout
        q_blocks = group_view(gathered, 3, 0)                     # [G, M, hidden/G]
        q = unshard(q_blocks.contiguous(), 1)
        ok = ok and torch.equal(q, full_qkv[:, :hidden])
        local2 = q @ shard_tensor(w_out, world, rank).t()
        gathered2 = torch.empty((world, m, local2.shape[1]), dtype=torch.int32)
        dist.all_gather_into_tensor(gathered2.view(world * m, -1), local2.contiguous())
        ok = ok and torch.equal(unshard(gathered2, 1), full_qkv[:, :hidden] @ w_out.t())
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharded_layers():
    world = 2
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
