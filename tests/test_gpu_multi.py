"""Two ranks on two GPUs (skipped with fewer): a chain of column-sharded RNS layers whose
outputs are exchanged (a) by the NCCL all-gather, (b) by peer stores from the GEMM
epilogue into symmetric memory plus a barrier and (c) by the same stores as NVLink multicast
stores, where the platform maps a multicast address.  All must reproduce, bit for bit, the
unsharded layers run on one GPU, including the absmax words that travel with the blocks."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

C0 = (127, 126, 125, 121)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from rns_llm_b200.backends import CudaRNSBackend
        from rns_llm_b200.parallel import (ColumnShardedRNSLinear, GatheredActivation, PeerArena, group_view,
                                           shard_tensor, unshard)
        backend = CudaRNSBackend()
        torch.manual_seed(77)                                     # the same full problem on every rank
        m, k = 1024, 1024
        x = torch.randn(m, k, dtype=torch.float16, device=device)
        w1 = (torch.randn(1536, k, device=device) * 0.04).half()
        b1 = (torch.randn(1536, device=device) * 0.1).half()
        w2 = (torch.randn(1024, 1536, device=device) * 0.04).half()

        def chain(arena, multicast=False):
            l1 = ColumnShardedRNSLinear(shard_tensor(w1, world, rank), shard_tensor(b1, world, rank),
                                        backend=backend, moduli=C0, rank=rank, world=world, peer_arena=arena,
                                        multicast=multicast)
            l2 = ColumnShardedRNSLinear(shard_tensor(w2, world, rank), None, backend=backend, moduli=C0, rank=rank,
                                        world=world, peer_arena=arena, multicast=multicast)
            if multicast and not (l1.multicast and l2.multicast):
                return None
            y1 = l1(x)
            carried = isinstance(y1, GatheredActivation) and y1.absmax_words is not None
            y2 = l2(y1)
            torch.cuda.synchronize()
            return unshard(y1, 1).clone(), unshard(y2, 1).clone(), carried

        # unsharded, on this rank alone
        f1 = ColumnShardedRNSLinear(w1, b1, backend=backend, moduli=C0, rank=0, world=1)
        f2 = ColumnShardedRNSLinear(w2, None, backend=backend, moduli=C0, rank=0, world=1)
        full1 = f1(x)
        full2 = unshard(f2(full1), 1)
        full1 = unshard(full1, 1)
        n1, n2, carried_nccl = chain(None)
        checks = {"nccl layer 1": torch.equal(n1, full1), "nccl layer 2": torch.equal(n2, full2),
                  "nccl absmax words": bool(carried_nccl)}
        peer_note = ""
        try:
            arena = PeerArena(64 << 20, device)
        except Exception as exc:                                  # platform without symmetric memory
            arena, peer_note = None, f"symmetric memory unavailable: {type(exc).__name__}: {exc}"
        flag = torch.tensor([1 if arena is not None else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()):
            for _ in range(3):                                    # buffers are reused: several rounds
                p1, p2, carried_peer = chain(arena)
                checks["peer layer 1"] = checks.get("peer layer 1", True) and torch.equal(p1, full1)
                checks["peer layer 2"] = checks.get("peer layer 2", True) and torch.equal(p2, full2)
                checks["peer absmax words"] = checks.get("peer absmax words", True) and bool(carried_peer)
            # the same exchange as multicast stores through NVSwitch, where the platform maps one
            mc = torch.tensor([1 if arena.multicast_base else 0], device=device)
            dist.all_reduce(mc, op=dist.ReduceOp.MIN)
            if int(mc.item()):
                for _ in range(3):
                    got = chain(arena, multicast=True)
                    checks["multicast layer 1"] = checks.get("multicast layer 1", True) and torch.equal(got[0], full1)
                    checks["multicast layer 2"] = checks.get("multicast layer 2", True) and torch.equal(got[1], full2)
                    checks["multicast absmax words"] = checks.get("multicast absmax words", True) and bool(got[2])
                peer_note += " multicast exchange checked"
            else:
                peer_note += " no multicast mapping: multicast exchange not run"
        backend.check_status()
        failed = [name for name, good in checks.items() if not good]
        results[rank] = (not failed, f"failed: {failed}; {peer_note}")
        print(f"rank {rank}: {sorted(checks)}; {peer_note}", flush=True)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_chain_nccl_and_peer_stores():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert all(results[r][0] for r in range(world)), dict(results)
