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


class _FakePrepared:
    kernel = "tcgen05"

    def __init__(self, w_q):
        self.w_q, self.n, self.k = w_q, int(w_q.shape[0]), int(w_q.shape[1])


class _FakeBackend:
    """Stand-in for CudaRNSBackend with plain torch arithmetic, for this file only: it
    lets the host logic of ColumnShardedRNSLinear (buffers, slots, gather) run on CPU."""

    def quantize_weight(self, weight):
        scale = weight.float().abs().amax(dim=1).clamp_min(1e-8) / 127.0
        return torch.clamp(torch.round(weight.float() / scale[:, None]), -127, 127).to(torch.int32), scale, None

    def prepare_weight_nk(self, w_q, moduli):
        return _FakePrepared(w_q)

    def supports_absmax_out(self, *, m, k, channels):
        return False

    def linear_forward(self, x, prepared, weight_scale, bias, *, per_row=False, out=None, absmax_in=None,
                       absmax_out=None, out_copies=(), absmax_copies=()):
        if x.ndim == 3:
            x = unshard(x.contiguous(), 1)
        s_a = x.float().abs().amax().clamp_min(1e-8) / 127.0
        x_q = torch.clamp(torch.round(x.float() / s_a), -127, 127).to(torch.int32)
        y = (x_q @ prepared.w_q.t()).float() * s_a * weight_scale[None, :]
        if bias is not None:
            y = y + bias[None, :]
        out.copy_(y.to(out.dtype))
        return out


def _layer_worker(rank: int, world: int, port: int, results):
    import torch.cuda as cuda
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # The layer keys its cached buffer by the current CUDA stream; there is none on CPU.
    class _NoStream:
        cuda_stream = 0
    cuda.current_stream = lambda device=None: _NoStream()
    try:
        from rns_llm_b200.parallel import ColumnShardedRNSLinear
        torch.manual_seed(99)
        weight, bias = torch.randn(8, 16), torch.randn(8)
        full = _FakeBackend()
        ok = True
        for reuse in (False, True):
            layer = ColumnShardedRNSLinear(shard_tensor(weight, world, rank), shard_tensor(bias, world, rank),
                                           backend=full, moduli=(127, 126, 125, 121), rank=rank, world=world,
                                           reuse_buffer=reuse)
            x1, x2 = torch.randn(5, 16), torch.randn(5, 16)
            y1 = layer(x1)
            kept = y1.clone()
            y2 = layer(x2)
            if reuse:
                ok = ok and y1.data_ptr() == y2.data_ptr()          # documented aliasing
            else:
                ok = ok and torch.equal(y1, kept) and y1.data_ptr() != y2.data_ptr()
            w_q, scale, _ = full.quantize_weight(weight)
            expect = full.linear_forward(x2, _FakePrepared(w_q), scale, bias, out=torch.empty(5, 8))
            ok = ok and torch.allclose(unshard(y2, 1), expect, atol=1e-5)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_layer_result_ownership_two_ranks():
    """A second forward must not change the tensor the first one returned, unless the
    layer was built with reuse_buffer=True (then both calls return the same storage)."""
    world = 2
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_layer_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


class _RecordingBackend(_FakeBackend):
    """Reports the many-token kernel as available and records what the layer asks of it."""

    def __init__(self):
        self.calls = []

    def supports_absmax_out(self, *, m, k, channels):
        return True

    def linear_forward(self, x, prepared, weight_scale, bias, *, per_row=False, out=None, absmax_in=None,
                       absmax_out=None, out_copies=(), absmax_copies=(), copies_multicast=False):
        self.calls.append({"out_copies": list(out_copies), "absmax_copies": list(absmax_copies),
                           "multicast": bool(copies_multicast), "absmax_out": absmax_out})
        return super().linear_forward(x, prepared, weight_scale, bias, per_row=per_row, out=out)


class _FakeArena:
    """The addressing of PeerArena without symmetric memory: four 'ranks' with made-up bases."""

    def __init__(self, rank: int, world: int, multicast_base: int):
        from rns_llm_b200.parallel import PeerArena
        self.rank, self.world = rank, world
        self.buffer = torch.zeros(1 << 20, dtype=torch.uint8)
        self.peer_bases = [0x10_0000_0000 * (r + 1) for r in range(world)]
        self.multicast_base = multicast_base
        self.nbytes, self._offset, self.barriers = int(self.buffer.numel()), 0, 0
        self.alloc = PeerArena.alloc.__get__(self)
        self.peer_addresses = PeerArena.peer_addresses.__get__(self)

    def barrier(self):
        self.barriers += 1


def test_exchange_addresses_of_a_sharded_layer(monkeypatch):
    """Per-peer stores go to every OTHER rank's slot, starting with the right-hand neighbour;
    the multicast form hands the kernel ONE address inside the multicast mapping, and only for
    shards whose shape the row-wide multicast store covers."""
    import torch.cuda as cuda
    from rns_llm_b200.parallel import ABSMAX_PAD, ColumnShardedRNSLinear

    class _NoStream:
        cuda_stream = 0
    monkeypatch.setattr(cuda, "current_stream", lambda device=None: _NoStream())
    rank, world, m, k = 1, 4, 8, 32
    mc_base = 0x7f_0000_0000
    for local, multicast, expect_mc in ((128, True, True), (128, False, False), (64, True, False)):
        backend, arena = _RecordingBackend(), _FakeArena(rank, world, mc_base)
        layer = ColumnShardedRNSLinear(torch.randn(local, k).half(), None, backend=backend, moduli=(127, 126, 125, 121),
                                       rank=rank, world=world, peer_arena=arena, multicast=multicast)
        assert layer.multicast == multicast
        y = layer(torch.randn(m, k).half())
        assert y.shape == (world, m, local) and arena.barriers == 1
        call = backend.calls[-1]
        block = (m * local + ABSMAX_PAD) * 2                      # bytes of one rank's block (fp16)
        mine = rank * block                                       # first layer of the arena: offset 0
        assert call["multicast"] == expect_mc
        if expect_mc:
            assert call["out_copies"] == [mc_base + mine]
            assert call["absmax_copies"] == [mc_base + mine + m * local * 2]
        else:
            order = [2, 3, 0]                                     # neighbours of rank 1, wrapping round
            assert call["out_copies"] == [arena.peer_bases[r] + mine for r in order]
            assert call["absmax_copies"] == [arena.peer_bases[r] + mine + m * local * 2 for r in order]
    # an arena without a multicast mapping: the flag is dropped at construction
    plain = ColumnShardedRNSLinear(torch.randn(128, k).half(), None, backend=_RecordingBackend(),
                                   moduli=(127, 126, 125, 121), rank=rank, world=world,
                                   peer_arena=_FakeArena(rank, world, 0), multicast=True)
    assert plain.multicast is False
