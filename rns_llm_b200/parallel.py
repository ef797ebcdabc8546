"""Column-sharded RNS linears: one process per GPU, weights split along the
output features, outputs exchanged with one NCCL all-gather per layer.

Every output column n of an RNS linear depends only on W[n,:], its scale and
bias, and on the (replicated) activation, so the layer splits along N with no
other communication: rank g quantises the full activation (cheap, and the
per-tensor scale needs all of it anyway), runs the fused GEMM on its
``N / world`` rows of the weight, and the fp16 shards are gathered.

``all_gather_into_tensor`` concatenates along dim 0, so G shards [M, N/G] arrive
as a [G, M, N/G] tensor.  The next sharded layer reads that layout directly
(the activation quantiser addresses element (m, c) as block c // (N/G), row m,
column c % (N/G)), so a layer stack never pays a transposing copy; ``unshard``
produces the ordinary [M, N] matrix when a caller needs it.

A layer also passes on the absmax of what it produced: every rank's GEMM epilogue
leaves max |y| of its shard in a word that travels at the end of the rank's block of
the gathered buffer, and the next sharded layer hands those G words to its quantiser,
which then skips its own pass over the activations (the reference recomputes the
per-tensor absmax in eager torch, src/rns_llm/layers/rns_linear.py:239-240).  Only a
tensor returned by ``forward`` itself carries the words; a view of part of it (one of
q, k, v) does not, because its absmax is another number.

Fused QKV is sharded inside each of q, k and v (rank g owns rows
[q_g; k_g; v_g]), so that the three projections of the gathered result are
again plain column blocks.

The reference has no multi-GPU path; the layer arithmetic is that of
``RNSLinear`` (src/rns_llm/layers/rns_linear.py:225-275 of the reference).
"""
from __future__ import annotations

from typing import Iterable, Sequence

import torch
import torch.distributed as dist
from torch import nn


def shard_rows(out_features: int, world: int, rank: int, groups: int = 1) -> list[slice]:
    """Row ranges of the full weight [N,K] owned by ``rank``: one contiguous
    range per group (``groups=3`` for a q|k|v-concatenated weight).  N must be
    divisible by ``groups * world``."""
    if out_features % (groups * world) != 0:
        raise ValueError(f"out_features={out_features} is not divisible by groups*world={groups * world}")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    per_group = out_features // groups
    per_rank = per_group // world
    return [slice(g * per_group + rank * per_rank, g * per_group + (rank + 1) * per_rank) for g in range(groups)]


def shard_tensor(full: torch.Tensor, world: int, rank: int, groups: int = 1) -> torch.Tensor:
    """Rows of ``full`` ([N,...]) owned by ``rank``, groups concatenated."""
    return torch.cat([full[s] for s in shard_rows(full.shape[0], world, rank, groups)], dim=0)


def unshard(gathered: torch.Tensor, groups: int = 1) -> torch.Tensor:
    """[G, M, N/G] (result of the all-gather) -> [M, N] in the column order of
    the unsharded layer."""
    world, m, local = gathered.shape
    per = local // groups
    # gathered[g, m, j*per + c] is column  j*(world*per) + g*per + c  of the full output
    return gathered.view(world, m, groups, per).permute(1, 2, 0, 3).reshape(m, groups * world * per)


ABSMAX_PAD = 8      # elements kept free behind each rank's block of a gathered buffer (>= 8 bytes, 16-byte multiple)


class PeerArena:
    """Symmetric memory for the gathered outputs of column-sharded layers: one buffer of the
    same size on every rank of the group, each rank's buffer mapped into every other rank
    (torch.distributed._symmetric_memory over CUDA peer access / NVLink).

    With it a sharded layer needs no all-gather: the GEMM epilogue stores every output tile
    into its slot of ALL ranks' buffers (plain peer stores, issued tile by tile while the
    GEMM runs), and after the launch the ranks only meet at a barrier.  Blocks are handed out
    in allocation order, which is the same on every rank, so a block sits at the same offset
    everywhere.  Construction is collective; when symmetric memory is not available here
    (no peer access, unsupported platform) it raises, and callers keep the NCCL all-gather.
    """

    def __init__(self, nbytes: int, device: torch.device, group=None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world - 1 > 7:
            raise ValueError("a peer arena serves at most 8 ranks")
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.peer_bases = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.peer_bases) != self.world or self.peer_bases[self.rank] != self.buffer.data_ptr():
            raise RuntimeError("symmetric memory returned an unexpected set of peer pointers")
        # NVLink multicast mapping of the same buffer (NVLS), 0 where the platform has none: a
        # store to it lands at the same offset on every rank.
        self.multicast_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self._offset = 0

    def alloc(self, nbytes: int) -> tuple[torch.Tensor, int]:
        """(local uint8 view, byte offset) of the next block; identical offsets on all ranks."""
        start = self._offset
        end = start + (int(nbytes) + 255) // 256 * 256
        if end > self.nbytes:
            raise RuntimeError(f"peer arena of {self.nbytes} bytes is full ({end} needed)")
        self._offset = end
        return self.buffer[start:start + int(nbytes)], start

    def peer_addresses(self, offset: int) -> list[int]:
        """Device address of byte ``offset`` in every OTHER rank's buffer, starting with the
        next rank and wrapping round: a kernel that stores to the copies in list order then
        aims at a different GPU on every rank at any moment, instead of all ranks writing
        into rank 0 first."""
        world = len(self.peer_bases)
        return [self.peer_bases[(self.rank + step) % world] + offset for step in range(1, world)]

    def barrier(self) -> None:
        """All ranks' stores issued before it (on the current stream) are visible to every
        rank after it; queued on the current stream, no host synchronisation."""
        self.handle.barrier(channel=0)


class GatheredActivation(torch.Tensor):
    """A gathered [G, M, N/G] output that knows where the G absmax words of its blocks
    are: ``absmax_words`` = (device address of rank 0's word, G, distance in 4-byte
    words).  Views and results of other operations are plain tensors again."""

    absmax_words: tuple[int, int, int] | None = None

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        # Anything computed from it (views included) is a plain tensor without the words.
        with torch._C.DisableTorchFunctionSubclass():
            result = func(*args, **(kwargs or {}))
        return result


def group_view(gathered: torch.Tensor, groups: int, index: int) -> torch.Tensor:
    """Group ``index`` (e.g. q, k or v) of a gathered [G, M, N/G] output as a
    [G, M, N/(G*groups)] view: itself a gathered activation of that group."""
    per = gathered.shape[2] // groups
    return gathered[:, :, index * per:(index + 1) * per]


class ColumnShardedRNSLinear(nn.Module):
    """The shard of an RNS linear that one rank owns.

    ``forward(x)`` takes the replicated activation, either [.., K] or a gathered
    [G, M, K/G] tensor from a previous sharded layer, and returns the gathered
    output [G, M, N/G] (``gather=True``) or the local shard [M, N/G].

    Exchange: one NCCL all-gather after the GEMM, or - with ``peer_arena`` - none: the GEMM
    epilogue stores each tile into every rank's buffer while it runs and the ranks meet at
    a barrier (many-token calls with a per-tensor scale; other calls fall back to the
    all-gather).  ``multicast=True`` makes those stores multicast stores through NVSwitch
    (one per 16 bytes instead of one per peer) where the arena has a multicast mapping, the
    outputs are two bytes wide and N/G is a multiple of 128.  A layer with a peer arena owns
    its output buffer (as ``reuse_buffer``).

    Ownership of the result: by default every call returns a freshly allocated
    tensor, as the reference's ``RNSLinear`` does.  ``out=`` writes into the
    caller's [G, M, N/G] buffer.  ``reuse_buffer=True`` (constructor) makes the
    layer keep ONE buffer per (M, dtype, stream) and return it from every call:
    the next forward with the same M on the same stream then overwrites the
    tensor the previous call returned - for layer stacks that consume each
    output before the layer runs again, not for callers that hold results.
    """

    def __init__(self, weight_shard: torch.Tensor, bias_shard: torch.Tensor | None, *, backend,
                 moduli: Iterable[int], rank: int, world: int, group=None, groups: int = 1,
                 activation_scale: str = "tensor", reuse_buffer: bool = False,
                 peer_arena: "PeerArena | None" = None, multicast: bool = False) -> None:
        super().__init__()
        self.reuse_buffer = bool(reuse_buffer) or peer_arena is not None
        self.peer_arena = peer_arena
        # One multimem.st through the arena's NVLink multicast mapping instead of a store per
        # peer (where the platform offers the mapping and the shard's shape allows it).
        self.multicast = bool(multicast) and peer_arena is not None and peer_arena.multicast_base != 0
        self._peer_blocks: dict[tuple[int, torch.dtype], tuple[torch.Tensor, int]] = {}
        if weight_shard.ndim != 2:
            raise ValueError("weight_shard must be [N/world, K]")
        if activation_scale not in ("tensor", "row"):
            raise ValueError("activation_scale must be 'tensor' or 'row'")
        self.backend = backend
        self.moduli = tuple(int(m) for m in moduli)
        self.rank, self.world, self.group, self.groups = int(rank), int(world), group, int(groups)
        self.local_features = int(weight_shard.shape[0])
        self.in_features = int(weight_shard.shape[1])
        self.out_features = self.local_features * self.world
        self.per_row = activation_scale == "row"
        w_q, scale, _ = backend.quantize_weight(weight_shard.contiguous())
        self.prepared = backend.prepare_weight_nk(w_q, self.moduli)
        if self.prepared.kernel != "tcgen05":
            raise ValueError("sharded layers need the tensor-core kernel (int8, K % 16 == 0, moduli >= 86)")
        self.weight_scale = scale
        self.bias = None if bias_shard is None else bias_shard.detach().float().contiguous()
        self._gather_buffers: dict[tuple[int, torch.dtype, int], torch.Tensor] = {}

    @classmethod
    def from_linear(cls, layer: nn.Linear, *, backend, moduli, rank: int, world: int, group=None,
                    groups: int = 1, activation_scale: str = "tensor") -> "ColumnShardedRNSLinear":
        weight = shard_tensor(layer.weight.detach(), world, rank, groups)
        bias = None if layer.bias is None else shard_tensor(layer.bias.detach(), world, rank, groups)
        return cls(weight, bias, backend=backend, moduli=moduli, rank=rank, world=world, group=group,
                   groups=groups, activation_scale=activation_scale)

    def _buffer(self, m: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        """Flat [G, M*N/G + ABSMAX_PAD] buffer: each rank's block is its [M, N/G] shard
        followed by a few spare elements, the first four bytes of which hold the shard's
        absmax word."""
        block = m * self.local_features + ABSMAX_PAD
        if not self.reuse_buffer:
            return torch.empty((self.world, block), dtype=dtype, device=device)
        stream = int(torch.cuda.current_stream(device).cuda_stream)
        key = (m, dtype, stream)
        buf = self._gather_buffers.get(key)
        if buf is None:
            buf = torch.empty((self.world, block), dtype=dtype, device=device)
            self._gather_buffers[key] = buf
        return buf

    def forward(self, x: torch.Tensor, *, gather: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
        """See the class docstring for who owns the returned tensor (fresh by default;
        the layer's own buffer, overwritten by the next call, with ``reuse_buffer``)."""
        if x.ndim == 3 and x.shape[0] * x.shape[2] == self.in_features and x.shape[2] != self.in_features:
            flat, m = x, int(x.shape[1])          # gathered activation [G, M, K/G]
        else:
            flat = x.reshape(-1, self.in_features)
            m = int(flat.shape[0])
        absmax_in = getattr(x, "absmax_words", None) if isinstance(x, GatheredActivation) else None
        if absmax_in is not None and self.per_row:
            absmax_in = None
        if out is not None:
            # Caller-owned [G, M, N/G] memory: no room for the absmax words.
            local = out[self.rank]
            self.backend.linear_forward(flat, self.prepared, self.weight_scale, self.bias,
                                        per_row=self.per_row, out=local, absmax_in=absmax_in)
            if gather and self.world > 1:
                dist.all_gather_into_tensor(out.view(self.world * m, self.local_features), local, group=self.group)
            return out if gather else local
        count = m * self.local_features
        report = (not self.per_row) and self.backend.supports_absmax_out(m=m, k=self.in_features,
                                                                         channels=len(self.moduli))
        use_peers = self.peer_arena is not None and report and self.world > 1 and gather
        if self.peer_arena is not None:
            buf, offset = self._peer_block(m, flat.dtype)
        else:
            buf, offset = self._buffer(m, flat.dtype, flat.device), 0
        gathered = buf[:, :count].view(self.world, m, self.local_features)      # stride(0) = count + pad
        local = gathered[self.rank]
        word = buf[self.rank, count:].data_ptr() if report else None
        out_copies: list[int] = []
        absmax_copies: list[int] = []
        use_mc = False
        if use_peers:
            size = buf.element_size()
            block = (count + ABSMAX_PAD) * size
            mine = offset + self.rank * block                      # my slot, at the same offset on every rank
            use_mc = (self.multicast and size == 2 and self.local_features % 128 == 0 and mine % 16 == 0)
            if use_mc:
                out_copies = [self.peer_arena.multicast_base + mine]
                absmax_copies = [self.peer_arena.multicast_base + mine + count * size]
            else:
                out_copies = self.peer_arena.peer_addresses(mine)
                absmax_copies = self.peer_arena.peer_addresses(mine + count * size)
        self.backend.linear_forward(flat, self.prepared, self.weight_scale, self.bias,
                                    per_row=self.per_row, out=local, absmax_in=absmax_in, absmax_out=word,
                                    out_copies=out_copies, absmax_copies=absmax_copies,
                                    **({"copies_multicast": True} if use_mc else {}))
        if not gather:
            return local
        if use_peers:
            self.peer_arena.barrier()
        elif self.world > 1:
            # In place: this rank's block (shard + absmax word) already sits at its slot.
            dist.all_gather_into_tensor(buf.view(-1), buf[self.rank], group=self.group)
        if not report:
            return gathered
        result = gathered.as_subclass(GatheredActivation)
        result.absmax_words = (buf[0, count:].data_ptr(), self.world,
                               (count + ABSMAX_PAD) * buf.element_size() // 4)
        return result

    def _peer_block(self, m: int, dtype: torch.dtype) -> tuple[torch.Tensor, int]:
        """This layer's [G, M*N/G + pad] buffer inside the peer arena (allocated on first use,
        in the same order on every rank) and its byte offset."""
        key = (m, dtype)
        hit = self._peer_blocks.get(key)
        if hit is None:
            block = m * self.local_features + ABSMAX_PAD
            raw, offset = self.peer_arena.alloc(self.world * block * dtype.itemsize)
            hit = (raw.view(dtype).view(self.world, block), offset)
            self._peer_blocks[key] = hit
        return hit


def sharded_qkv_from_linears(q_proj: nn.Linear, k_proj: nn.Linear, v_proj: nn.Linear, *, backend, moduli,
                             rank: int, world: int, group=None,
                             activation_scale: str = "tensor") -> ColumnShardedRNSLinear:
    """Rank-local shard of the fused q|k|v projection (rows [q_g; k_g; v_g])."""
    layers: Sequence[nn.Linear] = (q_proj, k_proj, v_proj)
    weight = torch.cat([shard_tensor(l.weight.detach(), world, rank) for l in layers], dim=0)
    bias = None
    if q_proj.bias is not None:
        bias = torch.cat([shard_tensor(l.bias.detach(), world, rank) for l in layers], dim=0)
    return ColumnShardedRNSLinear(weight, bias, backend=backend, moduli=moduli, rank=rank, world=world,
                                  group=group, groups=3, activation_scale=activation_scale)
