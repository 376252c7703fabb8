"""Output-row sharding of compressed linear layers across the GPUs of one node.

The reference has no multi-GPU code.  The format shards naturally by output rows: every
(chunk, row) record is decodable on its own and the tables are per layer, so rank ``r`` of ``P``
keeps rows ``[r*M/P, (r+1)*M/P)`` of ``rem`` and ``offsets`` plus the matching spans of ``exp``
(re-based so that the shard is again a self-contained weight in storage order), computes its slice
of the output with the same fused kernel, and the slices are concatenated with an all-gather of
the ``[batch, M/P]`` activations.  Only activations cross NVLink; weights never move.

Two ways to concatenate: :class:`RowShardedLinear` calls an all-gather (NCCL on GPUs, gloo on CPU);
:class:`PeerRowShardedLinear` lets the fused kernel store its results straight into every rank's output
buffer over NVLink (peer-mapped symmetric memory, counters instead of a collective), which removes
the collective's latency from every layer of a decode step.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor, nn

from . import ops
from .functional import FUSED_MAX_ROWS, ANSWeight, CompressedLinear, FusedCompressedLinear, HuffmanWeight

__all__ = ["row_range", "shard_rows", "RowShardedLinear", "shard_model_linears", "PeerArena", "PeerRowShardedLinear"]


def row_range(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced row range of ``rank`` (sizes differ by at most one row)."""
    return rows * rank // world, rows * (rank + 1) // world


def shard_rows(weight: HuffmanWeight, rank: int, world: int) -> HuffmanWeight:
    """The rows of ``weight`` owned by ``rank``, as a new weight of the same class sharing the tables.

    Works on any device; no re-encoding.  Each chunk's records of the row range form one
    contiguous span of ``exp`` (records are stored chunk-major, rows ascending); the spans are
    concatenated, each followed by the 64 padding words a decoder may look at, and the offsets
    are re-based onto the new buffer.
    """
    rem, exp, offsets = weight.rem, weight.exp, weight.offsets
    if rem.dim() == 2:
        rem = rem[None]
    if offsets.dim() == 1:
        offsets = offsets[None]
    S, M, _ = rem.shape
    lo, hi = row_range(M, rank, world)
    assert hi > lo, "a rank would own no rows"
    off64 = offsets.to(torch.int64)
    flat = off64.flatten()
    total = exp.numel()
    pieces: List[Tensor] = []
    new_off = torch.empty(S, hi - lo, dtype=torch.int64, device=offsets.device)
    at = 0
    pad = torch.zeros(64, dtype=exp.dtype, device=exp.device)
    for k in range(S):
        start = int(off64[k, lo])
        nxt = k * M + hi
        end = int(flat[nxt]) if nxt < S * M else total
        span = exp[start:end]
        # a span that ends at a slab boundary already carries its padding row; one more is harmless
        pieces += [span, pad]
        new_off[k] = off64[k, lo:hi] - start + at
        at += span.numel() + 64
    kwargs = {"rem": rem[:, lo:hi].contiguous(), "exp": torch.cat(pieces), "offsets": new_off.to(torch.int32)}
    if isinstance(weight, ANSWeight):
        return ANSWeight(LUT=weight.LUT, **kwargs)
    return HuffmanWeight(LUT1=weight.LUT1, LUT2=weight.LUT2, LUT3=weight.LUT3, LUT4=weight.LUT4,
                         code_lengths=weight.code_lengths, **kwargs)


class RowShardedLinear(nn.Module):
    """A :class:`CompressedLinear` holding only this rank's output rows; ``forward`` returns the full output.

    The local slice is computed by the fused kernel (or decode + GEMM above 8 rows) and the slices
    of all ranks are gathered along the feature dimension.  Row counts must be equal across ranks
    (``out_features % world == 0``) so that a single ``all_gather_into_tensor`` suffices.
    """

    def __init__(self, local: CompressedLinear, out_features: int, group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.local = local
        self.out_features = out_features
        self.group = group

    @classmethod
    def from_full(cls, full: CompressedLinear, rank: int, world: int, group=None) -> "RowShardedLinear":
        M = full.out_features
        assert M % world == 0, "out_features must divide evenly across ranks"
        lo, hi = row_range(M, rank, world)
        bias = None if full.bias is None else nn.Parameter(full.bias.detach()[lo:hi].clone(), requires_grad=False)
        return cls(CompressedLinear(shard_rows(full.weight, rank, world), bias), M, group)

    def forward(self, input: Tensor) -> Tensor:
        y = self.local(input)
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if world == 1:
            return y
        lead = y.shape[:-1]
        flat = y.reshape(-1, y.shape[-1]).contiguous()
        gathered = torch.empty(world, *flat.shape, dtype=flat.dtype, device=flat.device)
        if flat.is_cuda:
            dist.all_gather_into_tensor(gathered, flat, group=self.group)
        else:                                   # CPU process groups (tests): list form
            dist.all_gather(list(gathered.unbind(0)), flat, group=self.group)
        return gathered.permute(1, 0, 2).reshape(*lead, self.out_features)


class PeerArena:
    """Peer-mapped memory for the outputs of :class:`PeerRowShardedLinear` layers: one allocation per rank,
    mapped into every rank of the group, holding for each registered layer two counter words and the full
    output ``[8, out_features]``.

    Usage: ``slot = arena.add(out_features)`` for every layer (same order on every rank), then
    ``arena.commit()`` once (a collective call), then ``arena.output(slot)`` / ``arena.peers(slot)``.
    A single-rank arena (``group=None`` without an initialised process group, or ``world == 1``) uses
    plain device memory, so the same kernels run on one GPU.
    """

    HEADER = 256          # bytes in front of a layer's output: ready counter at +0, done counter at +128

    def __init__(self, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._sizes: List[int] = []
        self._offsets: List[int] = []
        self._total = 0
        self.buffer: Optional[Tensor] = None
        self.base_ptrs: List[int] = []
        self.launches: Optional[Tensor] = None

    def __deepcopy__(self, memo):
        return self           # shared, peer-mapped state: copies of a model (e.g. its graphed twin) use the same arena

    def add(self, out_features: int) -> int:
        assert self.buffer is None, "the arena is already committed"
        nbytes = self.HEADER + ((FUSED_MAX_ROWS * out_features * 2 + 255) // 256) * 256
        self._sizes.append(out_features)
        self._offsets.append(self._total)
        self._total += nbytes
        return len(self._sizes) - 1

    def commit(self) -> None:
        assert self.buffer is None and self._total > 0
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buffer = symm_mem.empty(self._total, dtype=torch.uint8, device=self.device)
            self.buffer.zero_()
            handle = symm_mem.rendezvous(self.buffer, self.group if self.group is not None else dist.group.WORLD)
            self.base_ptrs = [int(p) for p in handle.buffer_ptrs]
            self._handle = handle
        else:
            self.buffer = torch.zeros(self._total, dtype=torch.uint8, device=self.device)
            self.base_ptrs = [self.buffer.data_ptr()]
        self.launches = torch.zeros(2 * len(self._sizes), dtype=torch.int32, device=self.device)   # per layer: launches, block arrivals
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)          # every rank's counters are zero before anybody launches

    def output(self, slot: int) -> Tensor:
        """This rank's full-output buffer of the layer, ``[8, out_features]`` BF16 (a view of the arena)."""
        start = self._offsets[slot] + self.HEADER
        m = self._sizes[slot]
        return self.buffer[start:start + FUSED_MAX_ROWS * m * 2].view(torch.bfloat16).view(FUSED_MAX_ROWS, m)

    def peers(self, slot: int) -> Tensor:
        """The pointer table the exchange operators take (CPU int64, ``3 * world + 1`` entries)."""
        off = self._offsets[slot]
        y = [b + off + self.HEADER for b in self.base_ptrs]
        ready = [b + off for b in self.base_ptrs]
        done = [b + off + 128 for b in self.base_ptrs]
        return torch.tensor(y + ready + done + [self.launches.data_ptr() + 8 * slot], dtype=torch.int64)


class PeerRowShardedLinear(nn.Module):
    """Like :class:`RowShardedLinear`, but up to 8 rows of input take the exchange kernel: every rank's
    fused GEMV writes its slice of the output into all ranks' buffers and returns when the whole output
    has arrived, so no collective follows.  More than 8 rows fall back to the all-gather path.

    The returned tensor is a view of the arena: it is overwritten by the next call of this layer, and
    its consumers must run on the same stream (the kernel tells the peers that the buffer may be
    rewritten only after everything queued before it has finished).  All ranks must call the layers in
    the same order.
    """

    def __init__(self, local: CompressedLinear, out_features: int, arena: PeerArena, group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.local = local
        self.out_features = out_features
        self.arena = arena
        self.group = group
        self.slot = arena.add(out_features)
        self.row_base = row_range(out_features, arena.rank, arena.world)[0]
        self._peers: Optional[Tensor] = None
        self._fallback = RowShardedLinear(local, out_features, group)

    @classmethod
    def from_full(cls, full: CompressedLinear, arena: PeerArena, group=None) -> "PeerRowShardedLinear":
        M = full.out_features
        assert M % arena.world == 0, "out_features must divide evenly across ranks"
        lo, hi = row_range(M, arena.rank, arena.world)
        bias = None if full.bias is None else nn.Parameter(full.bias.detach()[lo:hi].clone(), requires_grad=False)
        return cls(CompressedLinear(shard_rows(full.weight, arena.rank, arena.world), bias), M, arena, group)

    def forward(self, input: Tensor) -> Tensor:
        lead = input.shape[:-1]
        x = input.reshape(-1, input.shape[-1])
        rows = x.shape[0]
        if rows > FUSED_MAX_ROWS or self.local.bias is not None:
            return self._fallback(input)
        if self._peers is None:
            assert self.arena.buffer is not None, "PeerArena.commit() has not been called"
            self._peers = self.arena.peers(self.slot)
        w = self.local.weight
        x = x.contiguous()
        if isinstance(w, ANSWeight):
            ops.gemv_bf16_ans_exchange(w.rem, w.exp, x, w.offsets, w.LUT, self._peers, self.arena.rank, self.row_base, self.out_features)
        else:
            ops.gemv_bf16_huffman_exchange(w.rem, w.exp, x, w.offsets, w.prepared(), self._peers, self.arena.rank, self.row_base,
                                           self.out_features)
        out = self.arena.output(self.slot)
        # rows of the buffer are laid out for `rows` rows of input: [rows, out_features] contiguous from its start
        return out.view(-1)[: rows * self.out_features].view(*lead, self.out_features)


def shard_model_linears(model: nn.Module, rank: int, world: int, group=None, arena: Optional[PeerArena] = None) -> None:
    """Replace every :class:`CompressedLinear` whose row count divides by ``world`` with its row shard
    (an all-gather layer, or an exchange layer when a :class:`PeerArena` is given; commit the arena afterwards)."""
    for name, mod in list(model.named_modules()):
        if isinstance(mod, CompressedLinear) and mod.out_features % world == 0:
            if arena is not None:
                model.set_submodule(name, PeerRowShardedLinear.from_full(mod, arena, group))
            else:
                model.set_submodule(name, RowShardedLinear.from_full(mod, rank, world, group))
        elif isinstance(mod, FusedCompressedLinear) and mod.sharded is None and mod.weight.shape[0] % world == 0:
            # stacked siblings: shard the stacked rows; the slices the siblings return stay views of the full output
            full = CompressedLinear(mod.weight, mod.bias)
            if arena is not None:
                mod.sharded = PeerRowShardedLinear.from_full(full, arena, group)
            else:
                mod.sharded = RowShardedLinear.from_full(full, rank, world, group)
            mod.weight = mod.sharded.local.weight          # keep only this rank's rows
            mod.bias = None
