"""Output-row sharding of compressed linear layers across the GPUs of one node.

The reference has no multi-GPU code.  The format shards naturally by output rows: every
(chunk, row) record is decodable on its own and the tables are per layer, so rank ``r`` of ``P``
keeps rows ``[r*M/P, (r+1)*M/P)`` of ``rem`` and ``offsets`` plus the matching spans of ``exp``
(re-based so that the shard is again a self-contained weight in storage order), computes its slice
of the output with the same fused kernel, and the slices are concatenated with an all-gather of
the ``[batch, M/P]`` activations.  Only activations cross NVLink; weights never move.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor, nn

from .functional import ANSWeight, CompressedLinear, HuffmanWeight

__all__ = ["row_range", "shard_rows", "RowShardedLinear", "shard_model_linears"]


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


def shard_model_linears(model: nn.Module, rank: int, world: int, group=None) -> None:
    """Replace every :class:`CompressedLinear` whose row count divides by ``world`` with its row shard."""
    for name, mod in list(model.named_modules()):
        if isinstance(mod, CompressedLinear) and mod.out_features % world == 0:
            model.set_submodule(name, RowShardedLinear.from_full(mod, rank, world, group))
