"""Row sharding of compressed weights (host logic, CPU) and the all-gather wrapper under a
two-process gloo group."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from _util import ROOT, bits_of, make_input, make_weight, tables_for

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402


def _compressed(algo, M, K, S, seed):
    from bf16_huffman_infer_b200 import ANSWeight, HuffmanWeight
    W = make_weight(M, K, seed)
    Wb = bits_of(W)
    tabs = tables_for(algo, oracle.histogram(Wb))
    rem, exp, offsets, _ = oracle.compress(Wb, algo, tabs, split_k=S)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    if algo == "huffman":
        w = HuffmanWeight(t(rem), t(exp), t(offsets), *[t(tabs[k]) for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")])
    else:
        w = ANSWeight(t(rem), t(exp), t(offsets), t(tabs["LUT"]))
    return W, Wb, tabs, w


@pytest.mark.parametrize("algo", ["huffman", "ans"])
@pytest.mark.parametrize("M,K,S,world", [(256, 512, 1, 2), (384, 768, 2, 3), (4224, 128, 1, 4), (8448, 128, 1, 2), (130, 384, 3, 2)])
def test_shard_rows_decodes_to_the_row_slice(algo, M, K, S, world):
    from bf16_huffman_infer_b200.tensor_parallel import row_range, shard_rows
    W, Wb, tabs, w = _compressed(algo, M, K, S, 3)
    covered = 0
    for rank in range(world):
        lo, hi = row_range(M, rank, world)
        sh = shard_rows(w, rank, world)
        assert sh.rem.shape == (S, hi - lo, K // S) and sh.offsets.shape == (S, hi - lo)
        assert type(sh) is type(w)
        # storage order is preserved: offsets ascend and every record is a whole number of 64-word rows
        flat = sh.offsets.flatten().to(torch.int64)
        gaps = torch.diff(torch.cat([flat, torch.tensor([sh.exp.numel()])]))
        assert (gaps > 0).all() and (gaps % 64 == 0).all()
        back = oracle.decode(algo, sh.rem.numpy(), sh.exp.numpy(), sh.offsets.numpy(), tabs)
        assert (back == Wb[lo:hi]).all()
        covered += hi - lo
    assert covered == M


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _DenseLocal(nn.Module):
    """Stands in for the fused kernel on CPU: the local rows of a dense weight."""

    def __init__(self, w):
        super().__init__()
        self.w = w

    def forward(self, x):
        return x @ self.w.T


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bf16_huffman_infer_b200.tensor_parallel import RowShardedLinear, row_range
        torch.manual_seed(0)
        W = torch.randn(64, 32)
        x = torch.randn(2, 3, 32)
        lo, hi = row_range(64, rank, world)
        layer = RowShardedLinear(_DenseLocal(W[lo:hi]), 64)
        y = layer(x)
        ok = torch.allclose(y, x @ W.T, atol=1e-6) and y.shape == (2, 3, 64)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_row_sharded_linear_gathers_under_gloo():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
