"""The row-sharded GEMV whose epilogue is the all-gather (exchange kernels), on ONE GPU.

Two ranks are played one after the other on the same device: each "rank" stores its slice of the
output into both ranks' buffers.  Kernels that wait for one another must never be separate launches
on one GPU, so the counters a launch would wait for are credited by the host beforehand (the peer's
"ready" and its "done" signal); no launch then waits for another.  The multi-process form
over NVLink is covered by test_gpu_exchange_multi.py on boxes with two GPUs.
"""
import ctypes as C
import os
import sys

import pytest
import torch

from _util import ROOT, Abi, bits_of, make_input, make_weight, rel_err, tables_for, to_device

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2


class Exchange(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("row_base", C.c_int), ("M_total", C.c_int),
                ("y", C.c_void_p * 8), ("ready", C.c_void_p * 8), ("done", C.c_void_p * 8), ("launches", C.c_void_p)]


@pytest.fixture(scope="module")
def abi():
    return Abi()


def _status(abi):
    s = C.c_int(-1)
    abi.check(abi.lib.bhi_debug_status(C.byref(s)))
    return s.value


def _shard(algo, M, K, S, seed, world):
    """Full layer on the host, one device dict per rank (rows split evenly), tables shared."""
    W = make_weight(M, K, seed)
    Wb = bits_of(W)
    tabs = tables_for(algo, oracle.histogram(Wb))
    keys = [k for k in tabs if k not in ("code_values", "freq", "cum")]
    shards = []
    for r in range(world):
        lo, hi = M * r // world, M * (r + 1) // world
        rem, exp, offsets, _ = oracle.compress(Wb[lo:hi], algo, tabs, split_k=S)
        shards.append(to_device(dict(rem=rem, exp=exp, offsets=offsets, **{k: tabs[k] for k in keys}), DEV))
    return Wb, shards


def _launch(abi, algo, w, x, ex):
    S, M, Nc = w["rem"].shape
    p = abi.p
    if algo == "huffman":
        rc = abi.lib.bhi_gemv_bf16_huffman_exchange(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(w["offsets"]),
                                                    p(abi.prepare(w)), S, M, Nc, x.shape[0], C.byref(ex), abi.stream())
    else:
        rc = abi.lib.bhi_gemv_bf16_ans_exchange(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(w["offsets"]),
                                                p(w["LUT"]), 8, S, M, Nc, x.shape[0], C.byref(ex), abi.stream())
    abi.check(rc)


@pytest.mark.parametrize("algo", ["huffman", "ans"])
@pytest.mark.parametrize("M,K,S,B", [(256, 1024, 2, 1), (512, 4096, 1, 3), (384, 512, 1, 8)])
def test_two_ranks_played_in_turn(abi, algo, M, K, S, B):
    world = 2
    Wb, shards = _shard(algo, M, K, S, 3, world)
    X = make_input(B, K, 5)
    x = X.to(DEV)
    ref = oracle.matvec(Wb, bits_of(X))
    y = [torch.zeros(8, M, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    counters = torch.zeros(world, 2, 32, dtype=torch.int32, device=DEV)      # [rank, ready/done, padded]
    launches = torch.zeros(world, 2, dtype=torch.int32, device=DEV)      # per rank: launch counter, block-arrival counter
    for call in range(3):                                                    # the counters keep counting across calls
        for r in range(world):
            ex = Exchange(world=world, rank=r, row_base=M * r // world, M_total=M)
            for q in range(world):
                ex.y[q] = y[q].data_ptr()
                ex.ready[q] = counters[q, 0].data_ptr()
                ex.done[q] = counters[q, 1].data_ptr()
            ex.launches = launches[r].data_ptr()
            # what the other rank would have signalled by now on rank r's words
            if r == 0:
                counters[r, 0, 0] += 1
                counters[r, 1, 0] += 1
            _launch(abi, algo, shards[r], x, ex)
            torch.cuda.synchronize()
            if r == 0:
                # rank 1 really signals below: take the credit back out of rank 0's words first, so that
                # both end this call at exactly world * launch number
                counters[r, 0, 0] -= 1
                counters[r, 1, 0] -= 1
        assert _status(abi) == 0
        for q in range(world):
            got = y[q][:B].float().cpu().numpy()
            assert rel_err(got, ref) <= TOL, (call, q)
        assert counters[:, 0, 0].tolist() == [world * (call + 1)] * world
        assert counters[:, 1, 0].tolist() == [world * (call + 1)] * world
        assert launches[:, 0].tolist() == [call + 1] * world
        for t in y:
            t.zero_()


@pytest.mark.parametrize("algo", ["huffman", "ans"])
def test_single_rank_arena_matches_plain_layer(algo):
    """PeerRowShardedLinear with a one-rank arena: same kernel arithmetic as CompressedLinear, same bits."""
    from bf16_huffman_infer_b200 import ANSWeight, CompressedLinear, HuffmanWeight
    from bf16_huffman_infer_b200.tensor_parallel import PeerArena, PeerRowShardedLinear
    M, K = 512, 2048
    W = make_weight(M, K, 8)
    cls = HuffmanWeight if algo == "huffman" else ANSWeight
    lin = CompressedLinear(cls.compress(W), None).to(DEV)
    arena = PeerArena(torch.device(DEV))
    peer = PeerRowShardedLinear(lin, M, arena)
    arena.commit()
    for B in (1, 4, 8, 1):
        x = make_input(B, K, B).to(DEV)
        with torch.no_grad():
            a = lin(x)
            b = peer(x)
        assert b.shape == a.shape and torch.equal(a, b)
    with torch.no_grad():
        big = make_input(9, K, 9).to(DEV)
        assert torch.equal(peer(big), lin(big))                      # more than 8 rows: the ordinary path


def test_results_too_large_to_stage_take_the_direct_stores(abi):
    """Many rows per CTA at batch 8: the staged-result buffer would not fit, each row is stored by the lanes
    that hold it; same results as the plain GEMV."""
    M, K, B = 80000, 128, 8
    Wb, shards = _shard("ans", M, K, 1, 4, 1)
    X = make_input(B, K, 6)
    x = X.to(DEV)
    y = torch.zeros(8, M, dtype=torch.bfloat16, device=DEV)
    counters = torch.zeros(2, 32, dtype=torch.int32, device=DEV)
    launches = torch.zeros(2, dtype=torch.int32, device=DEV)
    ex = Exchange(world=1, rank=0, row_base=0, M_total=M)
    ex.y[0] = y.data_ptr()
    ex.ready[0] = counters[0].data_ptr()
    ex.done[0] = counters[1].data_ptr()
    ex.launches = launches.data_ptr()
    for _ in range(2):
        _launch(abi, "ans", shards[0], x, ex)
    torch.cuda.synchronize()
    assert _status(abi) == 0
    plain = abi.gemv("ans", shards[0], x)
    assert torch.equal(plain, y[:B])
    assert rel_err(y[:B].float().cpu().numpy(), oracle.matvec(Wb, bits_of(X))) <= TOL


def test_wait_on_a_missing_peer_runs_out(abi):
    """A peer that never signals: both bounded waits expire, the kernel ends, the status word says so and
    the context stays usable."""
    M, K = 128, 512
    Wb, shards = _shard("ans", M, K, 1, 1, 2)
    x = make_input(1, K, 2).to(DEV)
    y = [torch.zeros(8, M, dtype=torch.bfloat16, device=DEV) for _ in range(2)]
    counters = torch.zeros(2, 2, 32, dtype=torch.int32, device=DEV)
    launches = torch.zeros(2, dtype=torch.int32, device=DEV)
    ex = Exchange(world=2, rank=0, row_base=0, M_total=M)
    for q in range(2):
        ex.y[q] = y[q].data_ptr()
        ex.ready[q] = counters[q, 0].data_ptr()
        ex.done[q] = counters[q, 1].data_ptr()
    ex.launches = launches.data_ptr()
    _launch(abi, "ans", shards[0], x, ex)
    torch.cuda.synchronize()
    assert _status(abi) in (8, 9)
    assert _status(abi) == 0                                        # reading clears it
    # rank 0's own rows were still written everywhere
    ref = oracle.matvec(Wb[: M // 2], bits_of(x.cpu()))
    for q in range(2):
        assert rel_err(y[q][:1, : M // 2].float().cpu().numpy(), ref) <= TOL
    assert torch.cuda.is_available() and float(torch.ones(4, device=DEV).sum()) == 4.0


def test_exchange_rejects_bad_descriptors(abi):
    Wb, shards = _shard("ans", 128, 512, 1, 1, 1)
    x = make_input(1, 512, 2).to(DEV)
    ex = Exchange(world=9, rank=0, row_base=0, M_total=128)
    with pytest.raises(RuntimeError, match="world"):
        _launch(abi, "ans", shards[0], x, ex)
    ex = Exchange(world=1, rank=0, row_base=64, M_total=128)
    with pytest.raises(RuntimeError, match="rows outside"):
        _launch(abi, "ans", shards[0], x, ex)
