"""GPU parity of the fused decode + tensor-core product (up to 128 rows of X) through the C ABI.

The product accumulates in FP32 on the tensor cores over the whole row and rounds once to BF16;
the bound is the same as for the GEMV: max|y - y_ref| / rms(y_ref) <= 1e-2 (after the half-ulp
allowance of a BF16 output) against the oracle's exact product of the decoded weights.
"""
import ctypes
import os
import sys

import pytest
import torch

from _util import ROOT, Abi, bits_of, make_input, make_weight, rel_err, tables_for, to_device

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-2
DEV = "cuda:0"


@pytest.fixture(scope="module")
def abi():
    return Abi()


def _device_layer(algo, M, K, S, seed):
    W = make_weight(M, K, seed, 0.02)
    Wb = bits_of(W)
    tabs = tables_for(algo, oracle.histogram(Wb))
    rem, exp, offsets, _ = oracle.compress(Wb, algo, tabs, split_k=S)
    w = to_device(dict(rem=rem, exp=exp, offsets=offsets, **{k: v for k, v in tabs.items()
                                                          if k not in ("code_values", "freq", "cum")}), DEV)
    return Wb, w


def _status(abi):
    status = ctypes.c_int(-1)
    abi.check(abi.lib.bhi_debug_status(ctypes.byref(status)))
    return status.value


SHAPES = [
    # M, K, S, seed
    (128, 128, 1, 0), (128, 384, 3, 2), (256, 512, 1, 3),
    (130, 512, 1, 5),            # last set of rows is ragged
    (40, 1024, 2, 4),            # fewer rows than two sets
    (4224, 128, 1, 6),           # crosses a 4096-row slab; more sets than SMs
    (512, 4096, 1, 0), (128, 12288, 3, 0),
    (64, 16384, 1, 7),           # records too large for the ring: decoded from global memory
]


# the two fused tensor-core kernels: path 0 = records staged in shared memory while the batch leaves room for them (up to
# about 48 rows), streams in registers beyond; path 2 = streams in registers at every batch
@pytest.mark.parametrize("path", [0, 2], ids=["staged", "registers"])
@pytest.mark.parametrize("prepared", [False, True], ids=["tables", "prepared"])
@pytest.mark.parametrize("algo", ["huffman", "ans"])
@pytest.mark.parametrize("M,K,S,seed", SHAPES)
def test_linear_matches_oracle(abi, path, prepared, algo, M, K, S, seed):
    if prepared and algo == "ans":
        pytest.skip("prepared tables exist for the Huffman coder only")
    Wb, w = _device_layer(algo, M, K, S, seed)
    previous = abi.set_path(path)
    try:
        for B in (9, 16, 24, 33, 48, 64, 100, 128, 1):
            X = make_input(B, K, seed + B)
            y = abi.linear(algo, w, X.to(DEV), prepared=prepared).float().cpu().numpy()
            ref = oracle.matvec(Wb, bits_of(X))
            assert rel_err(y, ref) <= TOL, (B, rel_err(y, ref))
        assert _status(abi) == 0, "a bounded wait expired inside the kernel"
    finally:
        abi.set_path(previous)


@pytest.mark.parametrize("path", [0, 2], ids=["staged", "registers"])
@pytest.mark.parametrize("method", ["limit6", "escape"])
@pytest.mark.parametrize("M,K,S", [(200, 4736, 1), (96, 4736 * 4, 4), (4224, 384, 3)])
def test_linear_other_tables_and_odd_block_counts(abi, path, method, M, K, S):
    """Tables without unresolved windows take the branch-free loops; 37 blocks per chunk end on half a stage pair."""
    W = make_weight(M, K, 21, 0.02)
    Wb = bits_of(W)
    tabs = tables_for("huffman", oracle.histogram(Wb), method)
    rem, exp, offsets, _ = oracle.compress(Wb, "huffman", tabs, split_k=S)
    w = to_device(dict(rem=rem, exp=exp, offsets=offsets, **{k: v for k, v in tabs.items() if k != "code_values"}), DEV)
    previous = abi.set_path(path)
    try:
        for B in (12, 32, 72):
            X = make_input(B, K, B)
            y = abi.linear("huffman", w, X.to(DEV), prepared=True).float().cpu().numpy()
            assert rel_err(y, oracle.matvec(Wb, bits_of(X))) <= TOL, B
        assert _status(abi) == 0
    finally:
        abi.set_path(previous)


@pytest.mark.parametrize("algo", ["huffman", "ans"])
def test_linear_agrees_with_gemv_rows(abi, algo):
    """The same X rows through the GEMV (8 at a time) and through the tensor-core product."""
    M, K, S = 384, 4096, 1
    Wb, w = _device_layer(algo, M, K, S, 11)
    X = make_input(24, K, 12).to(DEV)
    y = abi.linear(algo, w, X).float()
    parts = torch.cat([abi.gemv(algo, w, X[i:i + 8].contiguous()).float() for i in range(0, 24, 8)])
    scale = parts.pow(2).mean().sqrt().item()
    # both are BF16 roundings of FP32 sums in different orders: within one BF16 ulp of each other
    assert (y - parts).abs().max().item() <= 2 ** -7 * parts.abs().max().item() + 1e-3 * scale
    assert _status(abi) == 0


def test_linear_rejects_bad_arguments(abi):
    Wb, w = _device_layer("ans", 128, 128, 1, 0)
    X = make_input(129, 128, 0).to(DEV)
    with pytest.raises(RuntimeError, match="batch"):
        abi.linear("ans", w, X)
    X = make_input(17, 128, 0).to(DEV)
    flat = torch.empty(17 * 128 + 8, dtype=torch.bfloat16, device=DEV)
    off = flat[4:4 + 17 * 128].view(17, 128)     # 8-byte aligned only
    off.copy_(X)
    if off.data_ptr() % 16 != 0:
        with pytest.raises(RuntimeError, match="aligned"):
            abi.linear("ans", w, off)
