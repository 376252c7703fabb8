"""GPU parity through the C ABI: encode, decode and fused GEMV against the CPU oracle.

Integer / byte results (encoded buffers, decoded weights) must be bit-exact.  GEMV outputs are
BF16 roundings of an FP32 accumulation; the bound is max|y - y_ref| / rms(y_ref) <= 1e-2 against an
exact (double) product of the decoded weights.
"""
import os
import sys

import numpy as np
import pytest
import torch

from _util import (GOLDEN, ROOT, Abi, ans_tables, bits_of, make_input, make_weight, rel_err, tables_for, to_device)

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-2
DEV = "cuda:0"


@pytest.fixture(scope="module")
def abi():
    return Abi()


def _layer(algo, M, K, S, seed, std=0.02):
    W = make_weight(M, K, seed, std)
    Wb = bits_of(W)
    tabs = tables_for(algo, oracle.histogram(Wb))
    rem, exp, offsets, L = oracle.compress(Wb, algo, tabs, split_k=S)
    return W, Wb, tabs, rem, exp, offsets, L


SHAPES = [
    # M, K, S, seed
    (128, 128, 1, 0), (128, 256, 2, 1), (128, 384, 3, 2), (256, 512, 1, 3), (384, 1024, 2, 4),
    (130, 512, 1, 5),            # row count that is not a multiple of 128
    (4224, 128, 1, 6),           # crosses a 4096-row slab
    (512, 4096, 1, 0), (128, 12288, 3, 0), (128, 4736 * 4, 4, 1),
]


# kernel variants of the fused product: (kernel path, warps of the four-row kernel, prepared tables)
VARIANTS = {"auto": (0, 0, False), "auto-prepared": (0, 0, True), "generic": (1, 0, False),
            "rowwarp": (2, 0, False), "rowwarp-prepared": (2, 0, True),
            "quad32": (0, 32, False), "quad32-prepared": (0, 32, True), "quad16": (0, 16, False), "quad16-prepared": (0, 16, True)}
PATHS = [(0, 0), (0, 32), (0, 16), (2, 0), (1, 0)]


class use_path:
    """Selects a kernel path (and the warp count of the four-row kernel) for the duration of a block."""

    def __init__(self, abi, path, warps=0):
        self.abi, self.path, self.warps = abi, path, warps

    def __enter__(self):
        self.prev = self.abi.set_path(self.path)
        self.prev_warps = self.abi.set_quad_warps(self.warps)

    def __exit__(self, *exc):
        self.abi.set_path(self.prev)
        self.abi.set_quad_warps(self.prev_warps)


@pytest.mark.parametrize("variant", list(VARIANTS))
@pytest.mark.parametrize("algo", ["huffman", "ans"])
@pytest.mark.parametrize("M,K,S,seed", SHAPES)
def test_decode_and_gemv_match_oracle(abi, variant, algo, M, K, S, seed):
    path, warps, prepared = VARIANTS[variant]
    if prepared and algo == "ans":
        pytest.skip("prepared tables exist for the Huffman coder only")
    W, Wb, tabs, rem, exp, offsets, _ = _layer(algo, M, K, S, seed)
    w = to_device(dict(rem=rem, exp=exp, offsets=offsets, **{k: v for k, v in tabs.items()
                                                          if k not in ("code_values", "freq", "cum")}), DEV)
    with use_path(abi, path, warps):
        dense = abi.decode(algo, w, prepared=prepared)
        torch.cuda.synchronize()
        assert (bits_of(dense.cpu()) == Wb).all(), "decoded weight is not bit-exact"
        for B in (1, 2, 3, 4, 5, 6, 7, 8):
            X = make_input(B, K, seed)
            y = abi.gemv(algo, w, X.to(DEV), prepared=prepared).float().cpu().numpy()
            ref = oracle.matvec(Wb, bits_of(X))
            assert rel_err(y, ref) <= TOL, (B, rel_err(y, ref))
        status = __import__("ctypes").c_int(-1)
        abi.check(abi.lib.bhi_debug_status(__import__("ctypes").byref(status)))
        assert status.value == 0, "a bounded wait expired inside a staged kernel"


@pytest.mark.parametrize("algo", ["huffman", "ans"])
@pytest.mark.parametrize("M,K,S,seed", [(128, 256, 2, 1), (384, 1024, 1, 4), (4224, 128, 1, 6), (256, 4096, 1, 2),
                                        (128, 12288, 3, 0)])
def test_encoder_bytes_match_oracle(abi, algo, M, K, S, seed):
    W, Wb, tabs, rem, exp, offsets, L = _layer(algo, M, K, S, seed)
    g_rem, g_exp, g_off, g_rows = abi.encode(algo, W.to(DEV), S, tabs)
    assert (g_rows.cpu().numpy() == L).all()
    assert (g_off.cpu().numpy() == offsets).all()
    assert (g_rem.cpu().numpy() == rem).all()
    assert g_exp.numel() == exp.size and (g_exp.cpu().numpy() == exp).all()


@pytest.mark.parametrize("bits", [9, 10, 11, 12])
@pytest.mark.parametrize("M,K,S,seed", [(128, 256, 2, 1), (384, 1024, 1, 4), (4224, 128, 1, 6), (512, 4096, 1, 0),
                                        (128, 12288, 3, 0)])
def test_finer_ans_models(abi, bits, M, K, S, seed):
    """rANS with 9..12 probability bits (table of 2^bits words): encoder bytes, decoded weight and the fused product on
    every kernel path against the oracle run at the same precision."""
    W = make_weight(M, K, seed)
    Wb = bits_of(W)
    tabs = ans_tables(oracle.histogram(Wb), precision=bits)[0]
    rem, exp, offsets, L = oracle.compress(Wb, "ans", tabs, split_k=S)
    g_rem, g_exp, g_off, g_rows = abi.encode("ans", W.to(DEV), S, tabs)
    assert (g_rows.cpu().numpy() == L).all() and (g_off.cpu().numpy() == offsets).all()
    assert (g_rem.cpu().numpy() == rem).all()
    assert g_exp.numel() == exp.size and (g_exp.cpu().numpy() == exp).all()
    w = to_device(dict(rem=rem, exp=exp, offsets=offsets, LUT=tabs["LUT"]), DEV)
    for path, warps in PATHS:
        with use_path(abi, path, warps):
            assert (bits_of(abi.decode("ans", w).cpu()) == Wb).all(), "decoded weight is not bit-exact"
            for B in (1, 3, 8):
                X = make_input(B, K, seed)
                y = abi.gemv("ans", w, X.to(DEV)).float().cpu().numpy()
                assert rel_err(y, oracle.matvec(Wb, bits_of(X))) <= TOL, (path, warps, B)
    X = make_input(24, K, seed + 1)
    y = abi.linear("ans", w, X.to(DEV)).float().cpu().numpy()
    assert rel_err(y, oracle.matvec(Wb, bits_of(X))) <= TOL


def test_pathological_tables_long_codes(abi):
    """A wide exponent spread (std 1 weights scaled per row) gives codes beyond 16 bits: the third and
    fourth byte tables must work in both paths."""
    g = torch.Generator().manual_seed(9)
    W = (torch.randn(256, 1024, generator=g) * torch.logspace(-12, 4, 256)[:, None]).to(torch.bfloat16)
    Wb = bits_of(W)
    tabs = tables_for("huffman", oracle.histogram(Wb))
    assert int(tabs["code_lengths"].max()) > 16
    rem, exp, offsets, _ = oracle.compress(Wb, "huffman", tabs, split_k=1)
    w = to_device(dict(rem=rem, exp=exp, offsets=offsets, **{k: tabs[k] for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")}), DEV)
    X = make_input(2, 1024, 9)
    ref = oracle.matvec(Wb, bits_of(X))
    for path, warps in PATHS:
        with use_path(abi, path, warps):
            assert (bits_of(abi.decode("huffman", w).cpu()) == Wb).all()
            assert (bits_of(abi.decode("huffman", w, prepared=True).cpu()) == Wb).all()
            for prepared in (True, False):
                y = abi.gemv("huffman", w, X.to(DEV), prepared=prepared).float().cpu().numpy()
                assert rel_err(y, ref) <= TOL, (path, warps, prepared)


@pytest.mark.parametrize("method", ["escape", "limit6", "limit8"])
@pytest.mark.parametrize("M,K,S,seed", [(384, 1024, 2, 4), (512, 4096, 1, 0), (128, 12288, 3, 0)])
def test_own_table_builders_on_every_path(abi, method, M, K, S, seed):
    """Tables from the builders the reference does not have (escape-byte code, length-limited codes): device
    encoder bytes equal the oracle's, all decode paths are bit-exact, GEMV and the tensor-core product stay
    within tolerance.  With limit6 no 12-bit window is left unresolved, which selects the fused kernel's
    loop without the per-step test."""
    W = make_weight(M, K, seed)
    Wb = bits_of(W)
    tabs = tables_for("huffman", oracle.histogram(Wb), method=method)
    assert int(tabs["code_lengths"].max()) <= {"escape": 16, "limit6": 6, "limit8": 8}[method]
    rem, exp, offsets, L = oracle.compress(Wb, "huffman", tabs, split_k=S)
    g_rem, g_exp, g_off, g_rows = abi.encode("huffman", W.to(DEV), S, tabs)
    assert (g_rows.cpu().numpy() == L).all() and (g_off.cpu().numpy() == offsets).all()
    assert (g_rem.cpu().numpy() == rem).all() and (g_exp.cpu().numpy() == exp).all()
    w = to_device(dict(rem=rem, exp=exp, offsets=offsets, **{k: tabs[k] for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")}), DEV)
    X = make_input(8, K, seed)
    ref = oracle.matvec(Wb, bits_of(X))
    for path, warps in PATHS:
        with use_path(abi, path, warps):
            assert (bits_of(abi.decode("huffman", w).cpu()) == Wb).all()
            assert (bits_of(abi.decode("huffman", w, prepared=True).cpu()) == Wb).all()
            for B in (1, 5, 8):
                y = abi.gemv("huffman", w, X[:B].to(DEV), prepared=True).float().cpu().numpy()
                assert rel_err(y, ref[:B]) <= TOL, (path, warps, B)
    X = make_input(24, K, seed + 1)
    y = abi.linear("huffman", w, X.to(DEV), prepared=True).float().cpu().numpy()
    assert rel_err(y, oracle.matvec(Wb, bits_of(X))) <= TOL


def test_argument_errors_are_reported(abi):
    import ctypes as C
    z = torch.zeros(64, dtype=torch.int32, device=DEV)
    rc = abi.lib.bhi_gemv_bf16_ans(abi.p(z), abi.p(z), C.c_int64(64), abi.p(z), abi.p(z), abi.p(z), abi.p(z),
                                   8, 1, 128, 100, 1, abi.stream())
    assert rc == 1 and b"multiple of 128" in abi.lib.bhi_last_error()
    rc = abi.lib.bhi_gemv_bf16_ans(abi.p(z), abi.p(z), C.c_int64(64), abi.p(z), abi.p(z), abi.p(z), abi.p(z),
                                   8, 1, 128, 128, 9, abi.stream())
    assert rc == 1 and b"batch" in abi.lib.bhi_last_error()
    rc = abi.lib.bhi_gemv_bf16_ans(abi.p(z), abi.p(z), C.c_int64(64), abi.p(z), abi.p(z), abi.p(z), abi.p(z),
                                   13, 1, 128, 128, 1, abi.stream())
    assert rc == 1 and b"precision" in abi.lib.bhi_last_error()


REF_LAYOUT = sorted(f for f in os.listdir(GOLDEN) if f.startswith("ref_layout_") and f.endswith(".npz"))


@pytest.mark.parametrize("name", REF_LAYOUT or ["missing"])
def test_reference_buffers_decode_and_multiply(abi, name):
    """Buffers written by the reference's own CUDA encoder: our kernels must decode them to the
    original bits, our encoder must reproduce them, and our GEMV must agree with the reference's."""
    if name == "missing":
        pytest.skip("reference GPU fixtures not generated yet")
    z = np.load(os.path.join(GOLDEN, name))
    algo = str(z["algo"])
    keys = ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths") if algo == "huffman" else ("LUT",)
    w = to_device({k: z[k] for k in ("rem", "exp", "offsets") + keys}, DEV)
    Wb = z["w_bits"]
    for path, warps in PATHS:
        with use_path(abi, path, warps):
            assert (bits_of(abi.decode(algo, w).cpu()) == Wb).all()
            X = torch.from_numpy(z["x_bits"].view(np.int16)).view(torch.bfloat16)
            for b in (1, 3, 8):
                y = abi.gemv(algo, w, X[:b].to(DEV)).float().cpu().numpy()
                assert rel_err(y, oracle.matvec(Wb, z["x_bits"][:b])) <= TOL
                assert rel_err(y, z[f"ref_y_b{b}"]) <= TOL      # the reference's own fused output
    tabs = tables_for(algo, oracle.histogram(Wb))
    W = torch.from_numpy(Wb.view(np.int16)).view(torch.bfloat16)
    g_rem, g_exp, g_off, _ = abi.encode(algo, W.to(DEV), z["rem"].shape[0], tabs)
    assert (g_rem.cpu().numpy() == z["rem"]).all()
    assert (g_off.cpu().numpy() == z["offsets"].reshape(g_off.shape)).all()
    assert (g_exp.cpu().numpy() == z["exp"]).all()
