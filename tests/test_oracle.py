"""The CPU oracle against the reference's golden vectors, and its own invariants."""
import os
import sys

import numpy as np
import pytest

from _util import GOLDEN, ROOT, ans_tables, bits_of, huffman_tables, load_json, make_input, make_weight, tables_for

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

TABLES = {r["name"]: r for r in load_json("ref_tables.json")}
STREAMS = load_json("ref_streams.json")


def _one_stream_layer(symbols):
    """A [1, 128*ceil(n/2)] weight whose stream 0 carries `symbols` (other streams: first symbol)."""
    n = len(symbols) + (len(symbols) & 1)
    sym = list(symbols) + [symbols[0]] * (n - len(symbols))
    K = 64 * n
    e = np.full((1, K), symbols[0], np.uint16)
    for s, v in enumerate(sym):
        e[0, (s >> 1) * 128 + (s & 1)] = v
    return (e << 7).astype(np.uint16), sym


@pytest.mark.parametrize("rec", STREAMS, ids=[f"{r['table']}-{len(r['symbols'])}" for r in STREAMS])
def test_huffman_stream_bits_match_reference(rec):
    """Words the oracle stores for a stream == the reference's bit string, LSB first."""
    tabs, _ = huffman_tables(TABLES[rec["table"]]["hist"])
    w, sym = _one_stream_layer(rec["symbols"])
    rem, exp, offsets, L = oracle.compress(w, "huffman", tabs, split_k=1)
    words = exp.view(np.uint32)[offsets[0, 0]::64][: L[0, 0]]
    got = sum(int(x) << (32 * i) for i, x in enumerate(words))
    bits = rec["huffman_bitstring"]
    ref = int(bits, 2) if bits else 0
    extra = sym[len(rec["symbols"]):]
    nbits = len(bits)
    for s in extra:                      # the padding symbol appended to make the count even
        ref |= int(tabs["code_values"][s]) << nbits
        nbits += int(tabs["code_lengths"][s])
    assert got == ref
    # pure-Python restatement agrees with the C one
    pw, have = oracle.py_huffman_encode_stream(sym, tabs["code_lengths"], tabs["code_values"])
    assert have == nbits and pw == [int(x) for x in words[: len(pw)]]
    assert oracle.py_huffman_decode_stream([int(x) for x in words], len(sym), tabs) == sym


@pytest.mark.parametrize("rec", STREAMS, ids=[f"{r['table']}-{len(r['symbols'])}" for r in STREAMS])
def test_ans_stream_words_match_reference(rec):
    """Oracle words == the reference's blob read from its end, without the leading zero word the
    reference's two-word flush may leave (the device coder flushes only non-zero state)."""
    tabs, _ = ans_tables(TABLES[rec["table"]]["hist"])
    sym = rec["symbols"]
    blob = bytes.fromhex(rec["ans_blob_hex"])
    ref = [int.from_bytes(blob[i:i + 4], "big") for i in range(0, len(blob), 4)][::-1]
    while len(ref) > 1 and ref[0] == 0:
        ref.pop(0)
    got = oracle.py_ans_encode_stream(sym, tabs["freq"], tabs["cum"])
    assert got == ref
    assert oracle.py_ans_decode_stream(got, len(sym), tabs["LUT"].view(np.uint32)) == sym
    out, lens = oracle.ans_encode_op(np.array([sym], np.uint8), tabs["freq"], tabs["cum"])
    assert lens[0] == len(ref) and out.view(np.uint32)[0, : lens[0]].tolist() == ref


FINER = load_json("ref_ans_precision.json")


@pytest.mark.parametrize("rec", FINER, ids=[f"{r['table']}-p{r['precision']}-{len(r['symbols'])}" for r in FINER])
def test_ans_finer_models_match_reference(rec):
    """10- and 12-bit probability models: scaled frequencies and stream words equal the reference class's."""
    bits = rec["precision"]
    tabs, enc = ans_tables(rec["hist"], precision=bits)
    assert enc.freq == rec["freq"] and enc.cum == rec["cum"] and tabs["LUT"].size == 1 << bits
    sym = rec["symbols"]
    blob = bytes.fromhex(rec["ans_blob_hex"])
    ref = [int.from_bytes(blob[i:i + 4], "big") for i in range(0, len(blob), 4)][::-1]
    while len(ref) > 1 and ref[0] == 0:
        ref.pop(0)
    got = oracle.py_ans_encode_stream(sym, tabs["freq"], tabs["cum"], bits=bits)
    assert got == ref
    assert oracle.py_ans_decode_stream(got, len(sym), tabs["LUT"].view(np.uint32), bits=bits) == sym
    out, lens = oracle.ans_encode_op(np.array([sym], np.uint8), tabs["freq"], tabs["cum"])
    assert lens[0] == len(ref) and out.view(np.uint32)[0, : lens[0]].tolist() == ref


@pytest.mark.parametrize("bits", [10, 12])
@pytest.mark.parametrize("M,K,S,seed", [(128, 512, 1, 0), (128, 384, 3, 3), (4100, 128, 1, 4)])
def test_oracle_roundtrip_finer_ans_models(bits, M, K, S, seed):
    W = bits_of(make_weight(M, K, seed))
    hist = oracle.histogram(W)
    tabs = ans_tables(hist, precision=bits)[0]
    rem, exp, offsets, _ = oracle.compress(W, "ans", tabs, split_k=S)
    assert (oracle.decode("ans", rem, exp, offsets, tabs) == W).all()
    x = bits_of(make_input(2, K, seed))
    assert np.allclose(oracle.gemv("ans", rem, exp, offsets, tabs, x), oracle.matvec(W, x), rtol=0, atol=1e-3)
    _, exp8, _, _ = oracle.compress(W, "ans", tables_for("ans", hist), split_k=S)
    assert K < 384 or exp.size <= exp8.size      # two-symbol streams are all flush: no model helps there


@pytest.mark.parametrize("algo", ["huffman", "ans"])
@pytest.mark.parametrize("M,K,S,seed", [(128, 512, 1, 0), (128, 512, 2, 1), (256, 1024, 1, 2), (128, 384, 3, 3),
                                        (4100, 128, 1, 4)])
def test_oracle_roundtrip_bit_exact(algo, M, K, S, seed):
    W = bits_of(make_weight(M, K, seed))
    tabs = tables_for(algo, oracle.histogram(W))
    rem, exp, offsets, L = oracle.compress(W, algo, tabs, split_k=S)
    assert rem.shape == (S, M, K // S) and offsets.shape == (S, M)
    # record placement: 64 * L words per record, one padding row after each slab of 4096 rows
    flat_off = offsets.reshape(-1).astype(np.int64)
    size = np.diff(np.append(flat_off, exp.size))
    pad = np.zeros((S, M), np.int64)
    pad[:, 4095::4096] = 64
    pad[:, M - 1] = 64
    assert (size == (64 * L.astype(np.int64) + pad).reshape(-1)).all()
    back = oracle.decode(algo, rem, exp, offsets, tabs)
    assert (back == W).all()


@pytest.mark.parametrize("M,K,S,seed", [(128, 512, 1, 0), (128, 384, 3, 3), (4100, 128, 1, 4)])
def test_oracle_roundtrip_with_escape_byte_tables(M, K, S, seed):
    """The format does not care which prefix code fills the tables: the alternative builder's code
    round-trips through the same encoder and decoder, and is never larger."""
    W = bits_of(make_weight(M, K, seed))
    hist = oracle.histogram(W)
    tabs = tables_for("huffman", hist, method="escape")
    rem, exp, offsets, _ = oracle.compress(W, "huffman", tabs, split_k=S)
    assert (oracle.decode("huffman", rem, exp, offsets, tabs) == W).all()
    _, exp_ref, _, _ = oracle.compress(W, "huffman", tables_for("huffman", hist), split_k=S)
    assert exp.size <= exp_ref.size


def test_oracle_rem_permutation_and_split():
    W = bits_of(make_weight(128, 256, 7))
    rem, exp = oracle.split(W)
    assert (((rem.astype(np.uint16) << 8) & 0x8000) | (rem & 0x7F) | (exp.astype(np.uint16) << 7) == W).all()
    tabs = tables_for("ans", oracle.histogram(W))
    prem, _, _, _ = oracle.compress(W, "ans", tabs, split_k=1)
    for blk in range(2):
        for lane in range(32):
            for h in range(2):
                for t in range(2):
                    assert prem[0, 5, blk * 128 + lane * 4 + h * 2 + t] == rem[5, blk * 128 + h * 64 + lane * 2 + t]


def test_oracle_matvec_and_fused_gemv_agree():
    W = make_weight(256, 512, 3)
    X = make_input(3, 512, 3)
    Wb, Xb = bits_of(W), bits_of(X)
    ref = (X.double() @ W.double().T).numpy()
    y = oracle.matvec(Wb, Xb)
    assert np.allclose(y, ref, rtol=1e-6, atol=1e-7)
    for algo in ("huffman", "ans"):
        tabs = tables_for(algo, oracle.histogram(Wb))
        rem, exp, offsets, _ = oracle.compress(Wb, algo, tabs)
        yf = oracle.gemv(algo, rem, exp, offsets, tabs, Xb)
        assert np.abs(yf - ref).max() / np.sqrt((ref ** 2).mean()) < 1e-4


def test_encode_operators_on_cpu():
    """The two per-stream operators of the reference, restated: chars / words and their counts."""
    W = bits_of(make_weight(128, 256, 5))
    hist = oracle.histogram(W)
    htabs, henc = huffman_tables(hist)
    atabs, _ = ans_tables(hist)
    _, e = oracle.split(W)
    data = e[:4, :64].copy()
    lut = np.zeros((256, 32), np.uint8)
    for s, code in henc.huffman_codes.items():
        path = code[::-1]
        lut[s, : len(path)] = [ord(c) for c in path]
    chars, bits = oracle.huffman_encode_op(data, lut)
    for i in range(4):
        want = "".join(henc.huffman_codes[int(s)][::-1] for s in data[i])
        assert bits[i] == len(want) and bytes(chars[i, : bits[i]]).decode() == want
        assert (chars[i, bits[i]:] == ord("0")).all()
    words, cnt = oracle.ans_encode_op(data, atabs["freq"], atabs["cum"])
    for i in range(4):
        assert words.view(np.uint32)[i, : cnt[i]].tolist() == oracle.py_ans_encode_stream(data[i].tolist(), atabs["freq"], atabs["cum"])


def test_chunk_count_matches_known_values():
    known = {4096: 1, 12288: 3, 3584: 1, 18944: 4, 8192: 2, 28672: 7, 1024: 1, 512: 1, 384: 1, 256: -1, 128: -1, 100: -1}
    for k, s in known.items():
        assert oracle.chunk_count(k) == s, k


REF_LAYOUT = sorted(f for f in os.listdir(GOLDEN) if f.startswith("ref_layout_") and f.endswith(".npz"))


@pytest.mark.parametrize("name", REF_LAYOUT or ["missing"])
def test_layout_matches_reference_gpu_buffers(name):
    """Whole-layer buffers recorded from the reference's CUDA extension on a B200 (see
    tests/golden/make_golden_gpu.py): the oracle must reproduce them byte for byte and decode them."""
    if name == "missing":
        pytest.skip("reference GPU fixtures not generated yet")
    z = np.load(os.path.join(GOLDEN, name))
    W = z["w_bits"]
    algo = str(z["algo"])
    if algo == "huffman":
        tabs = {k: z[k] for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")}
        mine, _ = huffman_tables(oracle.histogram(W))
        for k in tabs:
            assert (mine[k] == tabs[k]).all(), k
        tabs["code_values"] = mine["code_values"]
    else:
        tabs, _ = ans_tables(oracle.histogram(W))
        assert (tabs["LUT"] == z["LUT"]).all()
    S = z["rem"].shape[0]
    rem, exp, offsets, _ = oracle.compress(W, algo, tabs, split_k=S)
    assert (rem == z["rem"]).all()
    assert (offsets == z["offsets"]).all()
    assert exp.shape == z["exp"].shape and (exp == z["exp"]).all()
    assert (oracle.decode(algo, z["rem"], z["exp"], z["offsets"], tabs) == W).all()
    if "ref_decoded_bits" in z:
        assert (z["ref_decoded_bits"] == W).all()
