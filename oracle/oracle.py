"""ctypes front end of the CPU oracle (``oracle/bhi_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, by the smoke test and by the benchmark's
CPU-baseline leg as the checker the CUDA kernels are compared with.  The shipped package never
imports it.  All arrays are numpy; BF16 tensors travel as their ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Dict, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libbhi_oracle.so")
_SRC_PATH = os.path.join(_HERE, "bhi_oracle.c")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle next to its source (OpenMP when the compiler has it)."""
    if not force and os.path.exists(_LIB_PATH) and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(_SRC_PATH):
        return _LIB_PATH
    base = ["gcc", "-O3", "-fPIC", "-std=c11", "-shared", "-o", _LIB_PATH, _SRC_PATH]
    for extra in (["-fopenmp"], []):
        r = subprocess.run(base + extra, capture_output=True, text=True)
        if r.returncode == 0:
            return _LIB_PATH
    raise RuntimeError("could not build the CPU oracle:\n" + r.stderr)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.bhi_oracle_layout_offsets.restype = C.c_int64
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def threads() -> int:
    return int(lib().bhi_oracle_threads())


def set_threads(n: int) -> int:
    """Use ``n`` worker threads from now on (launchers such as torchrun export OMP_NUM_THREADS=1); returns the count in effect."""
    lib().bhi_oracle_set_threads(C.c_int(int(n)))
    return threads()


def chunk_count(k: int) -> int:
    return int(lib().bhi_oracle_chunk_count(C.c_int(k)))


def histogram(w_bits: np.ndarray) -> np.ndarray:
    w = _c(w_bits, np.uint16)
    out = np.zeros(256, dtype=np.int64)
    lib().bhi_oracle_histogram(_p(w), C.c_int64(w.size), _p(out))
    return out


def split(w_bits: np.ndarray):
    w = _c(w_bits, np.uint16)
    rem = np.empty(w.shape, np.uint8)
    exp = np.empty(w.shape, np.uint8)
    lib().bhi_oracle_split(_p(w), C.c_int64(w.size), _p(rem), _p(exp))
    return rem, exp


def _set_ans_bits(n: int) -> None:
    """Tell the C oracle the rANS probability precision; ``n`` is the table length ``2^bits`` (or the frequency sum)."""
    bits = int(n).bit_length() - 1
    if n != 1 << bits or not 8 <= bits <= 12:
        raise ValueError(f"rANS table length {n} is not 2^8..2^12")
    lib().bhi_oracle_set_ans_bits(bits)



def compress(w_bits: np.ndarray, algo: str, tables: Dict[str, np.ndarray], split_k: Optional[int] = None):
    """Whole-layer encode into the device format.  ``tables`` holds ``code_lengths`` and
    ``code_values`` (Huffman) or ``freq`` and ``cum`` (rANS).  Returns ``rem, exp, offsets, L``."""
    w = _c(w_bits, np.uint16)
    M, K = w.shape
    S = split_k if split_k is not None else chunk_count(K)
    assert S > 0 and K % S == 0 and (K // S) % 128 == 0, (K, S)
    L = np.zeros((S, M), np.int32)
    offsets = np.zeros((S, M), np.int32)
    rem = np.empty((S, M, K // S), np.uint8)
    l = lib()
    l.bhi_oracle_pack_rem(_p(w), M, K, S, _p(rem))
    if algo == "huffman":
        cl = _c(tables["code_lengths"], np.uint8)
        cv = _c(tables["code_values"], np.uint32)
        l.bhi_oracle_huffman_row_words(_p(w), M, K, S, _p(cl), _p(L))
    elif algo == "ans":
        fr = _c(tables["freq"], np.uint32)
        cu = _c(tables["cum"], np.uint32)
        _set_ans_bits(int(fr.astype(np.int64).sum()))
        l.bhi_oracle_ans_row_words(_p(w), M, K, S, _p(fr), _p(cu), _p(L))
    else:
        raise ValueError(algo)
    total = int(l.bhi_oracle_layout_offsets(_p(L), S, M, _p(offsets)))
    exp = np.zeros(total, np.uint32)
    if algo == "huffman":
        l.bhi_oracle_huffman_emit(_p(w), M, K, S, _p(cl), _p(cv), _p(offsets), _p(exp))
    else:
        l.bhi_oracle_ans_emit(_p(w), M, K, S, _p(fr), _p(cu), _p(offsets), _p(exp))
    return rem, exp.view(np.int32), offsets, L


def _geom(rem: np.ndarray):
    if rem.ndim == 2:
        rem = rem[None]
    S, M, Nc = rem.shape
    return _c(rem, np.uint8), S, M, Nc


def decode(algo: str, rem, exp, offsets, tables) -> np.ndarray:
    """Dense BF16 bit patterns ``[M, S*Nc]`` from the compressed form."""
    rem, S, M, Nc = _geom(rem)
    exp = _c(exp, np.int32).view(np.uint32)
    offsets = _c(offsets, np.int32)
    out = np.empty((M, S * Nc), np.uint16)
    if algo == "huffman":
        t = [_c(tables[k], np.uint8) for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")]
        rc = lib().bhi_oracle_huffman_decode(_p(rem), _p(exp), C.c_int64(exp.size), _p(offsets),
                                             *[_p(x) for x in t], S, M, Nc, _p(out))
    else:
        lut = _c(tables["LUT"], np.int32).view(np.uint32)
        _set_ans_bits(lut.size)
        rc = lib().bhi_oracle_ans_decode(_p(rem), _p(exp), C.c_int64(exp.size), _p(offsets), _p(lut), S, M, Nc, _p(out))
    if rc != 0:
        raise RuntimeError(f"oracle decode failed (status {rc})")
    return out


def matvec(w_bits: np.ndarray, x_bits: np.ndarray) -> np.ndarray:
    """``Y[b, m] = sum_c X[b, c] * W[m, c]`` in double precision, returned as float32."""
    w = _c(w_bits, np.uint16)
    x = _c(x_bits, np.uint16)
    M, K = w.shape
    B = x.shape[0]
    assert x.shape[1] == K
    y = np.empty((B, M), np.float32)
    lib().bhi_oracle_matvec(_p(w), _p(x), B, M, C.c_int64(K), _p(y))
    return y


def gemv(algo: str, rem, exp, offsets, tables, x_bits: np.ndarray) -> np.ndarray:
    """Fused CPU decode + matvec (FP32 accumulate); the timed CPU baseline."""
    rem, S, M, Nc = _geom(rem)
    exp = _c(exp, np.int32).view(np.uint32)
    offsets = _c(offsets, np.int32)
    x = _c(x_bits, np.uint16)
    B = x.shape[0]
    y = np.empty((B, M), np.float32)
    if algo == "huffman":
        keep = [_c(tables[k], np.uint8) for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")]
        t = [_p(a) for a in keep]
        rc = lib().bhi_oracle_gemv(0, _p(rem), _p(exp), C.c_int64(exp.size), _p(offsets), *t, None,
                                   S, M, Nc, _p(x), B, _p(y))
    else:
        lut = _c(tables["LUT"], np.int32).view(np.uint32)
        _set_ans_bits(lut.size)
        rc = lib().bhi_oracle_gemv(1, _p(rem), _p(exp), C.c_int64(exp.size), _p(offsets),
                                   None, None, None, None, None, _p(lut), S, M, Nc, _p(x), B, _p(y))
    if rc != 0:
        raise RuntimeError(f"oracle gemv failed (status {rc})")
    return y


def huffman_encode_op(data: np.ndarray, code_chars: np.ndarray):
    """The reference's ``huffman_encode`` operator on the CPU: chars out + bit counts."""
    d = _c(data, np.uint8)
    streams, n = d.shape
    lut = _c(code_chars, np.uint8)
    out = np.full((streams, 32 * n), ord("0"), np.uint8)
    lens = np.zeros(streams, np.int32)
    lib().bhi_oracle_huffman_encode_op(_p(d), streams, n, _p(lut), _p(out), _p(lens))
    return out, lens


def ans_encode_op(data: np.ndarray, freq, cum):
    """The reference's ``ans_encode`` operator on the CPU: words out + word counts."""
    d = _c(data, np.uint8)
    streams, n = d.shape
    out = np.zeros((streams, 8 * n), np.uint32)
    lens = np.zeros(streams, np.int32)
    _set_ans_bits(int(np.asarray(freq, np.int64).sum()))
    lib().bhi_oracle_ans_encode_op(_p(d), streams, n, _p(_c(freq, np.uint32)), _p(_c(cum, np.uint32)), _p(out), _p(lens))
    return out.view(np.int32), lens


# ---- pure-Python single-stream restatements (small cases only) ---------------------------------
def py_huffman_encode_stream(symbols, code_lengths, code_values):
    """Words of one stream, LSB-first packing (functional.py:149-157)."""
    acc = 0
    have = 0
    for s in symbols:
        acc |= int(code_values[s]) << have
        have += int(code_lengths[s])
    nwords = (have + 31) // 32
    return [(acc >> (32 * i)) & 0xFFFFFFFF for i in range(nwords)], have


def py_huffman_decode_stream(words, n, tables):
    """Window decoder of src/kernel.cu:354-380 on one stream (``words`` may be over-read as 0)."""
    l1, l2, l3, l4, ln = (tables[k] for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths"))
    win, have, at, out = 0, 0, 0, []
    for _ in range(n):
        if have < 32:
            win |= (words[at] if at < len(words) else 0) << have
            at += 1
            have += 32
        for k, tab in enumerate((l1, l2, l3, l4)):
            sym = int(tab[(win >> (8 * k)) & 0xFF])
            if sym != 255:
                break
        out.append(sym)
        win >>= int(ln[sym])
        have -= int(ln[sym])
    return out


def py_ans_encode_stream(symbols, freq, cum, bits=8):
    """src/kernel.cu:767-811 on one stream; returns the words in stored (decode) order."""
    state = 1 << bits
    out = []
    for s in reversed(list(symbols)):
        f, c = int(freq[s]), int(cum[s])
        while (state >> 32) >= f:
            out.append(state & 0xFFFFFFFF)
            state >>= 32
        state = ((state // f) << bits) + (state % f) + c
    while state > 0:
        out.append(state & 0xFFFFFFFF)
        state >>= 32
    return out[::-1]


def py_ans_decode_stream(words, n, lut, bits=8):
    """src/kernel.cu:652-683 on one stream."""
    at = 1
    state = int(words[0])
    out = []
    for _ in range(n):
        if state < (1 << bits):
            state = (state << 32) | int(words[at])
            at += 1
        e = int(lut[state & ((1 << bits) - 1)]) & 0xFFFFFFFF
        state = ((e >> 12) & 0xFFF) * (state >> bits) + (e & 0xFFF)
        out.append(e >> 24)
    return out
