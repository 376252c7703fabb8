"""Shared helpers of the test-suite: seeded inputs, table construction, the ctypes view of the C ABI."""
import ctypes as C
import json
import os
import re

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
HEADER = os.path.join(ROOT, "include", "bf16_huffman_b200.h")
LIB = os.path.join(ROOT, "bf16_huffman_infer_b200", "libbf16_huffman_b200.so")


def make_weight(M, K, seed, std=0.02):
    """The synthetic layer of the benchmark configurations: N(0, std) from the CPU generator, BF16."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(M, K, dtype=torch.float32, generator=g) * std).to(torch.bfloat16)


def make_input(B, K, seed):
    g = torch.Generator().manual_seed(seed + 1000)
    return torch.randn(B, K, dtype=torch.float32, generator=g).to(torch.bfloat16)


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def huffman_tables(hist, method="reference"):
    from bf16_huffman_infer_b200.huffman import LUTHuffmanEncoder
    enc = LUTHuffmanEncoder()
    enc.build_lut(np.asarray(hist), method=method)
    return {"LUT1": enc.LUT1, "LUT2": enc.LUT2, "LUT3": enc.LUT3, "LUT4": enc.LUT4,
            "code_lengths": enc.code_lengths, "code_values": enc.code_values}, enc


def ans_tables(hist, precision=8):
    from bf16_huffman_infer_b200.ans import RANSEncoder
    enc = RANSEncoder([int(x) for x in hist], precision=precision)
    lut = np.array([(s << 24) | (f << 12) | r for s, f, r in enc.decode_lut], dtype=np.uint32)
    return {"freq": np.array(enc.freq, np.uint32), "cum": np.array(enc.cum, np.uint32), "LUT": lut.view(np.int32)}, enc


def ans_bits(w):
    """Probability precision of a rANS weight: its table has ``2^bits`` words."""
    return int(w["LUT"].numel() if hasattr(w["LUT"], "numel") else len(w["LUT"])).bit_length() - 1


def tables_for(algo, hist, method="reference"):
    return huffman_tables(hist, method)[0] if algo == "huffman" else ans_tables(hist)[0]


def load_json(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def header_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bhi_[a-z0-9_]+)\s*\(", text)))


def bf16_half_ulp(v):
    """Half the BF16 spacing at |v| (what rounding an exact value to BF16 may cost)."""
    v = np.abs(np.asarray(v, np.float64))
    e = np.floor(np.log2(np.maximum(v, 2.0 ** -126)))
    return 2.0 ** (e - 8)


def rel_err(y, y_ref):
    """The accuracy measure of the 1e-2 bound: max |y - y_ref| / rms(y_ref), where the unavoidable
    rounding of the exact value to the BF16 output type (half a BF16 ulp at y_ref) is not counted.
    Without that allowance no BF16-output kernel, the reference's included, could meet 1e-2 on a
    large output: a value of 2.6 rms sitting at the bottom of a binade already rounds by 1e-2 rms."""
    y = np.asarray(y, np.float64)
    y_ref = np.asarray(y_ref, np.float64)
    excess = np.maximum(np.abs(y - y_ref) - bf16_half_ulp(y_ref), 0.0)
    return float(excess.max() / max(np.sqrt((y_ref ** 2).mean()), 1e-30))


def raw_rel_err(y, y_ref):
    """max |y - y_ref| / rms(y_ref) with nothing taken off: the figure the 1e-2 bound is quoted on, BF16 output
    rounding included (it alone reaches 1e-2 rms for an output of 2.6 rms, see rel_err)."""
    y = np.asarray(y, np.float64)
    y_ref = np.asarray(y_ref, np.float64)
    return float(np.abs(y - y_ref).max() / max(np.sqrt((y_ref ** 2).mean()), 1e-30))


def bf16_round(v):
    """Round-to-nearest-even of float values to BF16, returned as float64."""
    t = torch.from_numpy(np.asarray(v, np.float64)).to(torch.float32).to(torch.bfloat16)
    return t.to(torch.float64).numpy()


def ulp_excess(y, y_ref):
    """How far |y - bf16(y_ref)| exceeds one BF16 ulp of y_ref, in units of rms(y_ref); <= 0 means every output
    is the correctly rounded value or its neighbour.  (An FP32 accumulation in another order than the
    reference's moves a sum by a few 1e-7 relative, enough to cross a rounding boundary, never two.)"""
    y = np.asarray(y, np.float64)
    y_ref = np.asarray(y_ref, np.float64)
    excess = np.abs(y - bf16_round(y_ref)) - 2.0 * bf16_half_ulp(y_ref)
    return float(excess.max() / max(np.sqrt((y_ref ** 2).mean()), 1e-30))


class Abi:
    """ctypes access to libbf16_huffman_b200.so taking torch CUDA tensors (data pointers only)."""

    def __init__(self):
        self.lib = C.CDLL(LIB)
        self.lib.bhi_last_error.restype = C.c_char_p

    @staticmethod
    def p(t):
        return C.c_void_p(0 if t is None else t.data_ptr())

    def check(self, rc):
        if rc != 0:
            raise RuntimeError(f"C ABI error {rc}: {self.lib.bhi_last_error().decode()}")

    @staticmethod
    def stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def set_path(self, path):
        return self.lib.bhi_set_kernel_path(C.c_int(path))

    def set_quad_warps(self, warps):
        return self.lib.bhi_set_quad_warps(C.c_int(warps))

    def prepare(self, w):
        """Fold the Huffman tables of `w` into a prepared blob (cached in the dict)."""
        if "_prepared" not in w:
            self.lib.bhi_huffman_prepared_bytes.restype = C.c_int
            blob = torch.empty(self.lib.bhi_huffman_prepared_bytes(), dtype=torch.uint8, device=w["rem"].device)
            p = self.p
            self.check(self.lib.bhi_huffman_prepare(p(w["LUT1"]), p(w["LUT2"]), p(w["LUT3"]), p(w["LUT4"]),
                                                    p(w["code_lengths"]), p(blob), self.stream()))
            self.check(self.lib.bhi_huffman_table_hint(p(blob), int(int(w["code_lengths"].max().item()) <= 6)))
            w["_prepared"] = blob
        return w["_prepared"]

    def gemv(self, algo, w, x, prepared=False):
        """w: dict of CUDA tensors (rem [S,M,Nc], exp, offsets, tables); x: bf16 [B, K] -> bf16 [B, M]."""
        S, M, Nc = w["rem"].shape
        B = x.shape[0]
        y = torch.empty(B, M, dtype=torch.bfloat16, device=x.device)
        p = self.p
        if algo == "huffman" and prepared:
            rc = self.lib.bhi_gemv_bf16_huffman_prepared(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(y),
                                                         p(w["offsets"]), p(self.prepare(w)), S, M, Nc, B, self.stream())
        elif algo == "huffman":
            rc = self.lib.bhi_gemv_bf16_huffman(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(y),
                                                p(w["offsets"]), p(w["LUT1"]), p(w["LUT2"]), p(w["LUT3"]), p(w["LUT4"]),
                                                p(w["code_lengths"]), S, M, Nc, B, self.stream())
        else:
            rc = self.lib.bhi_gemv_bf16_ans(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(y),
                                            p(w["offsets"]), p(w["LUT"]), ans_bits(w), S, M, Nc, B, self.stream())
        self.check(rc)
        return y

    def linear(self, algo, w, x, prepared=False):
        """Fused decode + tensor-core product: x bf16 [B <= 128, K] -> bf16 [B, M]."""
        S, M, Nc = w["rem"].shape
        B = x.shape[0]
        y = torch.empty(B, M, dtype=torch.bfloat16, device=x.device)
        p = self.p
        if algo == "huffman" and prepared:
            rc = self.lib.bhi_linear_bf16_huffman_prepared(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(y),
                                                           p(w["offsets"]), p(self.prepare(w)), S, M, Nc, B, self.stream())
        elif algo == "huffman":
            rc = self.lib.bhi_linear_bf16_huffman(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(y),
                                                  p(w["offsets"]), p(w["LUT1"]), p(w["LUT2"]), p(w["LUT3"]), p(w["LUT4"]),
                                                  p(w["code_lengths"]), S, M, Nc, B, self.stream())
        else:
            rc = self.lib.bhi_linear_bf16_ans(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(x), p(y),
                                              p(w["offsets"]), p(w["LUT"]), ans_bits(w), S, M, Nc, B, self.stream())
        self.check(rc)
        return y

    def decode(self, algo, w, prepared=False):
        S, M, Nc = w["rem"].shape
        y = torch.empty(M, S * Nc, dtype=torch.bfloat16, device=w["rem"].device)
        p = self.p
        if algo == "huffman" and prepared:
            rc = self.lib.bhi_huffman_decode_prepared(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(y),
                                                      p(w["offsets"]), p(self.prepare(w)), S, M, Nc, self.stream())
        elif algo == "huffman":
            rc = self.lib.bhi_huffman_decode(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(y), p(w["offsets"]),
                                             p(w["LUT1"]), p(w["LUT2"]), p(w["LUT3"]), p(w["LUT4"]), p(w["code_lengths"]),
                                             S, M, Nc, self.stream())
        else:
            rc = self.lib.bhi_ans_decode(p(w["rem"]), p(w["exp"]), C.c_int64(w["exp"].numel()), p(y), p(w["offsets"]),
                                         p(w["LUT"]), ans_bits(w), S, M, Nc, self.stream())
        self.check(rc)
        return y

    def encode(self, algo, W, S, tables):
        """Whole-layer encode through the C ABI; the prefix sum between the passes is done with torch."""
        from bf16_huffman_infer_b200.functional import _record_offsets
        dev = W.device
        M, K = W.shape
        p = self.p
        rows = torch.empty(S, M, dtype=torch.int32, device=dev)
        rem = torch.empty(S, M, K // S, dtype=torch.uint8, device=dev)
        if algo == "huffman":
            cl = torch.from_numpy(np.ascontiguousarray(tables["code_lengths"])).to(dev)
            cv = torch.from_numpy(np.ascontiguousarray(tables["code_values"]).view(np.int32)).to(dev)
            self.check(self.lib.bhi_huffman_size_pass(p(W), M, K, S, p(cl), p(rows), self.stream()))
            offsets, total = _record_offsets(rows)
            exp = torch.zeros(total, dtype=torch.int32, device=dev)
            self.check(self.lib.bhi_huffman_emit_pass(p(W), M, K, S, p(cl), p(cv), p(offsets), p(rem), p(exp), self.stream()))
        else:
            fr = torch.from_numpy(np.ascontiguousarray(tables["freq"]).view(np.int32)).to(dev)
            cu = torch.from_numpy(np.ascontiguousarray(tables["cum"]).view(np.int32)).to(dev)
            sw = torch.empty(S, M, 64, dtype=torch.uint8, device=dev)
            self.check(self.lib.bhi_ans_size_pass(p(W), M, K, S, p(fr), p(cu), p(rows), p(sw), self.stream()))
            offsets, total = _record_offsets(rows)
            exp = torch.zeros(total, dtype=torch.int32, device=dev)
            self.check(self.lib.bhi_ans_emit_pass(p(W), M, K, S, p(fr), p(cu), p(offsets), p(sw), p(rem), p(exp), self.stream()))
        torch.cuda.synchronize()
        return rem, exp, offsets, rows


def to_device(arrs, dev):
    out = {}
    for k, v in arrs.items():
        a = np.ascontiguousarray(v)
        if a.dtype == np.uint32:
            a = a.view(np.int32)
        out[k] = torch.from_numpy(a).to(dev)
    return out
