"""Generate ``tests/golden/ref_tables.json`` and ``tests/golden/ref_streams.json``.

Run where the reference project's sources are available:

    python tests/golden/make_golden_cpu.py /path/to/reference

It imports the reference's pure-Python modules ``bf16_huffman_infer/huffman.py`` and
``bf16_huffman_infer/ans.py`` by path (they need no GPU) and records

* for a set of exponent histograms: the Huffman tables (``LUT1..4``, ``code_lengths``, code
  strings) of ``LUTHuffmanEncoder.build_lut`` and the rANS model (``freq``, ``cum``, ``decode_lut``)
  of ``RANSEncoder(counts, precision=8)``, or the fact that the reference raised;
* for a few of those tables: short symbol streams with the output of the reference's slow
  single-stream codecs (``encode_to_bitstream`` / ``decode_with_lut``, ``compress`` / ``decompress``).

The histograms are stored in the fixture, so the tests do not depend on a random generator.
"""
import importlib.util
import json
import os
import sys

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BHI_REFERENCE_DIR", "reference")
HERE = os.path.dirname(os.path.abspath(__file__))


def load(name, rel):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


RH = load("ref_huffman", "bf16_huffman_infer/huffman.py")
RA = load("ref_ans", "bf16_huffman_infer/ans.py")


def exp_hist(M, K, seed, std=0.02):
    torch.manual_seed(seed)
    w = (torch.randn(M, K, dtype=torch.float32) * std).to(torch.bfloat16)
    e = (w.view(torch.int16).to(torch.int32) >> 7) & 0xFF
    return torch.bincount(e.flatten(), minlength=256).numpy().astype(np.int64)


def histograms():
    rng = np.random.default_rng(1234)
    out = []
    for seed in range(7):                       # the layer shapes of the GEMV sweep, small stand-ins
        out.append((f"normal_1024x4096_seed{seed}", exp_hist(1024, 4096, seed)))
    out.append(("normal_4096x4096_seed0", exp_hist(4096, 4096, 0)))
    out.append(("normal_256x512_seed3", exp_hist(256, 512, 3)))
    out.append(("normal_std1_512x512", exp_hist(512, 512, 11, std=1.0)))
    h = np.zeros(256, np.int64); h[7] = 5
    out.append(("single_symbol", h))
    h = np.zeros(256, np.int64); h[7] = 5; h[200] = 1
    out.append(("two_symbols", h))
    h = np.zeros(256, np.int64); h[:40] = [int(1.6 ** i) + 1 for i in range(40)]
    out.append(("geometric_1.6_x40", h))
    h = np.zeros(256, np.int64); h[:60] = [int(1.45 ** i) + 1 for i in range(60)]
    out.append(("geometric_1.45_x60", h))
    out.append(("uniform_random_256", rng.integers(1, 1000, 256).astype(np.int64)))
    h = np.zeros(256, np.int64); h[:16] = 100
    out.append(("flat_16", h))
    for i in range(16):
        k = int(rng.integers(2, 120))
        h = np.zeros(256, np.int64)
        h[rng.choice(256, k, replace=False)] = (rng.pareto(0.7, k) * 50 + 1).astype(np.int64)
        out.append((f"pareto_{i}", h))
    return out


def main():
    tables = []
    streams = []
    rng = np.random.default_rng(99)
    for name, h in histograms():
        rec = {"name": name, "hist": h.tolist()}
        enc = RH.LUTHuffmanEncoder()
        try:
            enc.build_lut(h)
            rec["huffman"] = {
                "LUT1": enc.LUT1.tolist(), "LUT2": enc.LUT2.tolist(),
                "LUT3": enc.LUT3.tolist(), "LUT4": enc.LUT4.tolist(),
                "code_lengths": enc.code_lengths.tolist(),
                "codes": {str(k): v for k, v in enc.huffman_codes.items()},
            }
        except AssertionError:
            rec["huffman"] = "AssertionError"
        ans = RA.RANSEncoder(h.tolist(), precision=8)
        rec["ans"] = {"freq": ans.freq, "cum": ans.cum, "decode_lut": [list(t) for t in ans.decode_lut]}
        tables.append(rec)

        if rec["huffman"] != "AssertionError" and len(streams) < 10:
            present = np.flatnonzero(h)
            p = h[present] / h[present].sum()
            for n in (1, 2, 64, 74):
                sym = rng.choice(present, size=n, p=p).astype(int).tolist()
                bits = RH.LUTHuffmanEncoder.encode_to_bitstream(np.array(sym), enc.huffman_codes, progress=False)
                import io, contextlib
                # The reference's decode_with_lut keeps its bit cursor in a numpy uint8 once the first
                # code length has been added (numpy 2 semantics), so its slicing goes wrong from the
                # second symbol on; only its first decoded symbol is a usable reference value.
                try:
                    with contextlib.redirect_stderr(io.StringIO()):   # the reference draws a progress bar
                        dec = [int(x) for x in enc.decode_with_lut(bits, n)][:1]
                except OverflowError:
                    dec = None
                blob = ans.compress(sym)
                back = ans.decompress(blob, n)
                streams.append({
                    "table": name, "symbols": sym,
                    "huffman_bitstring": bits, "huffman_decoded": dec,
                    "ans_blob_hex": blob.hex(), "ans_decoded": [int(x) for x in back],
                })
    with open(os.path.join(HERE, "ref_tables.json"), "w") as f:
        json.dump(tables, f, separators=(",", ":"))
    with open(os.path.join(HERE, "ref_streams.json"), "w") as f:
        json.dump(streams, f, separators=(",", ":"))
    print(f"{len(tables)} tables, {len(streams)} streams")
    finer_ans_models()


def finer_ans_models():
    """``RANSEncoder`` at 10 and 12 probability bits (the reference's class takes any precision; its kernels' table word
    holds up to 12): scaled frequencies and the blob of a few streams, in ``ref_ans_precision.json``."""
    rng = np.random.default_rng(1234)
    out = []
    for name, h in histograms()[:6]:
        present = np.flatnonzero(h)
        p = h[present] / h[present].sum()
        for bits in (10, 12):
            ans = RA.RANSEncoder(h.tolist(), precision=bits)
            for n in (1, 64, 74):
                sym = rng.choice(present, size=n, p=p).astype(int).tolist()
                blob = ans.compress(sym)
                assert [int(x) for x in ans.decompress(blob, n)] == sym
                out.append({"table": name, "precision": bits, "hist": h.tolist(), "freq": ans.freq, "cum": ans.cum,
                            "symbols": sym, "ans_blob_hex": blob.hex()})
    with open(os.path.join(HERE, "ref_ans_precision.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print(f"{len(out)} finer-model streams")


if __name__ == "__main__":
    main()
