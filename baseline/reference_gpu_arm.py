"""Times the reference's own fused GEMV kernels on the GPU (the kernels this package has to beat).

Run as a separate process (it registers the same operator namespace as this package, so the two
cannot share one): ``python baseline/reference_gpu_arm.py [--batch B]``.  It needs the unmodified
reference installed under ``baseline/_ref`` (``pip install --target baseline/_ref``, built for
sm_100a) and prints one JSON line: per Qwen3-8B linear shape and coder the time of one
``CompressedLinear`` forward through the reference's public API, captured once into a CUDA graph (its
launcher queries the device properties on every call, milliseconds of host time that a decode loop
under a graph does not pay) and replayed with the L2 flushed before every replay (CUDA events, median
of 10), the compressed bytes per second, and the decode tokens/s a whole Qwen3-8B stack of such
layers would give.  ``{"unavailable": reason}`` when the reference cannot be
imported or run.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHAPES = {"q_o": (4096, 4096), "k_v": (1024, 4096), "gate_up": (12288, 4096), "down": (4096, 12288)}
PER_MODEL = {"q_o": 2 * 36, "k_v": 2 * 36, "gate_up": 2 * 36, "down": 36}      # plus the output head, scaled from gate_up


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    args = ap.parse_args()
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "bf16_huffman_infer")):
        print(json.dumps({"unavailable": "the reference is not installed under baseline/_ref"}))
        return
    sys.path.insert(0, ref_dir)
    try:
        import torch
        from bf16_huffman_infer.functional import ANSWeight, CompressedLinear, HuffmanWeight
    except Exception as e:                                         # noqa: BLE001
        print(json.dumps({"unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
        return
    dev = "cuda:0"
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)
    out = {"batch": args.batch, "per_shape": []}
    step_us = {"huffman": 0.0, "ans": 0.0}
    try:
        for name, (M, K) in SHAPES.items():
            g = torch.Generator().manual_seed(0)
            W = (torch.randn(M, K, generator=g) * 0.02).to(torch.bfloat16)
            x = torch.randn(args.batch, K, device=dev, dtype=torch.bfloat16)
            for algo, cls in (("huffman", HuffmanWeight), ("ans", ANSWeight)):
                cw = cls.compress(W)
                nbytes = sum(b.nelement() * b.element_size() for b in cw.buffers())
                lin = CompressedLinear(cw, None).to(dev)
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side), torch.no_grad():
                    for _ in range(2):
                        lin(x)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph), torch.no_grad():
                    lin(x)
                ts = []
                for _ in range(13):
                    flush.zero_()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    graph.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1) * 1e3)
                del graph
                us = sorted(ts[3:])[5]
                alg = nbytes + args.batch * (K + M) * 2
                out["per_shape"].append({"shape": name, "M": M, "K": K, "algo": algo, "us": round(us, 2),
                                         "gbs": round(alg / us / 1e3, 1), "ratio": round(nbytes / (2.0 * M * K), 4)})
                step_us[algo] += us * PER_MODEL[name] + (us * 151936 / 12288 if name == "gate_up" else 0.0)
                del lin, cw
        out["tokens_per_s_equiv"] = {a: round(args.batch / (t * 1e-6), 1) for a, t in step_us.items()}
        out["note"] = "the reference's kernels built for sm_100a, one launch per projection (it has no stacked q/k/v or gate/up)"
    except Exception as e:                                         # noqa: BLE001
        out = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
