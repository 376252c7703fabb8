"""The two branches for more than 8 activation rows, one layer at a time.

For each layer shape and row count: the fused decode + tensor-core product (``mm_huffman_prepared`` / ``mm_ans``,
what ``BHI_TENSOR_ROWS`` turns on) against decode-to-dense followed by ``torch.matmul`` (the default branch, as in
the reference, ``functional.py:405-407``).  Timed on the device over enough distinct copies of the layer to exceed
L2, replayed from a CUDA graph::

    python -m bf16_huffman_infer_b200.examples.linear_bench [--shapes 4096x4096,12288x4096,4096x12288]
                                                          [--rows 16,64,128] [--algo huffman|ans] [--once]

``--once`` runs each branch a few times without graph or timing (for a profiler).
"""
import argparse
import json
import math

import torch

from bf16_huffman_infer_b200 import ANSWeight, HuffmanWeight, ops
from bf16_huffman_infer_b200.functional import mm_ans, mm_huffman_prepared


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="4096x4096,12288x4096,4096x12288")
    ap.add_argument("--rows", default="16,64,128")
    ap.add_argument("--algo", default="huffman", choices=["huffman", "ans"])
    ap.add_argument("--once", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    for shape in args.shapes.split(","):
        M, K = (int(v) for v in shape.split("x"))
        g = torch.Generator(device=dev).manual_seed(0)
        W = (torch.randn(M, K, dtype=torch.float32, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        cw = (HuffmanWeight if args.algo == "huffman" else ANSWeight).compress(W, to_cpu=False)
        copies = 1 if args.once else max(2, math.ceil(400e6 / cw.nbytes()))
        rems = [cw.rem.clone() for _ in range(copies)]
        exps = [cw.exp.clone() for _ in range(copies)]
        tables = cw.prepared() if args.algo == "huffman" else cw.LUT
        dense = torch.empty(M, K, dtype=torch.bfloat16, device=dev)

        def fused(i, X):
            if args.algo == "huffman":
                return mm_huffman_prepared(rems[i], exps[i], X, cw.offsets, tables)
            return mm_ans(rems[i], exps[i], X, cw.offsets, tables)

        def two_step(i, X):
            if args.algo == "huffman":
                ops.huffman_decode_prepared(rems[i], exps[i], dense, cw.offsets, tables)
            else:
                ops.ans_decode(rems[i], exps[i], dense, cw.offsets, tables)
            return X @ dense.T

        for B in (int(v) for v in args.rows.split(",")):
            X = torch.randn(B, K, device=dev, generator=g).to(torch.bfloat16)
            ref = X.float() @ W.float().T
            line = {"M": M, "K": K, "rows": B, "algo": args.algo}
            for name, fn in (("fused_us", fused), ("decode_gemm_us", two_step)):
                y = fn(0, X)
                torch.cuda.synchronize()
                err = ((y.float() - ref).abs().max() / ref.pow(2).mean().sqrt()).item()
                assert err < 2e-2, (name, err)
                if args.once:
                    for _ in range(3):
                        fn(0, X)
                    torch.cuda.synchronize()
                    continue
                stream = torch.cuda.Stream()
                with torch.cuda.stream(stream):
                    for i in range(copies):
                        fn(i, X)
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        for i in range(copies):
                            fn(i, X)
                    for _ in range(3):
                        graph.replay()
                    torch.cuda.synchronize()
                    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0.record()
                    for _ in range(5):
                        graph.replay()
                    t1.record()
                    torch.cuda.synchronize()
                line[name] = round(t0.elapsed_time(t1) * 1e3 / (5 * copies), 2)
            print(json.dumps(line), flush=True)
        del rems, exps, dense
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
