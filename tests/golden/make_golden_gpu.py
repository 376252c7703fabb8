"""Record whole-layer buffers produced by the UNMODIFIED reference on a CUDA device.

Needs the reference installed at ``baseline/_ref`` (``pip install --target baseline/_ref`` of the
reference project, built for sm_100a) and a GPU:

    python tests/golden/make_golden_gpu.py [extra_output_dir]      # writes tests/golden/ref_layout_*.npz

For a few small seeded layers it runs the reference's own ``HuffmanWeight.compress`` /
``ANSWeight.compress`` (or ``compress_split_n`` to force a K-split), its ``get_weight`` decode and its
fused GEMV, and stores inputs and outputs.  The reference is imported in this process only; the
package under test is never loaded here (both register the same operator namespace).
"""
import os
import shutil
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

from bf16_huffman_infer.functional import ANSWeight, HuffmanWeight, CompressedLinear  # noqa: E402

CASES = [
    # name, M, K, forced split (None = the reference's own choice), seed
    ("huffman_128x512", "huffman", 128, 512, None, 0),
    ("huffman_128x512_s2", "huffman", 128, 512, 2, 1),
    ("ans_128x512", "ans", 128, 512, None, 0),
    ("ans_256x384_s3", "ans", 256, 384, 3, 2),
    ("huffman_4224x128", "huffman", 4224, 128, 1, 3),        # crosses the 4096-row slab boundary
    ("huffman_256x1024_std1", "huffman", 256, 1024, None, 4),
]


def weight(M, K, seed, std):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(M, K, dtype=torch.float32, generator=g) * std).to(torch.bfloat16)


def main():
    out_dirs = [HERE] + [d for d in sys.argv[1:2] if os.path.isdir(d)]      # a second copy, e.g. on a scratch volume
    for name, algo, M, K, split, seed in CASES:
        std = 1.0 if "std1" in name else 0.02
        W = weight(M, K, seed, std)
        cls = HuffmanWeight if algo == "huffman" else ANSWeight
        cw = cls.compress(W) if split is None else cls.compress_split_n(W, n=split)
        bufs = {k: v.cpu().numpy() for k, v in cw.kwargs().items()}
        if bufs["rem"].ndim == 2:
            bufs["rem"] = bufs["rem"][None]
        cw = cw.cuda()
        dense = cw.get_weight().cpu()
        g = torch.Generator().manual_seed(seed + 1000)
        X = torch.randn(8, K, dtype=torch.float32, generator=g).to(torch.bfloat16)
        lin = CompressedLinear(cw, None)
        ys = {f"ref_y_b{b}": lin(X[:b].cuda()).float().cpu().numpy() for b in (1, 3, 8)}
        np.savez_compressed(
            os.path.join(HERE, f"ref_layout_{name}.npz"),
            algo=algo, w_bits=W.view(torch.int16).numpy().view(np.uint16),
            x_bits=X.view(torch.int16).numpy().view(np.uint16),
            ref_decoded_bits=dense.view(torch.int16).numpy().view(np.uint16),
            **bufs, **ys,
        )
        for d in out_dirs[1:]:
            shutil.copy(os.path.join(HERE, f"ref_layout_{name}.npz"), d)
        print(name, {k: v.shape for k, v in bufs.items()}, "decode exact:", bool(torch.equal(dense.view(torch.int16), W.view(torch.int16))))


if __name__ == "__main__":
    main()
