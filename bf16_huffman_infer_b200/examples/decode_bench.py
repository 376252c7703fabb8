"""Whole-model decode speed, the way the reference's README measures it: a Hugging Face causal LM with a
``StaticCache``, the one-token step CUDA-graphed, greedy decoding; first as plain BF16, then with
every linear layer compressed in place by ``convert_all_linear``.

    python -m bf16_huffman_infer_b200.examples.decode_bench                      # Qwen3-8B architecture
    python -m bf16_huffman_infer_b200.examples.decode_bench --layers 4 --tokens 32

There is no checkpoint offline, so the model is the named ARCHITECTURE with random weights
(N(0, 0.02), norms 1); token ids are random.  Prints one JSON line.  Attention, norms, RoPE and
sampling are Hugging Face's own kernels in both arms; only the linear layers differ.
"""
from __future__ import annotations

import argparse
import json
import time

import torch

ARCHS = {
    # hidden, intermediate, layers, heads, kv heads, head dim, vocab
    "qwen3-8b": (4096, 12288, 36, 32, 8, 128, 151936),
    "qwen3-1.7b": (2048, 6144, 28, 16, 8, 128, 151936),
}


def build(arch: str, layers: int | None, dev: torch.device):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    h, inter, n_layers, heads, kv, hd, vocab = ARCHS[arch]
    cfg = Qwen3Config(vocab_size=vocab, hidden_size=h, intermediate_size=inter, num_hidden_layers=layers or n_layers,
                      num_attention_heads=heads, num_key_value_heads=kv, head_dim=hd, max_position_embeddings=4096,
                      rope_theta=1e6, tie_word_embeddings=False)
    with torch.device(dev):
        model = Qwen3ForCausalLM(cfg).to(torch.bfloat16).eval()
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name:
                p.fill_(1.0)
            else:
                p.copy_((torch.randn(p.shape, device=dev, dtype=torch.float32, generator=g) * 0.02).to(torch.bfloat16))
    return cfg, model


def decode_speed(model, cfg, batch: int, prompt: int, tokens: int, dev: torch.device):
    """tokens/s of a greedy loop over the graphed one-token step, and of ``generate`` (the same graph replays plus
    Hugging Face's per-token host work), prompt processing excluded from both; plus the generated ids and how
    many one-token steps were graph replays / eager."""
    from transformers import StaticCache
    from .. import get_graphed_model
    cache = StaticCache(config=cfg, max_cache_len=prompt + tokens + 8)
    graphed = get_graphed_model(model, cache)
    ids = torch.randint(0, cfg.vocab_size, (batch, prompt), generator=torch.Generator().manual_seed(0)).to(dev)
    kw = dict(do_sample=False)
    graphed.generate(ids, max_new_tokens=4, min_new_tokens=4, **kw)                  # the first one-token step captures the graph
    torch.cuda.synchronize()

    def timed(n):
        t0 = time.perf_counter()
        out = graphed.generate(ids, max_new_tokens=n, min_new_tokens=n, **kw)
        torch.cuda.synchronize()
        return time.perf_counter() - t0, out

    t_short, _ = timed(1)                                                            # prompt + one token
    t_long, out = timed(tokens)
    generate_tps = batch * (tokens - 1) / (t_long - t_short)

    # the same greedy decoding driven directly: one graph replay and one argmax per token
    cache.reset()
    with torch.no_grad():
        tok = graphed(input_ids=ids).logits[:, -1:].argmax(-1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(tokens - 1):
            tok = graphed(input_ids=tok).logits[:, -1:].argmax(-1)
        e1.record()
        torch.cuda.synchronize()
    step_tps = batch * (tokens - 1) / (e0.elapsed_time(e1) * 1e-3)
    return step_tps, generate_tps, out, dict(graphed.graph_stats)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--arch", default="qwen3-8b", choices=sorted(ARCHS))
    ap.add_argument("--layers", type=int, default=None, help="fewer decoder layers than the architecture has")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--algo", default="huffman", choices=["huffman", "ans", "smallest"])
    ap.add_argument("--tables", default="limit6", choices=["limit6", "limit8", "escape", "reference"])
    ap.add_argument("--min-out-features", type=int, default=0)
    ap.add_argument("--no-fuse", action="store_true", help="keep q/k/v and gate/up as separate layers")
    args = ap.parse_args()

    from .. import convert_all_linear, get_model_size
    dev = torch.device("cuda", 0)
    cfg, model = build(args.arch, args.layers, dev)
    size_raw = get_model_size(model)
    dense_tps, dense_gen_tps, dense_ids, _ = decode_speed(model, cfg, args.batch, args.prompt, args.tokens, dev)
    t0 = time.perf_counter()
    convert_all_linear(model, min_out_features=args.min_out_features, progress=False, algo=args.algo,
                       fuse_siblings=not args.no_fuse, huffman_tables=args.tables)
    model.to(dev)
    torch.cuda.synchronize()
    convert_s = time.perf_counter() - t0
    size_comp = get_model_size(model)
    comp_tps, comp_gen_tps, comp_ids, stats = decode_speed(model, cfg, args.batch, args.prompt, args.tokens, dev)
    same = int((dense_ids == comp_ids).all())
    first_diff = None if same else int((dense_ids != comp_ids).any(0).nonzero()[0])
    print(json.dumps({
        "model": f"{args.arch} architecture, {cfg.num_hidden_layers} layers, random weights", "batch": args.batch,
        "prompt_tokens": args.prompt, "new_tokens": args.tokens, "algo": args.algo, "tables": args.tables,
        "fused_siblings": not args.no_fuse,
        "dense_bf16_tokens_per_s": round(dense_tps, 1), "compressed_tokens_per_s": round(comp_tps, 1),
        "through_generate": {"dense_bf16_tokens_per_s": round(dense_gen_tps, 1), "compressed_tokens_per_s": round(comp_gen_tps, 1)},
        "one_token_steps": stats,
        "model_bytes_bf16": size_raw, "model_bytes_compressed": size_comp, "ratio": round(size_comp / size_raw, 4),
        "convert_seconds": round(convert_s, 1),
        # lossless weights, but the fused kernel sums in another order than cuBLAS: greedy tokens of a random-weight
        # model (near-uniform logits) may part ways after some steps
        "same_greedy_tokens_as_dense": bool(same), "first_differing_position": first_diff,
    }))


if __name__ == "__main__":
    main()
