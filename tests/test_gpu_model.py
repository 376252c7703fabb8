"""Model-level checks on a GPU: convert_all_linear on a small random-init Qwen3-architecture model,
prompt logits against the uncompressed model, and the CUDA-graphed decode loop."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiny_model(seed=0):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = Qwen3Config(vocab_size=2048, hidden_size=2048, intermediate_size=6144, num_hidden_layers=2,
                      num_attention_heads=16, num_key_value_heads=2, head_dim=128, max_position_embeddings=256,
                      rope_theta=1e6, tie_word_embeddings=False)
    torch.manual_seed(seed)
    model = Qwen3ForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name:
                p.fill_(1.0)
            else:
                p.copy_((torch.randn(p.shape) * 0.02).to(torch.bfloat16))
    return cfg, model


def _generate(model, cache, ids, n):
    return model.generate(ids, max_new_tokens=n, min_new_tokens=n, do_sample=False, past_key_values=cache,
                          disable_compile=True)


def _same_decoding(run, ref, what, tol=0.05):
    """Two greedy runs (generate(..., output_logits=True, return_dict_in_generate=True)) decode the same thing.
    The eager run is handed an explicit mask by generate() and the captured step derives it from the cache, so the
    attention kernels differ and logits agree only to BF16 noise; with random weights the two best logits are
    sometimes closer than that.  So: tokens equal up to the first difference, logits close at every step up to and
    including it, and at that step the reference's two best logits closer than the noise."""
    a, b = run.sequences.cpu(), ref.sequences.cpu()
    prompt = a.shape[1] - len(run.logits)
    for step, (la, lb) in enumerate(zip(run.logits, ref.logits)):
        la, lb = la.float().cpu(), lb.float().cpu()
        noise = (la - lb).abs().max() / lb.pow(2).mean().sqrt()
        assert noise < tol, (what, step, float(noise))           # a wrong position or mask would give differences of order 1
        if not torch.equal(a[:, prompt + step], b[:, prompt + step]):
            top2 = lb.topk(2, dim=-1).values
            margin = ((top2[:, 0] - top2[:, 1]) / lb.pow(2).mean().sqrt()).min()
            assert margin <= noise, (what, step, float(margin), float(noise))
            return step
    return len(run.logits)


@pytest.mark.parametrize("batch", [1, 2])
def test_graphed_generate_matches_eager(batch):
    from transformers import StaticCache
    from bf16_huffman_infer_b200 import CompressedLinear, convert_all_linear, get_graphed_model, get_model_size

    cfg, model = _tiny_model()
    before = get_model_size(model)
    ids = torch.randint(0, cfg.vocab_size, (batch, 8), generator=torch.Generator().manual_seed(0))

    model.to(DEV)
    with torch.no_grad():
        raw_logits = model(ids.to(DEV)).logits.float().cpu()
    model.cpu()

    convert_all_linear(model, min_out_features=256, progress=False, algo="smallest")
    n_comp = sum(isinstance(m, CompressedLinear) for m in model.modules())
    assert n_comp >= 10            # a layer whose compressed form is not smaller stays an nn.Linear
    assert get_model_size(model) < before
    model.to(DEV)
    with torch.no_grad():
        logits = model(ids.to(DEV)).logits.float().cpu()       # 8 (or 16) rows: fused kernel / decode + GEMM
    scale = raw_logits.pow(2).mean().sqrt()
    assert (logits - raw_logits).abs().max() / scale < 0.05          # BF16 rounding differences through 2 layers

    cache = StaticCache(config=cfg, max_cache_len=64)
    opts = dict(max_new_tokens=12, min_new_tokens=12, do_sample=False, output_logits=True, return_dict_in_generate=True)
    eager = model.generate(ids.to(DEV), past_key_values=cache, disable_compile=True, **opts)
    graphed = get_graphed_model(model, cache)
    assert graphed is not model
    assert next(graphed.parameters()).data_ptr() == next(model.parameters()).data_ptr()
    runs = [graphed.generate(ids.to(DEV), **opts) for _ in range(2)]          # the second run reuses the captured graph
    # the call the reference's example makes: tokenizer-style inputs with an attention mask
    runs.append(graphed.generate(input_ids=ids.to(DEV), attention_mask=torch.ones_like(ids).to(DEV), **opts))
    for i, run in enumerate(runs):
        assert _same_decoding(run, eager, i) >= 1
        assert torch.equal(run.sequences, runs[0].sequences)          # graph replays are reproducible bit for bit
    stats = graphed.graph_stats
    assert stats["captures"] == 1, stats                               # one graph for this batch size ...
    assert stats["replays"] >= 3 * 9 and stats["eager_steps"] == 0, stats     # ... replayed for the one-token steps of all three runs
    # a hand-driven loop without mask or position ids (the same kernels as the captured step): identical tokens
    cache.reset()
    with torch.no_grad():
        tok = model(input_ids=ids.to(DEV), past_key_values=cache, use_cache=True).logits[:, -1:].argmax(-1)
        mine = [tok]
        for _ in range(11):
            tok = model(input_ids=tok, past_key_values=cache, use_cache=True).logits[:, -1:].argmax(-1)
            mine.append(tok)
    assert torch.equal(torch.cat(mine, 1).cpu(), runs[0].sequences[:, ids.shape[1]:].cpu())


def test_fused_siblings_give_the_same_tokens():
    """q/k/v and gate/up stacked into single compressed weights: same logits as the unfused
    compressed model up to BF16 rounding, graph-capturable, identical greedy tokens eager vs graphed."""
    from transformers import StaticCache
    from bf16_huffman_infer_b200 import FusedCompressedLinear, convert_all_linear, get_graphed_model

    cfg, model = _tiny_model(seed=1)
    ids = torch.randint(0, cfg.vocab_size, (1, 8), generator=torch.Generator().manual_seed(1))
    model.to(DEV)
    with torch.no_grad():
        raw_logits = model(ids.to(DEV)).logits.float().cpu()
    model.cpu()
    convert_all_linear(model, min_out_features=256, progress=False, algo="huffman", fuse_siblings=True)
    fused = [m for m in model.modules() if isinstance(m, FusedCompressedLinear)]
    assert len(fused) == 2 * cfg.num_hidden_layers
    assert fused[0].weight.shape[0] == (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    model.to(DEV)
    with torch.no_grad():
        logits = model(ids.to(DEV)).logits.float().cpu()
    assert (logits - raw_logits).abs().max() / raw_logits.pow(2).mean().sqrt() < 0.05
    cache = StaticCache(config=cfg, max_cache_len=64)
    opts = dict(max_new_tokens=10, min_new_tokens=10, do_sample=False, output_logits=True, return_dict_in_generate=True)
    eager = model.generate(ids.to(DEV), past_key_values=cache, disable_compile=True, **opts)
    graphed = get_graphed_model(model, cache)
    out = graphed.generate(ids.to(DEV), **opts)
    assert _same_decoding(out, eager, "fused") >= 1
    assert graphed.graph_stats["replays"] >= 8


def test_decode_bench_example_runs():
    """The whole-model example on a cut-down architecture: runs, reports both arms and a smaller model."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "bf16_huffman_infer_b200.examples.decode_bench", "--arch", "qwen3-1.7b",
                          "--layers", "2", "--tokens", "8", "--prompt", "4"], cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["dense_bf16_tokens_per_s"] > 0 and line["compressed_tokens_per_s"] > 0
    assert line["model_bytes_compressed"] < line["model_bytes_bf16"]


def test_checkpoint_reload_runs_the_same(tmp_path):
    """save_compressed -> load_compressed into a freshly built model -> .cuda() -> forward: the same logits bit for
    bit as the model that was saved, stacked q/k/v and gate/up layers included, and the same decoded tokens."""
    from transformers import Qwen3ForCausalLM, StaticCache
    from bf16_huffman_infer_b200 import (CompressedLinear, convert_all_linear, get_graphed_model, load_compressed,
                                         save_compressed)
    from bf16_huffman_infer_b200.functional import _FusedSlice

    cfg, model = _tiny_model(seed=2)
    ids = torch.randint(0, cfg.vocab_size, (2, 8), generator=torch.Generator().manual_seed(2))
    convert_all_linear(model, min_out_features=256, progress=False, algo="smallest", fuse_siblings=True)
    path = str(tmp_path / "tiny.safetensors")
    save_compressed(model, path)
    model.to(DEV)
    with torch.no_grad():
        want = model(ids.to(DEV)).logits.cpu()
        want1 = model(ids[:1, :1].to(DEV)).logits.cpu()          # one row: the fused kernels

    torch.manual_seed(123)
    fresh = Qwen3ForCausalLM(cfg).to(torch.bfloat16).eval()       # other random weights: everything must come from the file
    load_compressed(fresh, path)
    assert sum(isinstance(m, (CompressedLinear, _FusedSlice)) for m in fresh.modules()) >= 10
    fresh.to(DEV)
    with torch.no_grad():
        assert torch.equal(fresh(ids.to(DEV)).logits.cpu(), want)
        assert torch.equal(fresh(ids[:1, :1].to(DEV)).logits.cpu(), want1)
    cache = StaticCache(config=cfg, max_cache_len=64)
    opts = dict(max_new_tokens=6, min_new_tokens=6, do_sample=False)
    a = get_graphed_model(model, cache).generate(ids.to(DEV), **opts).cpu()
    b = get_graphed_model(fresh, cache).generate(ids.to(DEV), **opts).cpu()
    assert torch.equal(a, b)


@pytest.mark.parametrize("batch", [8, 16])
def test_qwen2_architecture_smallest_coder(batch):
    """The second model configuration of the benchmark, two layers deep: Qwen2.5-7B widths (hidden 3584, intermediate
    18944 - four K-chunks of 4736 columns in down_proj - 28 / 4 heads, q/k/v WITH bias), algo='smallest', decoding at
    batch 8 (fused kernels) and batch 16 (decode to dense, then a library GEMM), eager and through the captured step."""
    from transformers import Qwen2Config, Qwen2ForCausalLM, StaticCache
    from bf16_huffman_infer_b200 import ANSWeight, CompressedLinear, HuffmanWeight, convert_all_linear, get_graphed_model

    cfg = Qwen2Config(vocab_size=2048, hidden_size=3584, intermediate_size=18944, num_hidden_layers=2,
                      num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=256, rope_theta=1e6,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    model = Qwen2ForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name:
                p.fill_(1.0)
            else:
                p.copy_((torch.randn(p.shape) * 0.02).to(torch.bfloat16))
    assert model.model.layers[0].self_attn.q_proj.bias is not None
    ids = torch.randint(0, cfg.vocab_size, (batch, 8), generator=torch.Generator().manual_seed(0))
    opts = dict(max_new_tokens=6, min_new_tokens=6, do_sample=False, output_logits=True, return_dict_in_generate=True)
    model.to(DEV)
    cache = StaticCache(config=cfg, max_cache_len=32)
    raw = model.generate(ids.to(DEV), past_key_values=cache, disable_compile=True, **opts)
    model.cpu()

    convert_all_linear(model, min_out_features=512, progress=False, algo="smallest")
    comp = [m for m in model.modules() if isinstance(m, CompressedLinear)]
    assert len(comp) == 2 * 7 + 1                                  # every projection and the output head
    assert {type(m.weight) for m in comp} <= {HuffmanWeight, ANSWeight}
    down = model.model.layers[0].mlp.down_proj
    assert tuple(down.weight.rem.shape) == (4, 3584, 4736)
    model.to(DEV)
    cache.reset()
    eager = model.generate(ids.to(DEV), past_key_values=cache, disable_compile=True, **opts)
    # the maximum over batch x vocabulary logits of a model this wide sits a little above the two-layer toy's
    assert _same_decoding(eager, raw, "compressed vs bf16", tol=0.1) >= 1
    graphed = get_graphed_model(model, cache)
    out = graphed.generate(ids.to(DEV), **opts)
    assert _same_decoding(out, eager, "graphed vs eager", tol=0.1) >= 1
    assert graphed.graph_stats["replays"] >= 4 and graphed.graph_stats["eager_steps"] == 0
