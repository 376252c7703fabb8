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
    eager = _generate(model, cache, ids.to(DEV), 12).cpu()
    graphed = get_graphed_model(model, cache)
    assert graphed is not model
    assert next(graphed.parameters()).data_ptr() == next(model.parameters()).data_ptr()
    for _ in range(2):                                                # second run reuses the captured graph
        out = graphed.generate(ids.to(DEV), max_new_tokens=12, min_new_tokens=12, do_sample=False).cpu()
        assert torch.equal(out, eager)


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
    eager = _generate(model, cache, ids.to(DEV), 10).cpu()
    graphed = get_graphed_model(model, cache)
    out = graphed.generate(ids.to(DEV), max_new_tokens=10, min_new_tokens=10, do_sample=False).cpu()
    assert torch.equal(out, eager)


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
