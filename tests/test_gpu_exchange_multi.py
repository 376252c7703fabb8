"""Exchange kernels across two GPUs of one node: one process per GPU, outputs written into the peers'
symmetric memory over NVLink by the kernel's epilogue.  Needs two visible GPUs; skipped otherwise."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, algo, out):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from bf16_huffman_infer_b200 import ANSWeight, CompressedLinear, HuffmanWeight
        from bf16_huffman_infer_b200.tensor_parallel import PeerArena, PeerRowShardedLinear
        cls = HuffmanWeight if algo == "huffman" else ANSWeight
        g = torch.Generator().manual_seed(0)                                  # same weights on every rank
        shapes = [(1024, 2048), (2048, 1024), (512, 2048)]
        fulls, peers = [], []
        arena = PeerArena(dev)
        for M, K in shapes:
            W = (torch.randn(M, K, generator=g) * 0.02).to(torch.bfloat16)
            full = CompressedLinear(cls.compress(W), None)
            peers.append(PeerRowShardedLinear.from_full(full, arena).to(dev))
            fulls.append(full.to(dev))
        arena.commit()

        def chain(mods, x):                                                   # 2048 -> 1024 -> 2048 -> 512
            return mods[2](mods[1](mods[0](x)))

        ok = True
        for B in (1, 3, 8):
            x = torch.randn(B, 2048, generator=g).to(torch.bfloat16).to(dev)
            with torch.no_grad():
                for _ in range(3):                                            # repeated calls reuse the same buffers
                    want = chain(fulls, x)
                    got = chain(peers, x).clone()
                    ok = ok and torch.equal(want, got)
        # the same chain inside a CUDA graph, replayed
        x = torch.randn(1, 2048, generator=g).to(torch.bfloat16).to(dev)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            chain(peers, x)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph), torch.no_grad():
            y = chain(peers, x)
        with torch.no_grad():
            want = chain(fulls, x)
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        ok = ok and torch.equal(want, y)
        import ctypes
        from bf16_huffman_infer_b200 import _build
        lib = ctypes.CDLL(_build.LIB_PATH)
        status = ctypes.c_int(-1)
        lib.bhi_debug_status(ctypes.byref(status))
        ok = ok and status.value == 0
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            out.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


def _model_worker(rank, world, port, out):
    """A small decoder: convert (siblings stacked), shard every layer over the ranks, compare logits and the
    graphed greedy tokens with the unsharded compressed model."""
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import copy
        from transformers import Qwen3Config, Qwen3ForCausalLM, StaticCache
        from bf16_huffman_infer_b200 import convert_all_linear, get_graphed_model
        from bf16_huffman_infer_b200.tensor_parallel import PeerArena, PeerRowShardedLinear, shard_model_linears
        cfg = Qwen3Config(vocab_size=2048, hidden_size=2048, intermediate_size=6144, num_hidden_layers=2,
                          num_attention_heads=16, num_key_value_heads=2, head_dim=128, max_position_embeddings=256,
                          rope_theta=1e6, tie_word_embeddings=False)
        torch.manual_seed(0)
        model = Qwen3ForCausalLM(cfg).to(torch.bfloat16).eval()
        with torch.no_grad():
            for name, p in model.named_parameters():
                p.fill_(1.0) if "norm" in name else p.copy_((torch.randn(p.shape) * 0.02).to(torch.bfloat16))
        convert_all_linear(model, min_out_features=256, progress=False, algo="huffman", fuse_siblings=True)
        sharded = copy.deepcopy(model)
        model.to(dev)
        arena = PeerArena(dev)
        shard_model_linears(sharded, rank, world, arena=arena)
        sharded.to(dev)
        arena.commit()
        n_peer = sum(isinstance(m, PeerRowShardedLinear) for m in sharded.modules())
        ids = torch.randint(0, cfg.vocab_size, (1, 8), generator=torch.Generator().manual_seed(0)).to(dev)
        with torch.no_grad():
            a = model(ids).logits.float()
            b = sharded(ids).logits.float()
        ok = n_peer >= 6 and bool((a - b).abs().max() / a.pow(2).mean().sqrt() < 0.02)
        # one-token steps under a CUDA graph: same greedy tokens as the unsharded model
        ca, cb = StaticCache(config=cfg, max_cache_len=64), StaticCache(config=cfg, max_cache_len=64)
        ta = get_graphed_model(model, ca).generate(ids, max_new_tokens=8, min_new_tokens=8, do_sample=False)
        tb = get_graphed_model(sharded, cb).generate(ids, max_new_tokens=8, min_new_tokens=8, do_sample=False)
        ok = ok and torch.equal(ta, tb)
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            out.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


def _run(worker, *extra):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, *extra, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    assert out.get(timeout=10) == 1


def test_sharded_model_over_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(_model_worker)


@pytest.mark.parametrize("algo", ["huffman", "ans"])
def test_exchange_over_two_gpus(algo):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(_worker, algo)
