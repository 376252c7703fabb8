"""Benchmark of the fused decode+GEMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload qwen3-8b+fused|qwen3-8b|llama3-70b[+fused]|tiny|layer:MxK|stack:NxMxK]
                    [--algo huffman|ans|smallest] [--tables limit6|escape|reference] [--batch B] [--exchange peer|nccl]

One "step" is one decode token's worth of the hot path: every compressed linear layer of a
decoder of the named shape applied once, in model order, to a batch of B activation rows (B = 1
by default).  Weights are synthetic stand-ins for the checkpoints the reference benchmarks
(N(0, 0.02) BF16, one seed per matrix, generated on the device and checked bit-exact after
decode); attention, norms and sampling are not part of the path and are not run.

Printed JSON line (rank 0):
  value    decode tokens/s with activations resident on the device, whole step replayed as one
           CUDA graph, CUDA-event timed, max over ranks;
  e2e      the same step through the Python module API with the activations coming from pinned
           host memory every step and the last layer's output read back to the host;
  roofline algorithmic compressed bytes per launch / average launch time of the fused kernel,
           against the measured HBM copy bandwidth of MEASURED_PEAKS.json;
  cpu_baseline  the CPU restatement of the reference's fused path (oracle/, all host threads) on a
           bounded sample of the same workload;
  other_tables  (one GPU, Huffman) the same stack encoded with the other table builders ("escape": smallest;
           "reference": the reference's own, byte-identical buffers), timed the same way;
  ans      the same stack with the rANS coder at 8 (the reference's), 10 and 12 probability bits;
  batch_sweep  tokens/s of the same stack at batch 1, 2, 4, 8 with the uncompressed torch stack beside each;
  per_shape  every Qwen3-8B linear shape x both coders on its own: time per launch over more than L2 of distinct
           copies, compressed GB/s, fraction of the measured HBM peak;
  reference_gpu  the reference's own kernels built for sm_100a on the same shapes (a subprocess);
  llama3_70b  the Llama-3-70B-shape stack, timed the same way (rows sharded over the ranks when N > 1);
  dense_bf16_torch  the uncompressed stack as torch nn.Linear layers on the same GPU.
With N > 1 one extra, untimed step compares every layer's exchanged output with an NCCL all-gather of the
ranks' slices (`exchange_verified`).
`--impl reference` times the CPU path alone and prints the same line shape.
With N > 1 (launched under torchrun) every layer is sharded by output rows across the ranks; the
slices are put together by the kernel's own epilogue (stores into every rank's buffer over NVLink,
`--exchange peer`, the default) or by an NCCL all-gather (`--exchange nccl`).  Strong scaling: the
model is fixed.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np
import torch

WORKLOADS = {
    # name: (layers, hidden, intermediate, q_heads, kv_heads, head_dim, vocab)
    "qwen3-8b": (36, 4096, 12288, 32, 8, 128, 151936),
    "llama3-70b": (80, 8192, 28672, 64, 8, 128, 128256),
    "qwen2.5-7b": (28, 3584, 18944, 28, 4, 128, 152064),
    "tiny": (2, 1024, 3072, 8, 2, 128, 8192),
}
# DRAM bytes read + written per launch / algorithmic bytes of the fused Huffman GEMV, from the ncu capture
# summarised in profiles/quad_gemv_huffman_12288x4096_b1.md (dram__bytes_read.sum + dram__bytes_write.sum)
TRAFFIC_OVER_ALGORITHMIC = 1.0046
QWEN3_SHAPES = {"q_o": (4096, 4096), "k_v": (1024, 4096), "gate_up": (12288, 4096), "down": (4096, 12288)}


def host_threads():
    """Cores this process may use (launchers export OMP_NUM_THREADS=1, which must not shrink the CPU arm)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def load_by_path(name, rel):
    """A pure-Python module of the package by file path: the CPU arm must not load the package's native libraries."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def fuse_shapes(shapes):
    """Stack q/k/v and gate/up of every block (one launch each), as convert_all_linear(fuse_siblings=True) does."""
    out, i = [], 0
    while i < len(shapes):
        name, m, k = shapes[i]
        kind = name.split(".")[-1]
        group = {"q_proj": ("q_proj", "k_proj", "v_proj"), "gate_proj": ("gate_proj", "up_proj")}.get(kind)
        if group and [s[0].split(".")[-1] for s in shapes[i:i + len(group)]] == list(group):
            rows = sum(s[1] for s in shapes[i:i + len(group)])
            out.append((name.rsplit(".", 1)[0] + "." + "+".join(group), rows, k))
            i += len(group)
        else:
            out.append(shapes[i])
            i += 1
    return out


def layer_shapes(name):
    if name.endswith("+fused"):
        return fuse_shapes(layer_shapes(name[:-6]))
    if name.startswith("layer:"):                      # a single matrix, e.g. layer:4096x4096
        m, k = (int(v) for v in name[6:].split("x"))
        return [("layers.0.single", m, k)]
    if name.startswith("stack:"):                      # N distinct matrices of one shape, e.g. stack:8x12288x4096:
        n, m, k = (int(v) for v in name[6:].split("x"))  # small, yet larger than L2 (for profiler captures)
        return [(f"layers.{i}.single", m, k) for i in range(n)]
    L, h, inter, qh, kvh, hd, vocab = WORKLOADS[name]
    per_layer = [("q_proj", qh * hd, h), ("k_proj", kvh * hd, h), ("v_proj", kvh * hd, h), ("o_proj", h, qh * hd),
                 ("gate_proj", inter, h), ("up_proj", inter, h), ("down_proj", h, inter)]
    shapes = []
    for i in range(L):
        shapes += [(f"layers.{i}.{n}", m, k) for n, m, k in per_layer]
    shapes.append(("lm_head", vocab, h))
    return shapes


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.rows = []
        self.proc = None
        self.index = index

    def __enter__(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "window": "timed region, then the same replay for 0.5 s"}


# ---- the CPU arm (oracle): bounded sample of the workload ------------------------------------------------
def cpu_arm(workload, algo, batch, budget_s=12.0, tables="reference", ans_precision=8):
    """Times the CPU restatement of the fused path on the first matrices of the stack, in model order,
    until about `budget_s` seconds of CPU work have been measured, and scales to a whole step by
    weight count."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    RANSEncoder = load_by_path("_bench_ans_tables", "bf16_huffman_infer_b200/ans.py").RANSEncoder
    LUTHuffmanEncoder = load_by_path("_bench_huffman_tables", "bf16_huffman_infer_b200/huffman.py").LUTHuffmanEncoder
    oracle.set_threads(host_threads())

    def tables_for_bits(a, bits):
        hist = oracle.histogram(bits)
        if a == "huffman":
            enc = LUTHuffmanEncoder()
            enc.build_lut(hist, method=tables)
            return {"LUT1": enc.LUT1, "LUT2": enc.LUT2, "LUT3": enc.LUT3, "LUT4": enc.LUT4,
                    "code_lengths": enc.code_lengths, "code_values": enc.code_values}
        enc = RANSEncoder([int(v) for v in hist], precision=ans_precision)
        lut = np.array([(s << 24) | (f << 12) | r for s, f, r in enc.decode_lut], dtype=np.uint32)
        return {"freq": np.array(enc.freq, np.uint32), "cum": np.array(enc.cum, np.uint32), "LUT": lut.view(np.int32)}

    shapes = layer_shapes(workload)
    total_weights = sum(m * k for _, m, k in shapes)
    timed_weights, seconds, used = 0, 0.0, []
    for idx, (name, M, K) in enumerate(shapes):
        g = torch.Generator().manual_seed(idx)
        W = (torch.randn(M, K, dtype=torch.float32, generator=g) * 0.02).to(torch.bfloat16)
        Wb = W.view(torch.int16).numpy().view(np.uint16)
        a = "huffman" if algo == "smallest" else algo
        tabs = tables_for_bits(a, Wb)
        rem, exp, offsets, _ = oracle.compress(Wb, a, tabs)
        x = torch.randn(batch, K, generator=g).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
        t0 = time.perf_counter()
        oracle.gemv(a, rem, exp, offsets, tabs, x)
        seconds += time.perf_counter() - t0
        timed_weights += M * K
        used.append(name)
        if seconds > budget_s:
            break
    step_seconds = seconds * total_weights / timed_weights
    return {
        "value": batch / step_seconds, "unit": "tokens/s", "cores": oracle.threads(), "kind": "port",
        "sample": f"first {len(used)} matrices of the stack ({used[0]} .. {used[-1]}; {timed_weights / 1e6:.0f}M of "
                  f"{total_weights / 1e6:.0f}M weights), {seconds:.1f} s of CPU time measured, scaled by weight count",
    }, step_seconds


# ---- our arm ------------------------------------------------------------------------------------------
def build_stack(workload, algo, rank, world, dev, verify=True, exchange="peer"):
    """Compress every matrix of the stack on the device; returns modules, shapes and byte counts."""
    from bf16_huffman_infer_b200 import ANSWeight, CompressedLinear, HuffmanWeight
    from bf16_huffman_infer_b200.tensor_parallel import PeerArena, PeerRowShardedLinear, RowShardedLinear, shard_rows

    mods, meta = [], []
    arena = PeerArena(dev) if world > 1 and exchange == "peer" else None
    for idx, (name, M, K) in enumerate(layer_shapes(workload)):
        g = torch.Generator(device=dev).manual_seed(idx)
        W = (torch.randn(M, K, dtype=torch.float32, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        if algo == "huffman":
            cw = HuffmanWeight.compress(W, to_cpu=False)
        elif algo == "ans":
            cw = ANSWeight.compress(W, to_cpu=False)
        else:
            cands = [HuffmanWeight.compress(W, to_cpu=False), ANSWeight.compress(W, to_cpu=False)]
            cw = min(cands, key=lambda w: w.nbytes())
        if world > 1:
            assert M % world == 0, f"{name}: {M} rows do not divide across {world} ranks"
            cw = shard_rows(cw, rank, world)
        if verify:
            lo, hi = (M * rank // world, M * (rank + 1) // world)
            assert torch.equal(cw.get_weight().view(torch.int16), W[lo:hi].view(torch.int16)), f"{name}: decode is not bit-exact"
        lin = CompressedLinear(cw, None)
        if world == 1:
            mod = lin
        elif arena is not None:
            mod = PeerRowShardedLinear(lin, M, arena)
        else:
            mod = RowShardedLinear(lin, M)
        mods.append(mod)
        info = {"name": name, "M": M, "K": K, "local_rows": cw.shape[0], "bytes": cw.nbytes(), "algo": cw.algo}
        if "+" in name:                                   # stacked siblings: remember where the first one ends
            L_, h_, inter_, qh_, kvh_, hd_, _v = WORKLOADS[workload.replace("+fused", "")]
            if name.endswith("q_proj+k_proj+v_proj"):
                info["q_rows"] = qh_ * hd_
            else:
                info["first_rows"] = inter_
        meta.append(info)
        del W
    if arena is not None:
        # Peer-mapped memory needs every rank to succeed; if any cannot map it, all fall back to the all-gather.
        import torch.distributed as dist
        ok = torch.ones(1, device=dev)
        try:
            arena.commit()
        except Exception as e:                                    # noqa: BLE001  (report and fall back)
            print(f"[bench] rank {rank}: peer memory unavailable ({e}); using the NCCL all-gather", file=sys.stderr)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            mods = [RowShardedLinear(m.local, m.out_features) for m in mods]
            meta[0]["exchange_fallback"] = True
    return mods, meta


def run_step(mods, meta, xs, batch):
    """One pass over the stack.  Activations follow the model's data flow where shapes allow
    (o_proj eats q_proj's output, down_proj eats gate_proj's); the rest read the hidden state."""
    h = xs["hidden"]
    out = None
    q = gate = None
    for mod, info in zip(mods, meta):
        kind = info["name"].split(".")[-1]
        if kind == "o_proj":
            out = mod(q)
        elif kind == "down_proj":
            out = mod(gate)
        else:
            out = mod(h)
            if kind.startswith("q_proj"):
                q = out[..., :info["q_rows"]] if "q_rows" in info else out
            elif kind.startswith("gate_proj"):
                gate = out[..., :info["first_rows"]] if "first_rows" in info else out
    return out


def capture_step(mods, meta, xs, B):
    """Warm up eagerly (this also folds the decode tables), then capture one pass over the stack as a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(2):
            run_step(mods, meta, xs, B)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), torch.no_grad():
        y_static = run_step(mods, meta, xs, B)
    return graph, y_static


def timed_region(fn, steps, world, dev):
    """CUDA-event time of `steps` calls of fn, bracketed by barrier + synchronize, max over ranks (ms)."""
    import torch.distributed as dist

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def quick_tokens_per_s(mods, meta, dev, B, steps, world=1):
    """tokens/s of the stack at batch B (graph replay, activations resident): for the sweeps beside the headline."""
    hidden = meta[0]["K"] if "K" in meta[0] else mods[0].in_features
    xs = {"hidden": torch.randn(B, hidden, device=dev).to(torch.bfloat16)}
    graph, _ = capture_step(mods, meta, xs, B)
    for _ in range(3):
        graph.replay()
    ms = timed_region(graph.replay, steps, world, dev) / steps
    del graph
    return B / (ms * 1e-3), ms


def verify_exchange(mods, meta, xs, B, world):
    """One untimed pass: every layer's exchanged output against an NCCL all-gather of the ranks' own slices."""
    import torch.distributed as dist
    ok = True
    with torch.no_grad():
        h = xs["hidden"]
        q = gate = None
        for mod, info in zip(mods, meta):
            kind = info["name"].split(".")[-1]
            x = q if kind == "o_proj" else gate if kind == "down_proj" else h
            full = mod(x).clone()
            part = mod.local(x).contiguous()
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            ok = ok and torch.equal(full, torch.cat(parts, dim=-1))
            if kind.startswith("q_proj"):
                q = full[..., :info["q_rows"]] if "q_rows" in info else full
            elif kind.startswith("gate_proj"):
                gate = full[..., :info["first_rows"]] if "first_rows" in info else full
    flag = torch.tensor([1.0 if ok else 0.0], device=xs["hidden"].device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item() == 1.0)


def ours(args, rank, world, dev, light=False):
    """Builds and times one stack.  light=True: device-resident timing only (for the side runs)."""
    from bf16_huffman_infer_b200 import set_ans_precision, set_huffman_tables

    t_setup = time.time()
    set_huffman_tables(args.tables)
    set_ans_precision(args.ans_precision)
    mods, meta = build_stack(args.workload, args.algo, rank, world, dev, exchange=args.exchange)
    hidden = meta[0]["K"]
    B = args.batch
    g = torch.Generator().manual_seed(12345)
    x_host = torch.randn(B, hidden, generator=g).to(torch.bfloat16).pin_memory()
    xs = {"hidden": x_host.to(dev)}
    torch.cuda.synchronize()
    setup_s = time.time() - t_setup

    graph, y_static = capture_step(mods, meta, xs, B)
    y_host = torch.empty(y_static.shape, dtype=y_static.dtype).pin_memory()

    def e2e_step():
        xs["hidden"].copy_(x_host, non_blocking=True)
        graph.replay()
        y_host.copy_(y_static, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    steps = max(3, args.steps // 4) if light else args.steps
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    with ClockSampler(dev.index) as clocks:
        ms = timed_region(graph.replay, steps, world, dev)
        if not light:
            # A short timed region (tens of milliseconds at N = 8) ends before nvidia-smi has printed a line: keep the same
            # load running, untimed, for half a second.  The count comes from the rank-maximum time, so every rank replays
            # the same number of steps (the exchange kernels need all of them).
            extra = max(1, int(0.5 / max(ms / steps * 1e-3, 1e-6)))
            for _ in range(extra):
                graph.replay()
            torch.cuda.synchronize()
    ms_e2e = None
    if not light:
        for _ in range(2):
            e2e_step()
        ms_e2e = timed_region(e2e_step, steps, world, dev)

    ms_step = ms / steps
    launches_per_step = len(mods)
    alg_bytes = sum(m["bytes"] + B * m["K"] * 2 + B * m["local_rows"] * 2 for m in meta)
    peak, peak_kind = peaks()
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    total_bytes_all_ranks = alg_bytes * world
    line = {
        "metric": "decode tokens/s (hot path: all compressed linear layers of one token)", "value": B / (ms_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 weights decoded from u8+entropy-coded u8, fp32 accumulate",
        "data": "synthetic", "impl": "ours",
        "config": {
            "workload": f"{args.workload}-shape linear stack ({len(mods)} matrices, {sum(m['M'] * m['K'] for m in meta) / 1e9:.2f}G weights), "
                        f"batch {B}, algo {args.algo}"
                        + (f" ({args.tables} table builder)" if args.algo != "ans" else "") + f", rows sharded over {world} GPU(s)",
            "batch": B, "algo": args.algo, "tables": args.tables if args.algo != "ans" else f"{args.ans_precision}-bit model", "l2": "inputs larger than L2 (the step streams every compressed weight once)",
            "compressed_bytes_per_rank": int(sum(m["bytes"] for m in meta)),
            "ratio": sum(m["bytes"] for m in meta) / (2.0 * sum(m["local_rows"] * m["K"] for m in meta)),
            "setup_s": round(setup_s, 1),
            "exchange": ("none (one GPU)" if world == 1 else
                         "results stored into every rank's buffer by the kernel's epilogue (peer memory over NVLink)"
                         if args.exchange == "peer" and not meta[0].get("exchange_fallback") else "NCCL all-gather after every matrix"),
        },
        "gpu_launches": launches_per_step * steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": alg_bytes / launches_per_step * TRAFFIC_OVER_ALGORITHMIC,
                     "traffic_source": "algorithmic bytes x 1.0046, the ratio of dram__bytes_read.sum + dram__bytes_write.sum to "
                                       "algorithmic bytes in profiles/quad_gemv_huffman_12288x4096_b1.md",
                     "algorithmic_bytes_per_launch": alg_bytes / launches_per_step,
                     "avg_launch_us": ms_step * 1e3 / launches_per_step,
                     "frac_of_nominal_8tbs": achieved / 8000.0,
                     "kernel": ("quad_kernel<HuffCodec, B, 2> (four weight rows per warp group, one mma.sync tile per block for all rows of X)"
                                if args.algo == "huffman" and args.tables.startswith("limit") and B > 0 else
                                "quad_kernel / staged_kernel by table kind and batch")},
        "clocks": clocks.summary(),
    }
    if ms_e2e is not None:
        line["e2e"] = {"value": B / (ms_e2e / steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(x_host.numel() * 2),
                       "d2h_bytes_per_step": int(y_host.numel() * 2)}
    if world > 1:
        line["config"]["aggregate_compressed_gbs"] = total_bytes_all_ranks / (ms_step * 1e-3) / 1e9
        if all(hasattr(m, "local") for m in mods):
            line["exchange_verified"] = verify_exchange(mods, meta, xs, B, world)
    del graph
    return line, mods, meta, xs


def side_run(args, rank, world, dev, **override):
    """The same measurement with some options changed, reduced to its headline figures; frees the stack."""
    alt = argparse.Namespace(**{**vars(args), **override})
    other, m2, _, x2 = ours(alt, rank, world, dev, light=True)
    del m2, x2
    torch.cuda.empty_cache()
    out = {"value": other["value"], "unit": "tokens/s", "ms_per_step": other["ms_per_step"], "ratio": other["config"]["ratio"],
           "frac": other["roofline"]["frac"], "batch": other["config"]["batch"]}
    if "exchange_verified" in other:
        out["exchange_verified"] = other["exchange_verified"]
    return out


def per_shape_arm(dev, steps=5):
    """Every Qwen3-8B linear shape x both coders on its own: graph replay over more than L2 of distinct copies."""
    import math
    from bf16_huffman_infer_b200 import ANSWeight, CompressedLinear, HuffmanWeight
    peak, _ = peaks()
    rows = []
    for name, (M, K) in QWEN3_SHAPES.items():
        g = torch.Generator(device=dev).manual_seed(0)
        W = (torch.randn(M, K, dtype=torch.float32, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        for algo, cls in (("huffman", HuffmanWeight), ("ans", ANSWeight)):
            cw = cls.compress(W, to_cpu=False)
            nbytes = cw.nbytes()
            copies = max(2, math.ceil(400e6 / nbytes))
            mods = []
            for i in range(copies):
                twin = cls(cw.rem.clone(), cw.exp.clone(), *[getattr(cw, k) for k in list(cw.kwargs())[2:]])
                mods.append(CompressedLinear(twin, None))
            for B in (1, 8):
                x = torch.randn(B, K, device=dev).to(torch.bfloat16)

                def run(mods=mods, x=x):
                    for m in mods:
                        m(x)

                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side), torch.no_grad():
                    run()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph), torch.no_grad():
                    run()
                for _ in range(3):
                    graph.replay()
                us = timed_region(graph.replay, steps, 1, dev) * 1e3 / (steps * copies)
                alg = nbytes + B * (K + M) * 2
                rows.append({"shape": name, "M": M, "K": K, "algo": algo, "batch": B, "us": round(us, 2),
                             "gbs": round(alg / us / 1e3, 1), "frac": round(alg / us / 1e3 / peak, 3),
                             "ratio": round(nbytes / (2.0 * M * K), 4)})
                del graph
            del mods, cw
        del W
        torch.cuda.empty_cache()
    return rows


def reference_gpu_arm(batch):
    """The reference's own kernels (built for sm_100a, installed under baseline/_ref) in a process of their own."""
    script = os.path.join(ROOT, "baseline", "reference_gpu_arm.py")
    try:
        r = subprocess.run([sys.executable, script, "--batch", str(batch)], capture_output=True, text=True, timeout=420)
        lines = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
        if r.returncode != 0 or not lines:
            return {"unavailable": ("exit %d: " % r.returncode + (r.stderr.strip().splitlines() or ["no output"])[-1])[:300]}
        return json.loads(lines[-1])
    except Exception as e:                                         # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


def dense_arm(args, dev, batches):
    """The same stack as plain BF16 nn.Linear layers (torch / cuBLAS), graph-replayed on the same GPU, at every batch asked for."""
    shapes = layer_shapes(args.workload.replace("+fused", ""))      # an uncompressed model keeps its projections separate
    need = sum(m * k for _, m, k in shapes) * 2
    free, _ = torch.cuda.mem_get_info(dev)
    if need > free * 0.9:
        return {"unavailable": f"needs {need / 1e9:.0f} GB, {free / 1e9:.0f} GB free"}
    mods = []
    for idx, (name, M, K) in enumerate(shapes):
        g = torch.Generator(device=dev).manual_seed(idx)
        lin = torch.nn.Linear(K, M, bias=False, dtype=torch.bfloat16, device=dev)
        with torch.no_grad():
            lin.weight.copy_((torch.randn(M, K, dtype=torch.float32, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        mods.append(lin)
    meta = [{"name": n, "K": k} for n, _, k in shapes]
    out = {}
    for B in batches:
        value, ms_step = quick_tokens_per_s(mods, meta, dev, B, args.steps)
        out[str(B)] = {"value": value, "unit": "tokens/s", "ms_per_step": ms_step, "weight_bytes": need, "gbs": need / (ms_step * 1e-3) / 1e9}
    del mods
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-8b+fused",
                    help="one of %s, optionally with +fused (q/k/v and gate/up stacked into one launch each), "
                         "or layer:MxK for a single matrix, or stack:NxMxK for N distinct matrices of one shape" % sorted(WORKLOADS))
    ap.add_argument("--algo", default="huffman", choices=["huffman", "ans", "smallest"])
    ap.add_argument("--ans-precision", type=int, default=8, choices=[8, 9, 10, 11, 12], help="probability bits of the rANS model")
    ap.add_argument("--tables", default="limit6", choices=["limit6", "limit8", "escape", "reference"],
                    help="Huffman table builder: 'limit6' (the package default: codes of at most 6 bits, fastest), 'escape' "
                         "(near-entropy on every histogram, smallest) or 'reference' (the reference's own code, bit-identical "
                         "compressed bytes); all fill the reference's table format")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="with more than one GPU: how the row slices of every matrix are put together")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-dense", action="store_true", help="skip the uncompressed BF16 torch comparison")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the side measurements (other table builders, rANS, batch sweep, per-shape, reference kernels, 70B shape)")
    ap.add_argument("--no-70b", action="store_true", help="skip the Llama-3-70B-shape stack")
    args = ap.parse_args()

    # The contract is ONE line on stdout.  Libraries write there too (NCCL prints its version when its first communicator
    # comes up): everything but the result line goes to stderr.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(result_fd, (json.dumps(obj) + "\n").encode())

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        # the reference's CPU path (restated in oracle/), all host threads, rank 0 only
        if rank != 0:
            return
        per_step = []
        base = None
        for _ in range(max(1, min(args.steps, 3))):
            base, step_seconds = cpu_arm(args.workload, args.algo, args.batch, budget_s=12.0, tables=args.tables, ans_precision=args.ans_precision)
            per_step.append(step_seconds)
        step_seconds = float(np.median(per_step))
        base["value"] = args.batch / step_seconds
        emit({
            "metric": "decode tokens/s (hot path: all compressed linear layers of one token)", "value": base["value"],
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(per_step), "warmup": 0, "ms_per_step": step_seconds * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 weights, fp32 accumulate",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": f"{args.workload}-shape linear stack, batch {args.batch}, algo {args.algo}", "batch": args.batch,
                       "algo": args.algo, "tables": args.tables},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        })
        return

    assert torch.cuda.is_available(), "bench.py --impl ours needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    import bf16_huffman_infer_b200  # noqa: F401  (fails loudly if the native libraries are missing)

    line, mods, meta, xs = ours(args, rank, world, dev)
    extras = not args.no_extras
    qwen = args.workload.startswith("qwen3-8b")
    if extras and world == 1:
        # the same stack at the other batch sizes of the fused path
        sweep = {str(args.batch): {"value": line["value"], "ms_per_step": line["ms_per_step"]}}
        for B in (1, 2, 4, 8):
            if str(B) not in sweep:
                v, ms = quick_tokens_per_s(mods, meta, dev, B, max(3, args.steps // 4))
                sweep[str(B)] = {"value": v, "ms_per_step": ms}
        line["batch_sweep"] = sweep
    del mods, xs
    torch.cuda.empty_cache()
    if extras and world == 1 and args.algo == "huffman":
        free, _ = torch.cuda.mem_get_info(dev)
        if line["config"]["compressed_bytes_per_rank"] * 1.4 < free:
            line["other_tables"] = {t: side_run(args, rank, world, dev, tables=t) for t in ("escape", "reference") if t != args.tables}
            # rANS: the reference's 8-bit probabilities and the finer models its table word allows
            line["ans"] = {str(p): side_run(args, rank, world, dev, algo="ans", ans_precision=p) for p in (8, 10, 12)}
        else:
            line["other_tables"] = {"unavailable": "not enough free device memory for a second stack"}
    if extras and world == 1 and qwen:
        line["per_shape"] = per_shape_arm(dev)
    if extras and qwen and not args.no_70b:
        # the 70B shape the tensor-parallel configuration names, same coder and tables, rows sharded over the ranks
        free, _ = torch.cuda.mem_get_info(dev)
        if free > 118e9 / world + 8e9:
            line["llama3_70b"] = side_run(args, rank, world, dev, workload="llama3-70b+fused")
        else:
            line["llama3_70b"] = {"unavailable": f"{free / 1e9:.0f} GB free on the device"}
    if rank == 0:
        if world == 1 and not args.no_dense:
            batches = (1, 2, 4, 8) if "batch_sweep" in line else (args.batch,)
            dense = dense_arm(args, dev, batches)
            if "unavailable" in dense:
                line["dense_bf16_torch"] = dense
            else:
                line["dense_bf16_torch"] = dense[str(args.batch)]
                for B, entry in line.get("batch_sweep", {}).items():
                    entry["dense_bf16_torch"] = dense[B]["value"]
        if extras and world == 1 and qwen:
            line["reference_gpu"] = reference_gpu_arm(args.batch)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], _ = cpu_arm(args.workload, args.algo, args.batch, tables=args.tables, ans_precision=args.ans_precision)
        emit(line)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
