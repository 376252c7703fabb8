"""Host-side logic of the package that needs no GPU, and the C ABI's export table."""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

from _util import HEADER, LIB, ROOT, bits_of, header_symbols, make_weight

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402


def test_library_exports_every_declared_symbol():
    names = header_symbols()
    assert len(names) >= 12, names
    lib = ctypes.CDLL(LIB)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in {HEADER} but not exported"
    assert lib.bhi_abi_version() >= 1


def test_operator_schemas_registered():
    import bf16_huffman_infer_b200.ops  # noqa: F401
    ns = torch.ops.bf16_huffman_infer
    want = {
        "gemv_bf16_huffman": "(Tensor A_rem, Tensor A_exp, Tensor X, Tensor(a!) Y, Tensor offsets, Tensor LUT1, Tensor LUT2, Tensor LUT3, Tensor LUT4, Tensor code_lengths) -> ()",
        "huffman_encode": "(Tensor data, Tensor LUT, Tensor(a!) output, Tensor(b!) output_lengths) -> ()",
        "huffman_decode": "(Tensor A_rem, Tensor A_exp, Tensor(a!) Y, Tensor offsets, Tensor LUT1, Tensor LUT2, Tensor LUT3, Tensor LUT4, Tensor code_lengths) -> ()",
        "gemv_bf16_ans": "(Tensor A_rem, Tensor A_exp, Tensor X, Tensor(a!) Y, Tensor offsets, Tensor LUT) -> ()",
        "ans_encode": "(Tensor data, Tensor freq, Tensor cum, Tensor(a!) output, Tensor(b!) output_lengths) -> ()",
        "ans_decode": "(Tensor A_rem, Tensor A_exp, Tensor(a!) Y, Tensor offsets, Tensor LUT) -> ()",
    }
    for name, sig in want.items():
        assert str(getattr(ns, name).default._schema) == f"bf16_huffman_infer::{name}{sig}"


def test_no_cpu_kernel_is_registered():
    """Calling an operator with CPU tensors must fail, not fall back."""
    import bf16_huffman_infer_b200.ops as ops
    z = torch.zeros(1, 128, 128, dtype=torch.uint8)
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.ans_decode(z, torch.zeros(64, dtype=torch.int32), torch.zeros(128, 128, dtype=torch.bfloat16),
                       torch.zeros(1, 128, dtype=torch.int32), torch.zeros(256, dtype=torch.int32))


def test_public_names():
    import bf16_huffman_infer_b200 as pkg
    for name in ("convert_all_linear", "convert", "HuffmanWeight", "ANSWeight", "CompressedLinear",
                 "linear_huffman", "get_graphed_model", "get_model_size"):
        assert hasattr(pkg, name), name


def test_split_merge_bf16():
    from bf16_huffman_infer_b200.utils import merge_bf16, split_bf16
    w = make_weight(64, 128, 0)
    w[0, 0] = float("-0.0")
    w[0, 1] = float("inf")
    rem, exp = split_bf16(w)
    orem, oexp = oracle.split(bits_of(w))
    assert (rem.numpy() == orem).all() and (exp.numpy() == oexp).all()
    assert torch.equal(merge_bf16(rem, exp).view(torch.int16), w.view(torch.int16))


def test_chunk_count_matches_oracle():
    from bf16_huffman_infer_b200.utils import chunk_count_for_k, get_block_size_n
    for k in list(range(128, 33000, 128)):
        try:
            s = chunk_count_for_k(k)
        except RuntimeError:
            s = -1
        assert s == oracle.chunk_count(k), k
    assert get_block_size_n(torch.empty(4, 12288)) == (3,)
    with pytest.raises(RuntimeError):
        get_block_size_n(torch.empty(4, 100))


@pytest.mark.parametrize("S,M", [(1, 128), (3, 5000), (2, 8192), (1, 4096), (2, 4097)])
def test_record_offsets_match_oracle(S, M):
    from bf16_huffman_infer_b200.functional import _record_offsets
    rng = np.random.default_rng(S * 1000 + M)
    L = rng.integers(1, 20, (S, M)).astype(np.int32)
    off, total = _record_offsets(torch.from_numpy(L))
    want = np.zeros((S, M), np.int32)
    n = oracle.lib().bhi_oracle_layout_offsets(L.ctypes.data_as(ctypes.c_void_p), S, M, want.ctypes.data_as(ctypes.c_void_p))
    assert total == n and (off.numpy() == want).all()


def test_get_model_size_and_shallow_copy():
    from bf16_huffman_infer_b200.utils import get_model_size, shallow_copy_model
    m = torch.nn.Sequential(torch.nn.Linear(8, 4), torch.nn.BatchNorm1d(4))
    size = get_model_size(m)
    assert size == sum(p.numel() * p.element_size() for p in m.parameters()) + sum(b.numel() * b.element_size() for b in m.buffers())
    c = shallow_copy_model(m)
    assert c is not m and c[0] is not m[0] and c[0].weight is m[0].weight


def test_compressed_checkpoint_roundtrip(tmp_path):
    """save_compressed / load_compressed rebuild the compressed modules (plain and stacked) on the CPU."""
    import numpy as np
    from _util import tables_for
    from bf16_huffman_infer_b200 import CompressedLinear, HuffmanWeight, ANSWeight, load_compressed, save_compressed
    from bf16_huffman_infer_b200.functional import FusedCompressedLinear, _FusedSlice

    def compressed(algo, M, K, seed):
        W = make_weight(M, K, seed)
        Wb = bits_of(W)
        tabs = tables_for(algo, oracle.histogram(Wb))
        rem, exp, offsets, _ = oracle.compress(Wb, algo, tabs)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
        if algo == "huffman":
            return HuffmanWeight(t(rem), t(exp), t(offsets), *[t(tabs[k]) for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths")])
        return ANSWeight(t(rem), t(exp), t(offsets), t(tabs["LUT"]))

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(512, 256, bias=True)
            self.k_proj = torch.nn.Linear(512, 128, bias=True)
            self.o_proj = torch.nn.Linear(512, 512, bias=False)
            self.norm = torch.nn.LayerNorm(512)

    src = Block().to(torch.bfloat16)
    owner = FusedCompressedLinear(compressed("huffman", 384, 512, 1), torch.nn.Parameter(torch.randn(384).to(torch.bfloat16)), [(0, 256), (256, 384)])
    src.q_proj = _FusedSlice(owner, 0, True)
    src.k_proj = _FusedSlice(owner, 1, False)
    src.o_proj = CompressedLinear(compressed("ans", 512, 512, 2), None)
    path = str(tmp_path / "model.safetensors")
    save_compressed(src, path)

    dst = load_compressed(Block().to(torch.bfloat16), path)
    assert isinstance(dst.o_proj, CompressedLinear) and isinstance(dst.o_proj.weight, ANSWeight)
    assert isinstance(dst.q_proj, _FusedSlice) and dst.q_proj.leader and not dst.k_proj.leader
    assert dst.k_proj._owner is dst.q_proj._owner and dst.q_proj._owner.splits == [(0, 256), (256, 384)]
    a, b = src.state_dict(), dst.state_dict()
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k
    # a manifest that does not describe the model it is applied to is refused before anything is replaced
    class Other(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(512, 256, bias=True)
            self.k_proj = torch.nn.Linear(512, 128, bias=True)
            self.o_proj = torch.nn.Linear(256, 512, bias=False)      # other input width
            self.norm = torch.nn.LayerNorm(512)
    other = Other().to(torch.bfloat16)
    with pytest.raises(ValueError, match="does not fit"):
        load_compressed(other, path)
    assert isinstance(other.q_proj, torch.nn.Linear)


@pytest.mark.parametrize("bits", [10, 12])
def test_checkpoint_keeps_the_ans_table_size(tmp_path, bits):
    """A rANS weight built at 10 or 12 probability bits has a 2^bits-word table; the manifest records it, the loader
    rebuilds a buffer of that size, and the decoded weight (CPU oracle) is unchanged by the trip."""
    import numpy as np
    from _util import ans_tables
    from bf16_huffman_infer_b200 import ANSWeight, CompressedLinear, load_compressed, save_compressed
    W = make_weight(128, 512, 5)
    Wb = bits_of(W)
    tabs = ans_tables(oracle.histogram(Wb), precision=bits)[0]
    rem, exp, offsets, _ = oracle.compress(Wb, "ans", tabs)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    src = torch.nn.Sequential(torch.nn.Linear(512, 128, bias=False)).to(torch.bfloat16)
    src[0] = CompressedLinear(ANSWeight(t(rem), t(exp), t(offsets), t(tabs["LUT"])), None)
    path = str(tmp_path / "ans.safetensors")
    save_compressed(src, path)
    dst = load_compressed(torch.nn.Sequential(torch.nn.Linear(512, 128, bias=False)).to(torch.bfloat16), path)
    w = dst[0].weight
    assert isinstance(w, ANSWeight) and w.LUT.numel() == 1 << bits
    back = oracle.decode("ans", w.rem.numpy(), w.exp.numpy(), w.offsets.numpy(), {"LUT": w.LUT.numpy()})
    assert (back == Wb).all()


def test_set_ans_precision_bounds():
    from bf16_huffman_infer_b200 import set_ans_precision
    previous = set_ans_precision(12)
    try:
        assert set_ans_precision(8) == 12
        for bad in (7, 13):
            with pytest.raises(ValueError):
                set_ans_precision(bad)
    finally:
        set_ans_precision(previous)
