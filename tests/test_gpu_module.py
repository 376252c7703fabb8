"""The Python surface on a GPU: weight containers, the F.linear hook, both branches (<= 8 rows fused,
> 8 rows decode + GEMM) and the optional tensor-core branch, bias, model surgery, and the per-stream encode operators."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.nn.functional as F
from torch import nn

from _util import ROOT, bits_of, huffman_tables, ans_tables, make_input, make_weight, rel_err

sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-2
DEV = "cuda:0"


@pytest.mark.parametrize("algo,method", [("huffman", "reference"), ("huffman", "limit6"), ("huffman", "escape"), ("ans", None)])
@pytest.mark.parametrize("M,K", [(256, 512), (128, 12288), (384, 4096)])
def test_compress_matches_oracle_and_decodes(algo, method, M, K):
    from bf16_huffman_infer_b200 import ANSWeight, HuffmanWeight, set_huffman_tables
    W = make_weight(M, K, 11)
    cls = HuffmanWeight if algo == "huffman" else ANSWeight
    previous = set_huffman_tables(method) if method else None
    try:
        cw = cls.compress(W)
    finally:
        if method:
            set_huffman_tables(previous)
    assert cw.rem.device.type == "cpu"            # like the reference, compress hands back CPU tensors
    Wb = bits_of(W)
    tabs = huffman_tables(oracle.histogram(Wb), method)[0] if algo == "huffman" else ans_tables(oracle.histogram(Wb))[0]
    rem, exp, offsets, _ = oracle.compress(Wb, algo, tabs)
    assert (cw.rem.numpy() == rem).all() and (cw.exp.numpy() == exp).all() and (cw.offsets.numpy() == offsets).all()
    if algo == "huffman":
        for k in ("LUT1", "LUT2", "LUT3", "LUT4", "code_lengths"):
            assert (getattr(cw, k).numpy() == tabs[k]).all()
    else:
        assert (cw.LUT.numpy() == tabs["LUT"]).all()
    cw = cw.to(DEV)
    assert torch.equal(cw.get_weight().cpu().view(torch.int16), W.view(torch.int16))
    assert set(cw.kwargs()) == ({"rem", "exp", "offsets", "LUT1", "LUT2", "LUT3", "LUT4", "code_lengths"}
                                if algo == "huffman" else {"rem", "exp", "offsets", "LUT"})


@pytest.mark.parametrize("bits", [10, 12])
def test_finer_ans_model_through_the_python_surface(bits, tmp_path):
    """set_ans_precision: compress builds a 2^bits-word table, the operators infer the precision from it, the layer is
    never larger than with 8 bits, and a checkpoint of it loads back."""
    from bf16_huffman_infer_b200 import ANSWeight, checkpoint, convert_all_linear, set_ans_precision
    M, K = 384, 4096
    W = make_weight(M, K, 5)
    Wb = bits_of(W)
    base = ANSWeight.compress(W)
    previous = set_ans_precision(bits)
    try:
        cw = ANSWeight.compress(W)
        model = nn.Sequential(nn.Linear(K, M, bias=False)).to(torch.bfloat16)
        with torch.no_grad():
            model[0].weight.copy_(W)
        convert_all_linear(model, min_out_features=0, algo="ans")
    finally:
        assert set_ans_precision(previous) == bits
    assert cw.LUT.numel() == 1 << bits and cw.exp.numel() <= base.exp.numel()
    tabs = ans_tables(oracle.histogram(Wb), precision=bits)[0]
    rem, exp, offsets, _ = oracle.compress(Wb, "ans", tabs)
    assert (cw.LUT.numpy() == tabs["LUT"]).all() and (cw.exp.numpy() == exp).all() and (cw.offsets.numpy() == offsets).all()
    cw = cw.to(DEV)
    assert torch.equal(cw.get_weight().cpu().view(torch.int16), W.view(torch.int16))
    for B in (1, 8, 24):
        X = make_input(B, K, B)
        y = F.linear(X.to(DEV), cw).float().cpu().numpy()
        assert rel_err(y, oracle.matvec(Wb, bits_of(X))) <= TOL
    path = str(tmp_path / "finer.safetensors")
    checkpoint.save_compressed(model, path)
    fresh = nn.Sequential(nn.Linear(K, M, bias=False)).to(torch.bfloat16)
    checkpoint.load_compressed(fresh, path)
    assert fresh[0].weight.LUT.numel() == 1 << bits
    X = make_input(2, K, 3).to(DEV)
    assert torch.equal(fresh.to(DEV)(X), model.to(DEV)(X))


@pytest.mark.parametrize("algo", ["huffman", "ans"])
def test_linear_hook_both_branches_and_bias(algo):
    from bf16_huffman_infer_b200 import ANSWeight, CompressedLinear, HuffmanWeight
    M, K = 256, 1024
    W = make_weight(M, K, 5)
    bias = make_weight(1, M, 6)[0]
    cls = HuffmanWeight if algo == "huffman" else ANSWeight
    cw = cls.compress(W)
    lin = CompressedLinear(cw, nn.Parameter(bias.clone())).to(DEV)
    plain = CompressedLinear(cw, None).to(DEV)
    assert (lin.out_features, lin.in_features) == (M, K)
    for shape in [(1, K), (8, K), (2, 3, K), (9, K), (4, 8, K), (128, K), (5, 26, K)]:
        rows = int(np.prod(shape[:-1]))
        x = make_input(rows, K, 3).view(shape)
        with torch.no_grad():
            y = lin(x.to(DEV))
            y0 = plain(x.to(DEV))
        assert y.shape == shape[:-1] + (M,) and y.dtype == torch.bfloat16
        ref0 = x.double().view(-1, K) @ W.double().T
        assert rel_err(y0.float().cpu().view(-1, M).numpy(), ref0.numpy()) <= TOL
        if rows <= 8:
            # fused branch: the bias is added to the BF16 result afterwards, as the reference does
            assert torch.equal(y, y0 + lin.bias[None, :].expand_as(y0).reshape(y0.shape))
        else:
            # decode + GEMM branch: bias inside the GEMM epilogue, one rounding
            assert rel_err(y.float().cpu().view(-1, M).numpy(), (ref0 + bias.double()).numpy()) <= TOL


@pytest.mark.parametrize("algo", ["huffman", "ans"])
def test_optional_tensor_core_branch(algo, monkeypatch):
    """With TENSOR_MAX_ROWS raised, 9..128 rows go through the fused tensor-core product."""
    import bf16_huffman_infer_b200.functional as fn
    M, K = 256, 1024
    W = make_weight(M, K, 7)
    bias = make_weight(1, M, 8)[0]
    cls = fn.HuffmanWeight if algo == "huffman" else fn.ANSWeight
    lin = fn.CompressedLinear(cls.compress(W), nn.Parameter(bias.clone())).to(DEV)
    calls = []
    for name in ("mm_huffman_prepared", "mm_ans"):
        real = getattr(fn, name)
        monkeypatch.setattr(fn, name, lambda *a, _real=real, **k: (calls.append(1), _real(*a, **k))[1])
    monkeypatch.setattr(fn, "TENSOR_MAX_ROWS", 128)
    for rows in (9, 64, 128, 130):
        x = make_input(rows, K, rows)
        with torch.no_grad():
            y = lin(x.to(DEV))
        ref = x.double() @ W.double().T + bias.double()
        assert rel_err(y.float().cpu().numpy(), ref.numpy()) <= 2 * TOL          # bias added after a first BF16 rounding
    assert len(calls) == 3                                                        # 130 rows: decode + GEMM


def test_per_stream_operators_match_oracle():
    import bf16_huffman_infer_b200.ops as ops
    W = make_weight(128, 512, 2)
    Wb = bits_of(W)
    hist = oracle.histogram(Wb)
    htabs, henc = huffman_tables(hist)
    atabs, _ = ans_tables(hist)
    _, e = oracle.split(Wb)
    data = np.ascontiguousarray(e[:, :64])
    lut = np.zeros((256, 32), np.uint8)
    for s, code in henc.huffman_codes.items():
        lut[s, : len(code)] = [ord(c) for c in code[::-1]]
    d = torch.from_numpy(data).to(DEV)
    chars = torch.full((128, 64 * 32), ord("0"), dtype=torch.uint8, device=DEV)
    bits = torch.zeros(128, dtype=torch.int32, device=DEV)
    ops.huffman_encode(d, torch.from_numpy(lut).to(DEV), chars, bits)
    oc, ob = oracle.huffman_encode_op(data, lut)
    assert (bits.cpu().numpy() == ob).all() and (chars.cpu().numpy() == oc).all()
    words = torch.zeros(128, 64 * 8, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(128, dtype=torch.int32, device=DEV)
    ops.ans_encode(d, torch.from_numpy(atabs["freq"].view(np.int32)).to(DEV),
                   torch.from_numpy(atabs["cum"].view(np.int32)).to(DEV), words, cnt)
    ow, on = oracle.ans_encode_op(data, atabs["freq"], atabs["cum"])
    assert (cnt.cpu().numpy() == on).all() and (words.cpu().numpy() == ow).all()


@pytest.mark.parametrize("algo", ["huffman", "ans"])
def test_compress_groups_agrees_with_layer_encoder(algo):
    """The operator-driven path of the reference and the two-pass encoder store the same words."""
    from bf16_huffman_infer_b200 import ANSWeight, HuffmanWeight
    from bf16_huffman_infer_b200.utils import split_bf16
    M, K = 128, 512
    W = make_weight(M, K, 8).to(DEV)
    cls = HuffmanWeight if algo == "huffman" else ANSWeight
    codec = cls.get_codec(W)
    _, exp = split_bf16(W)
    x = exp.view(M, -1, 64, 2).transpose(1, 2).reshape(M, 64, -1).contiguous()      # [rows, stream, symbol]
    words, row_words = cls.compress_groups(x, codec)
    cw = cls.compress_split_n(W, n=1)
    words = words.view(M, 64, -1).cpu().numpy()
    for m in range(M):
        L = int(row_words[m])
        rec = cw.exp.numpy()[int(cw.offsets[0, m]): int(cw.offsets[0, m]) + 64 * L].reshape(L, 64)
        assert (rec == words[m, :, :L].T).all(), m


def test_convert_all_linear_on_a_small_model():
    from bf16_huffman_infer_b200 import CompressedLinear, convert_all_linear, get_model_size

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = nn.Linear(2048, 1024, bias=True)
            self.down = nn.Linear(1024, 2048, bias=False)
            self.small = nn.Linear(2048, 64)

        def forward(self, x):
            return self.small(self.down(F.silu(self.up(x))))

    torch.manual_seed(0)
    model = Block().to(torch.bfloat16)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_((torch.randn(p.shape) * 0.02).to(torch.bfloat16))
    x = make_input(4, 2048, 1)
    with torch.no_grad():
        ref = model.to(DEV)(x.to(DEV)).float().cpu()
    model.cpu()
    before = get_model_size(model)
    for algo in ("smallest",):
        convert_all_linear(model, min_out_features=1024, progress=False, algo=algo)
    assert isinstance(model.up, CompressedLinear) and isinstance(model.down, CompressedLinear)
    assert isinstance(model.small, nn.Linear)
    assert model.up.weight.rem.device.type == "cpu"
    assert get_model_size(model) < 0.85 * before
    with torch.no_grad():
        out = model.to(DEV)(x.to(DEV)).float().cpu()
    assert rel_err(out.numpy(), ref.numpy()) <= 2e-2          # two BF16 layers of rounding differences
    sd = model.state_dict()
    assert any(k.startswith("up.weight.rem") for k in sd)


def test_fused_call_is_graph_capturable():
    from bf16_huffman_infer_b200 import CompressedLinear, HuffmanWeight
    W = make_weight(256, 512, 3)
    lin = CompressedLinear(HuffmanWeight.compress(W), None).to(DEV)
    x = make_input(1, 512, 3).to(DEV)
    static_x = x.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s), torch.no_grad():
        for _ in range(2):
            lin(static_x)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g), torch.no_grad():
        static_y = lin(static_x)
    static_x.copy_(make_input(1, 512, 4).to(DEV))
    g.replay()
    torch.cuda.synchronize()
    ref = make_input(1, 512, 4).double() @ W.double().T
    assert rel_err(static_y.float().cpu().numpy(), ref.numpy()) <= TOL
