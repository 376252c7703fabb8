"""Compressed-weight containers, the ``F.linear`` hook and model surgery.

Public surface and behaviour follow the reference's ``bf16_huffman_infer/functional.py``
(``HuffmanWeight`` :66-242, ``ANSWeight`` :245-310, ``CompressedLinear`` :313-320, ``convert``
:323-375, ``convert_all_linear`` :378-387, ``linear_huffman`` :390-411, ``mv_ans`` / ``linear_ans``
:414-466).  The tensors a weight holds (``rem``, ``exp``, ``offsets`` and the tables) are laid out
exactly as the reference lays them out, byte for byte.

What is different underneath: a layer is encoded by two CUDA passes over the BF16 weight (size
pass, prefix sum of the record sizes, emit pass) instead of expanding every symbol to 32
characters and assembling the format with tensor ops; the per-stream operators the reference
uses for that are still available (``compress_groups``) and produce the same words.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import os

import torch
import torch.nn.functional as F
from torch import Tensor, nn
from tqdm import tqdm

from . import ops
from .ans import RANSEncoder
from .huffman import LUTHuffmanEncoder
from .utils import get_block_size_n, split_bf16

OP_PER_LANE = 1
ANS_PRECISION = 8
SLAB_ROWS = 4096          # rows encoded per slab; 64 padding words follow every slab
FUSED_MAX_ROWS = 8        # up to here: fused decode + GEMV; beyond: decode, then a library GEMM (as the reference)
# Rows up to which the fused decode + tensor-core product (mm_huffman_prepared / mm_ans, at most 128) is used
# instead of decode + GEMM.  Off by default: on B200 it is within 5 % of decode + library GEMM up to 32 rows and
# behind it beyond (python -m bf16_huffman_infer_b200.examples.linear_bench), but needs no dense scratch.
# BHI_TENSOR_ROWS=32 (or up to 128) turns it on.
TENSOR_MAX_ROWS = int(os.environ.get("BHI_TENSOR_ROWS", "0"))
# Which prefix code HuffmanWeight.compress builds (huffman.py; every choice yields tables of the reference's
# format, readable by any decoder of it, the reference's included):
#   "limit6"    (default) optimal code with no length above 6 bits: any two codes fit the 12-bit index of the fused
#               kernels' folded table, so they never leave their two-symbols-per-lookup loop (fastest; about 4 %
#               larger than "escape" on N(0, s) weights; falls back to "escape" beyond 64 distinct exponents);
#   "escape"    escape-byte code, near-entropy on every histogram (smallest);
#   "reference" the reference's own builder, bit for bit (and so its compressed bytes); on some histograms its
#               repair loop lengthens the frequent codes by 2 bits.
# See set_huffman_tables() and convert_all_linear(huffman_tables=...).
HUFFMAN_TABLES = os.environ.get("BHI_HUFFMAN_TABLES", "limit6")


def set_huffman_tables(method: str) -> str:
    """Choose the table builder used by later ``HuffmanWeight.compress`` calls; returns the previous choice."""
    global HUFFMAN_TABLES
    assert method in ("reference", "escape") or (method.startswith("limit") and method[5:].isdigit()), method
    previous, HUFFMAN_TABLES = HUFFMAN_TABLES, method
    return previous


def set_ans_precision(bits: int) -> int:
    """Probability precision (8..12 bits) of the rANS models built by later ``ANSWeight.compress`` calls; returns the
    previous value.  8 is the reference's constant (``functional.py:16``) and what its kernels read; a finer model
    codes the exponents in fewer words but needs a ``2^bits``-word table per weight, which only this package's kernels
    accept (the record and table-word formats are unchanged)."""
    global ANS_PRECISION
    if not 8 <= int(bits) <= 12:
        raise ValueError("rANS precision must be in [8, 12]")
    previous, ANS_PRECISION = ANS_PRECISION, int(bits)
    return previous


__all__ = [
    "linear_huffman",
    "linear_ans",
    "HuffmanWeight",
    "ANSWeight",
    "CompressedLinear",
    "FusedCompressedLinear",
    "convert_all_linear",
    "convert",
    "fuse_sibling_linears",
    "set_huffman_tables",
    "set_ans_precision",
]

# projections that read the same input inside one block of the usual decoder architectures
SIBLING_GROUPS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


def _work_device(a: Tensor) -> torch.device:
    if a.is_cuda:
        return a.device
    if not torch.cuda.is_available():
        raise RuntimeError("bf16_huffman_infer_b200 needs a CUDA device: there is no CPU implementation")
    return torch.device("cuda", torch.cuda.current_device())


def _exp_histogram(a: Tensor) -> Tensor:
    """256 exponent counts of a BF16 tensor (int64, on the CPU)."""
    bits = a.contiguous().view(torch.int16).flatten()
    exp = ((bits >> 7) & 0xFF).to(torch.int64)
    return torch.bincount(exp, minlength=256).cpu()


def _record_offsets(words_per_row: Tensor) -> Tuple[Tensor, int]:
    """Word offset of every record from the per-record row counts ``[S, M]``.

    Records are stored chunk-major with rows ascending; after every slab of ``SLAB_ROWS`` rows (and
    after the last, partial slab of a chunk) 64 zero words are inserted, because a Huffman
    decoder may look one record row past the end of a record (reference ``functional.py:177``,
    ``:204-231``).
    """
    S, M = words_per_row.shape
    sizes = words_per_row.to(torch.int64) * 64
    pad = torch.zeros(M, dtype=torch.int64, device=sizes.device)
    pad[SLAB_ROWS - 1::SLAB_ROWS] = 64
    pad[M - 1] = 64
    sizes = (sizes + pad[None, :]).flatten()
    ends = torch.cumsum(sizes, 0)
    total = int(ends[-1].item())
    if total >= 2 ** 31:
        raise RuntimeError("compressed exponent plane exceeds 2^31 words; split the layer")
    return (ends - sizes).to(torch.int32).view(S, M), total


def mv_huffman(
    A_rem: Tensor, A_exp: Tensor, X: Tensor, offsets: Tensor,
    LUT1: Tensor, LUT2: Tensor, LUT3: Tensor, LUT4: Tensor, code_lengths: Tensor,
) -> Tensor:
    """``X @ W.T`` for at most 8 rows of ``X`` from the Huffman-coded ``W`` (reference ``functional.py:28-63``)."""
    if A_rem.dim() == 2:
        A_rem = A_rem[None, :, :]
    if offsets.dim() == 1:
        offsets = offsets[None, :]
    split_k, M, N = A_rem.shape
    X = X.view(-1, split_k, N)
    assert N % 128 == 0
    assert X.dtype == torch.bfloat16
    assert A_rem.device.type == A_exp.device.type == X.device.type == "cuda"
    assert A_rem.device == A_exp.device == X.device
    Y = torch.empty((X.size(0), M), dtype=torch.bfloat16, device=A_rem.device)
    ops.gemv_bf16_huffman(
        A_rem.contiguous(), A_exp.contiguous(), X.contiguous(), Y, offsets.contiguous(),
        LUT1.contiguous(), LUT2.contiguous(), LUT3.contiguous(), LUT4.contiguous(), code_lengths.contiguous(),
    )
    return Y


def mv_huffman_prepared(A_rem: Tensor, A_exp: Tensor, X: Tensor, offsets: Tensor, prepared: Tensor) -> Tensor:
    """:func:`mv_huffman` with the tables already folded (see :meth:`HuffmanWeight.prepared`)."""
    if A_rem.dim() == 2:
        A_rem = A_rem[None, :, :]
    split_k, M, N = A_rem.shape
    X = X.view(-1, split_k, N)
    assert N % 128 == 0
    assert X.dtype == torch.bfloat16
    assert A_rem.device == A_exp.device == X.device and A_rem.device.type == "cuda"
    Y = torch.empty((X.size(0), M), dtype=torch.bfloat16, device=A_rem.device)
    ops.gemv_bf16_huffman_prepared(A_rem.contiguous(), A_exp.contiguous(), X.contiguous(), Y, offsets.contiguous(), prepared)
    return Y


def mv_ans(A_rem: Tensor, A_exp: Tensor, X: Tensor, offsets: Tensor, LUT: Tensor) -> Tensor:
    """``X @ W.T`` for at most 8 rows of ``X`` from the rANS-coded ``W`` (reference ``functional.py:414-444``)."""
    if A_rem.dim() == 2:
        A_rem = A_rem[None, :, :]
    if offsets.dim() == 1:
        offsets = offsets[None, :]
    split_k, M, N = A_rem.shape
    X = X.view(-1, split_k, N)
    assert N % 128 == 0
    assert X.dtype == torch.bfloat16
    assert A_rem.device.type == A_exp.device.type == X.device.type == "cuda"
    assert A_rem.device == A_exp.device == X.device
    Y = torch.empty((X.size(0), M), dtype=torch.bfloat16, device=A_rem.device)
    ops.gemv_bf16_ans(A_rem.contiguous(), A_exp.contiguous(), X.contiguous(), Y, offsets.contiguous(), LUT.contiguous())
    return Y


def mm_huffman_prepared(A_rem: Tensor, A_exp: Tensor, X: Tensor, offsets: Tensor, prepared: Tensor) -> Tensor:
    """``X @ W.T`` for at most 128 rows of ``X`` from the Huffman-coded ``W``: rows of ``W`` are decoded
    into shared memory and multiplied there on the tensor cores.  Stands in for the reference's
    ``huffman_decode`` + ``F.linear`` pair (``functional.py:405-407``) in that range."""
    if A_rem.dim() == 2:
        A_rem = A_rem[None, :, :]
    split_k, M, N = A_rem.shape
    X = X.view(-1, split_k, N)
    assert N % 128 == 0
    assert X.dtype == torch.bfloat16
    assert A_rem.device == A_exp.device == X.device and A_rem.device.type == "cuda"
    Y = torch.empty((X.size(0), M), dtype=torch.bfloat16, device=A_rem.device)
    ops.linear_bf16_huffman_prepared(A_rem.contiguous(), A_exp.contiguous(), X.contiguous(), Y, offsets.contiguous(), prepared)
    return Y


def mm_ans(A_rem: Tensor, A_exp: Tensor, X: Tensor, offsets: Tensor, LUT: Tensor) -> Tensor:
    """Same for the rANS-coded ``W`` (stands in for ``ans_decode`` + ``F.linear``, reference
    ``functional.py:476-478``)."""
    if A_rem.dim() == 2:
        A_rem = A_rem[None, :, :]
    split_k, M, N = A_rem.shape
    X = X.view(-1, split_k, N)
    assert N % 128 == 0
    assert X.dtype == torch.bfloat16
    assert A_rem.device == A_exp.device == X.device and A_rem.device.type == "cuda"
    Y = torch.empty((X.size(0), M), dtype=torch.bfloat16, device=A_rem.device)
    ops.linear_bf16_ans(A_rem.contiguous(), A_exp.contiguous(), X.contiguous(), Y, offsets.contiguous(), LUT.contiguous())
    return Y


class HuffmanWeight(nn.Module):
    """A ``[M, K]`` BF16 weight with Huffman-coded exponents.

    Buffers: ``rem`` u8 ``[S, M, K/S]``, ``exp`` i32 ``[words]``, ``offsets`` i32 ``[S, M]``, ``LUT1..LUT4``
    and ``code_lengths`` u8 ``[256]``.  Passing an instance as the weight of ``F.linear`` dispatches to
    :func:`linear_huffman`.
    """

    algo = "huffman"

    def __init__(self, rem: Tensor, exp: Tensor, offsets: Tensor,
                 LUT1: Tensor, LUT2: Tensor, LUT3: Tensor, LUT4: Tensor, code_lengths: Tensor):
        super().__init__()
        self.rem = nn.Buffer(rem)
        self.exp = nn.Buffer(exp)
        self.offsets = nn.Buffer(offsets)
        self.LUT1 = nn.Buffer(LUT1)
        self.LUT2 = nn.Buffer(LUT2)
        self.LUT3 = nn.Buffer(LUT3)
        self.LUT4 = nn.Buffer(LUT4)
        self.code_lengths = nn.Buffer(code_lengths)

    # -- container protocol ---------------------------------------------------------------
    def kwargs(self) -> Dict[str, Tensor]:
        return dict(self.named_buffers())

    @property
    def shape(self) -> Tuple[int, int]:
        s, m, n = self.rem.shape
        return (m, s * n)

    def nbytes(self) -> int:
        return sum(b.nelement() * b.element_size() for b in self.buffers())

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        if func is not F.linear:
            return NotImplemented
        return linear_huffman(*args, **(kwargs or {}))

    def prepared(self) -> Tensor:
        """The decode tables folded for the fused kernels (built on first use on each device, so the
        first call has to happen outside CUDA-graph capture; warm-up iterations take care of that).
        Not a buffer: it is derived data and stays out of ``state_dict`` and size accounting."""
        blob = self.__dict__.get("_prepared")
        tables = (self.LUT1, self.LUT2, self.LUT3, self.LUT4, self.code_lengths)
        src = tuple((t.data_ptr(), t._version) for t in tables)      # in-place loads (load_state_dict) bump the version
        if blob is None or blob.device != self.rem.device or self.__dict__.get("_prepared_src") != src:
            blob = torch.empty(ops.PREPARED_BYTES, dtype=torch.uint8, device=self.rem.device)
            ops.huffman_prepare(*tables, blob)
            # codes of at most 6 bits: every 12-bit window holds two whole codes (the kernels pick their warp layout by it)
            ops.huffman_table_hint(blob, int(self.code_lengths.max().item()) <= 6)
            self.__dict__["_prepared"] = blob
            self.__dict__["_prepared_src"] = src
        return blob

    def get_weight(self) -> Tensor:
        """Dense BF16 ``[M, K]`` (reference ``functional.py:99-108``)."""
        assert self.rem.device.type == "cuda"
        weight = torch.empty(self.shape, dtype=torch.bfloat16, device=self.rem.device)
        ops.huffman_decode_prepared(self.rem, self.exp, weight, self.offsets, self.prepared())
        return weight

    # -- encoding -----------------------------------------------------------------------------
    @classmethod
    def get_codec(cls, a: Tensor) -> LUTHuffmanEncoder:
        """Code tables from the exponent histogram of ``a`` (reference ``functional.py:110-117``)."""
        codec = LUTHuffmanEncoder()
        codec.build_lut(_exp_histogram(a.to(_work_device(a))), method=HUFFMAN_TABLES)
        return codec

    @classmethod
    def get_lut_kwargs(cls, codec: LUTHuffmanEncoder) -> Dict[str, Tensor]:
        return {
            "LUT1": torch.from_numpy(codec.LUT1.copy()),
            "LUT2": torch.from_numpy(codec.LUT2.copy()),
            "LUT3": torch.from_numpy(codec.LUT3.copy()),
            "LUT4": torch.from_numpy(codec.LUT4.copy()),
            "code_lengths": torch.from_numpy(codec.code_lengths.copy()),
        }

    @classmethod
    def compress_groups(cls, x: Tensor, codec: LUTHuffmanEncoder) -> Tuple[Tensor, Tensor]:
        """Per-stream operator path: ``x`` u8 ``[rows, 64, n]`` -> (words i32 ``[rows*64, n]``, rows' word counts).

        Same result as reference ``functional.py:129-159`` (character expansion by the
        ``huffman_encode`` operator, then LSB-first packing), kept for operator compatibility and
        as a cross-check of :meth:`compress_split_n`.
        """
        dev = x.device
        rows, groups, n = x.shape
        flat = x.reshape(rows * groups, n).contiguous()
        chars = torch.full((rows * groups, n * 32), ord("0"), dtype=torch.uint8, device=dev)
        bits = torch.zeros(rows * groups, dtype=torch.int32, device=dev)
        table = torch.zeros(256, 32, dtype=torch.uint8)
        for sym, code in codec.huffman_codes.items():
            path = code[::-1]                      # stored reversed; the stream wants root first
            table[sym, :len(path)] = torch.tensor([ord(c) for c in path], dtype=torch.uint8)
        ops.huffman_encode(flat, table.to(dev), chars, bits)
        nbytes = (bits + 7) // 8
        row_words = (nbytes.view(rows, groups).amax(dim=1) + 3) // 4
        weights = (1 << torch.arange(8, device=dev, dtype=torch.int32))
        packed = ((chars.view(rows * groups, -1, 8).to(torch.int32) - ord("0")) * weights).sum(-1).to(torch.uint8)
        return packed.view(torch.int32), row_words.to(torch.int32)

    @classmethod
    def _tables_on(cls, codec, dev) -> Dict[str, Tensor]:
        return {
            "code_lengths": torch.from_numpy(codec.code_lengths.copy()).to(dev),
            "code_values": torch.from_numpy(codec.code_values.view("int32").copy()).to(dev),
        }

    @classmethod
    def _encode_layer(cls, w: Tensor, split_k: int, codec) -> Tuple[Tensor, Tensor, Tensor]:
        """Two-pass device encode of ``w`` (BF16 ``[M, K]`` on a CUDA device)."""
        dev = w.device
        M, K = w.shape
        t = cls._tables_on(codec, dev)
        rows = torch.empty(split_k, M, dtype=torch.int32, device=dev)
        ops.huffman_size_pass(w, split_k, t["code_lengths"], rows)
        offsets, total = _record_offsets(rows)
        rem = torch.empty(split_k, M, K // split_k, dtype=torch.uint8, device=dev)
        exp = torch.zeros(total, dtype=torch.int32, device=dev)
        ops.huffman_emit_pass(w, split_k, t["code_lengths"], t["code_values"], offsets, rem, exp)
        return rem, exp, offsets

    @classmethod
    def compress_split_n(cls, a: Tensor, n: int = 2, to_cpu: bool = True):
        """Encode ``a`` with ``n`` K-chunks (reference ``functional.py:195-238``)."""
        assert a.dim() == 2 and a.dtype == torch.bfloat16
        assert a.size(1) % n == 0 and (a.size(1) // n) % 128 == 0, a.shape
        w = a.detach().to(_work_device(a)).contiguous()
        codec = cls.get_codec(w)
        rem, exp, offsets = cls._encode_layer(w, n, codec)
        # the buffers must be complete in memory before a fused kernel with launch overlap reads them
        torch.cuda.current_stream(w.device).synchronize()
        if to_cpu:
            rem, exp, offsets = rem.cpu(), exp.cpu(), offsets.cpu()
            luts = cls.get_lut_kwargs(codec)
        else:
            luts = {k: v.to(w.device) for k, v in cls.get_lut_kwargs(codec).items()}
        return cls(rem=rem, exp=exp, offsets=offsets, **luts)

    @classmethod
    def compress(cls, a: Tensor, to_cpu: bool = True):
        """Encode with the format's own K-chunk choice (reference ``functional.py:240-242``)."""
        return cls.compress_split_n(a, n=get_block_size_n(a)[0], to_cpu=to_cpu)


class ANSWeight(HuffmanWeight):
    """A ``[M, K]`` BF16 weight with rANS-coded exponents (8-bit probabilities unless :func:`set_ans_precision` says otherwise).

    Buffers: ``rem``, ``exp``, ``offsets`` as for :class:`HuffmanWeight`, and ``LUT`` i32 ``[2^precision]`` holding
    ``sym << 24 | freq << 12 | (slot - cum[sym])`` per slot (reference ``functional.py:245-310``).
    """

    algo = "ans"

    def __init__(self, rem: Tensor, exp: Tensor, offsets: Tensor, LUT: Tensor):
        nn.Module.__init__(self)
        self.rem = nn.Buffer(rem)
        self.exp = nn.Buffer(exp)
        self.offsets = nn.Buffer(offsets)
        self.LUT = nn.Buffer(torch.as_tensor(LUT))

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        if func is not F.linear:
            return NotImplemented
        return linear_ans(*args, **(kwargs or {}))

    def get_weight(self) -> Tensor:
        assert self.rem.device.type == "cuda"
        weight = torch.empty(self.shape, dtype=torch.bfloat16, device=self.rem.device)
        ops.ans_decode(self.rem, self.exp, weight, self.offsets, self.LUT)
        return weight

    @classmethod
    def get_codec(cls, a: Tensor) -> RANSEncoder:
        return RANSEncoder(_exp_histogram(a.to(_work_device(a))).tolist(), precision=ANS_PRECISION)

    @classmethod
    def get_lut_kwargs(cls, codec: RANSEncoder) -> Dict[str, Tensor]:
        if max(codec.freq) > 0xFFF:
            raise ValueError("one exponent value holds the whole 12-bit model: its frequency does not fit the table word")
        lut = torch.tensor(codec.decode_lut, dtype=torch.int32)
        return {"LUT": (lut[:, 0] << 24) | (lut[:, 1] << 12) | lut[:, 2]}

    @classmethod
    def compress_groups(cls, x: Tensor, codec: RANSEncoder) -> Tuple[Tensor, Tensor]:
        """Per-stream operator path (reference ``functional.py:297-310``): words i32 ``[rows*64, 8n]``, rows' word counts."""
        dev = x.device
        rows, groups, n = x.shape
        flat = x.reshape(rows * groups, n).contiguous()
        words = torch.zeros(rows * groups, n * 8, dtype=torch.int32, device=dev)
        counts = torch.zeros(rows * groups, dtype=torch.int32, device=dev)
        freq = torch.tensor(codec.freq, dtype=torch.int32, device=dev)
        cum = torch.tensor(codec.cum, dtype=torch.int32, device=dev)
        ops.ans_encode(flat, freq, cum, words, counts)
        return words, counts.view(rows, groups).amax(dim=1)

    @classmethod
    def _encode_layer(cls, w: Tensor, split_k: int, codec) -> Tuple[Tensor, Tensor, Tensor]:
        dev = w.device
        M, K = w.shape
        freq = torch.tensor(codec.freq, dtype=torch.int32, device=dev)
        cum = torch.tensor(codec.cum, dtype=torch.int32, device=dev)
        rows = torch.empty(split_k, M, dtype=torch.int32, device=dev)
        per_stream = torch.empty(split_k, M, 64, dtype=torch.uint8, device=dev)
        ops.ans_size_pass(w, split_k, freq, cum, rows, per_stream)
        offsets, total = _record_offsets(rows)
        rem = torch.empty(split_k, M, K // split_k, dtype=torch.uint8, device=dev)
        exp = torch.zeros(total, dtype=torch.int32, device=dev)
        ops.ans_emit_pass(w, split_k, freq, cum, offsets, per_stream, rem, exp)
        return rem, exp, offsets


class CompressedLinear(nn.Module):
    """``nn.Linear`` replacement whose weight is a :class:`HuffmanWeight` / :class:`ANSWeight` (reference ``functional.py:313-320``)."""

    def __init__(self, weight: HuffmanWeight, bias: Optional[Tensor]) -> None:
        super().__init__()
        self.weight = weight
        self.bias = bias

    @property
    def out_features(self) -> int:
        return self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self.weight.shape[1]

    def forward(self, input: Tensor) -> Tensor:
        return F.linear(input, self.weight, self.bias)


def _linear_compressed(input: Tensor, weight: HuffmanWeight, bias: Optional[Tensor], fused, tensor) -> Tensor:
    assert input.dim() >= 2, input
    shape = input.shape
    input = input.flatten(0, -2)
    if input.size(0) <= max(FUSED_MAX_ROWS, min(TENSOR_MAX_ROWS, 128)):
        output = fused(input) if input.size(0) <= FUSED_MAX_ROWS else tensor(input)
        if bias is not None:
            output += bias[None, :]
    else:
        output = F.linear(input, weight.get_weight(), bias)
    return output.unflatten(0, shape[:-1])


def linear_huffman(input: Tensor, weight: HuffmanWeight, bias: Optional[Tensor] = None) -> Tensor:
    """``F.linear`` on a Huffman-coded weight: fused decode+GEMV up to 8 rows, decode then GEMM beyond
    (reference ``functional.py:390-411``); optionally the fused tensor-core product up to ``TENSOR_MAX_ROWS``."""
    return _linear_compressed(
        input, weight, bias,
        lambda x: mv_huffman_prepared(weight.rem, weight.exp, x, weight.offsets, weight.prepared()),
        lambda x: mm_huffman_prepared(weight.rem, weight.exp, x, weight.offsets, weight.prepared()))


def linear_ans(input: Tensor, weight: ANSWeight, bias: Optional[Tensor] = None) -> Tensor:
    """Same for an rANS-coded weight (reference ``functional.py:447-466``)."""
    return _linear_compressed(
        input, weight, bias,
        lambda x: mv_ans(weight.rem, weight.exp, x, weight.offsets, weight.LUT),
        lambda x: mm_ans(weight.rem, weight.exp, x, weight.offsets, weight.LUT))


def _buffers_size(w: nn.Module) -> int:
    return sum(b.nelement() * b.element_size() for b in w.buffers())


def convert(linear: nn.Linear, name, disable_precision_check: bool = True, algo: str = "huffman"):
    """Compress one ``nn.Linear``; returns a :class:`CompressedLinear`, or ``linear`` itself when
    compression does not pay (ratio >= 1) or, if checking is enabled, when the fused output is off
    by 2 % or more on a random input (reference ``functional.py:323-375``).  The module comes back
    on the device ``linear`` was on."""
    assert algo in ("huffman", "ans", "smallest")
    home = linear.weight.device
    if algo == "huffman":
        weight = HuffmanWeight.compress(linear.weight)
    elif algo == "ans":
        weight = ANSWeight.compress(linear.weight)
    else:
        weight = min(
            [HuffmanWeight.compress(linear.weight), ANSWeight.compress(linear.weight)],
            key=_buffers_size,
        )
    module = CompressedLinear(weight=weight, bias=linear.bias)

    ori_size = linear.weight.nelement() * linear.weight.element_size()
    ratio = _buffers_size(module.weight) / ori_size

    work = _work_device(linear.weight)
    linear.to(work)
    module.to(work)
    x = torch.randn(1, linear.in_features, dtype=torch.bfloat16, device=work)
    with torch.no_grad():
        y1 = linear(x)
        y2 = module(x)
    max_rtol = ((y2 - y1).abs() / y1.abs().clamp(min=1e-4)).max().item()
    linear.to(home)
    module.to(home)

    fallback = False
    if ratio >= 1:
        print(f"\nWarning! {name} ratio = {ratio:.2%}")
        fallback = True
    if not disable_precision_check and max_rtol >= 0.02:
        print(f"\nWarning! {name} output mismatch: max rtol = {max_rtol:.2f}")
        fallback = True
    if fallback:
        print("Fallback to regular nn.Linear")
        return linear
    return module


class FusedCompressedLinear(nn.Module):
    """Several ``nn.Linear`` layers that read the same input, stored as ONE compressed weight (their
    rows concatenated) and computed by ONE fused launch.

    A 1024-row projection cannot fill a B200 on its own (7 rows per SM); stacking q/k/v (or
    gate/up) gives the kernel enough rows and saves the fixed cost of the extra launches.  The
    reference attacks the same problem with side streams (``cudastream_utils.py:7-47``).  Each
    original module is replaced by a :class:`_FusedSlice`; the first one in call order computes the
    stacked output, the others return their slice of it.
    """

    def __init__(self, weight: HuffmanWeight, bias: Optional[Tensor], splits):
        super().__init__()
        self.weight = weight
        self.bias = bias
        self.splits = list(splits)            # [(start, stop), ...] in stacking order
        self.sharded: Optional[nn.Module] = None   # set by tensor_parallel.shard_model_linears: computes the full output
        self._last_in = None
        self._last_out = None
        self._readers_left = 0                      # slices that have not picked up the last output yet

    def run(self, input: Tensor) -> Tensor:
        out = self.sharded(input) if self.sharded is not None else F.linear(input, self.weight, self.bias)
        self._last_in = (input.data_ptr(), input._version, tuple(input.shape))
        self._last_out = out
        self._readers_left = len(self.splits) - 1
        return out

    def cached(self, input: Tensor) -> Tensor:
        """The leader's output for this very input.  It is kept only until every other slice has read it once:
        a later tensor that happens to get the same address (and version 0) must not match a stale entry."""
        key = (input.data_ptr(), input._version, tuple(input.shape))
        if self._last_out is None or self._last_in != key:
            out = self.run(input)
            self._readers_left -= 1
        else:
            out = self._last_out
            self._readers_left -= 1
        if self._readers_left <= 0:
            self._last_in = self._last_out = None
        return out


class _FusedSlice(nn.Module):
    """Stands where one of the stacked layers was; ``leader`` recomputes, the others reuse."""

    def __init__(self, owner: FusedCompressedLinear, index: int, leader: bool):
        super().__init__()
        self.__dict__["_owner"] = owner       # not a submodule: the owner is registered once, on the leader
        if leader:
            self.fused = owner
        self.index = index
        self.leader = leader

    @property
    def out_features(self) -> int:
        a, b = self._owner.splits[self.index]
        return b - a

    def forward(self, input: Tensor) -> Tensor:
        owner = self._owner
        out = owner.run(input) if self.leader else owner.cached(input)
        a, b = owner.splits[self.index]
        return out[..., a:b]


def fuse_sibling_linears(model: nn.Module, groups=SIBLING_GROUPS, algo: str = "huffman", progress: bool = False) -> int:
    """Stack and compress sibling ``nn.Linear`` layers (same parent, same input width, all with or all
    without bias) named as in ``groups``.  Call before :func:`convert_all_linear`, which then handles
    the remaining layers.  Returns the number of groups fused."""
    todo = []
    for pname, parent in model.named_modules():
        for names in groups:
            mods = [getattr(parent, n, None) for n in names]
            if not all(isinstance(m, nn.Linear) for m in mods):
                continue
            if len({m.in_features for m in mods}) != 1 or len({m.bias is None for m in mods}) != 1:
                continue
            todo.append((pname, parent, names, mods))
    for pname, parent, names, mods in tqdm(todo, disable=not progress):
        home = mods[0].weight.device
        stacked = torch.cat([m.weight.detach() for m in mods], dim=0)
        bias = None if mods[0].bias is None else nn.Parameter(torch.cat([m.bias.detach() for m in mods]), requires_grad=False)
        if algo == "huffman":
            weight = HuffmanWeight.compress(stacked)
        elif algo == "ans":
            weight = ANSWeight.compress(stacked)
        else:
            weight = min([HuffmanWeight.compress(stacked), ANSWeight.compress(stacked)], key=_buffers_size)
        if _buffers_size(weight) >= stacked.nelement() * stacked.element_size():
            continue                                      # does not pay: leave the layers alone
        bounds, at = [], 0
        for m in mods:
            bounds.append((at, at + m.out_features))
            at += m.out_features
        owner = FusedCompressedLinear(weight, bias, bounds).to(home)
        for i, n in enumerate(names):
            setattr(parent, n, _FusedSlice(owner, i, leader=(i == 0)))
    return len(todo)


def convert_all_linear(model: nn.Module, min_out_features: int = 4096, progress: bool = True,
                       algo: str = "huffman", fuse_siblings: bool = False, huffman_tables: Optional[str] = None) -> None:
    """Replace, in place, every ``nn.Linear`` with at least ``min_out_features`` outputs
    (reference ``functional.py:378-387``).  Not in the reference: ``fuse_siblings=True`` first stacks
    q/k/v and gate/up projections into single compressed weights (:class:`FusedCompressedLinear`);
    ``huffman_tables`` picks the table builder for this call (:func:`set_huffman_tables`)."""
    previous = set_huffman_tables(huffman_tables) if huffman_tables is not None else None
    try:
        if fuse_siblings:
            fuse_sibling_linears(model, algo=algo, progress=progress)
        targets = [name for name, mod in model.named_modules()
                   if isinstance(mod, nn.Linear) and mod.out_features >= min_out_features]
        for name in tqdm(targets, disable=not progress):
            model.set_submodule(name, convert(model.get_submodule(name), name, algo=algo))
    finally:
        if previous is not None:
            set_huffman_tables(previous)
