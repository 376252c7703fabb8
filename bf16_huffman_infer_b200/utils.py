"""Small helpers that define parts of the compressed format (byte split, K-chunk count) and
model bookkeeping.  Same names and behaviour as the reference's ``bf16_huffman_infer/utils.py``.
"""
from __future__ import annotations

import copy
from typing import Tuple

import torch
from torch import Tensor, nn

__all__ = [
    "split_bf16", "merge_bf16", "get_block_size_n", "get_model_size", "print_stats", "shallow_copy_model",
]


def split_bf16(x: Tensor) -> Tuple[Tensor, Tensor]:
    """BF16 tensor -> ``(rem, exp)`` uint8 planes (reference ``utils.py:7-12``).

    ``exp`` is the 8-bit biased exponent (bits 14..7); ``rem`` packs the sign into bit 7 above
    the 7 mantissa bits.
    """
    assert x.dtype == torch.bfloat16
    bits = x.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    exp = ((bits >> 7) & 0xFF).to(torch.uint8)
    rem = (((bits >> 8) & 0x80) | (bits & 0x7F)).to(torch.uint8)
    return rem, exp


def merge_bf16(rem: Tensor, exp: Tensor) -> Tensor:
    """Inverse of :func:`split_bf16` (the reassembly of reference ``src/kernel.cu:149-160``)."""
    r = rem.to(torch.int32)
    e = exp.to(torch.int32)
    bits = ((r << 8) & 0x8000) | (r & 0x7F) | (e << 7)
    bits = torch.where(bits >= 0x8000, bits - 0x10000, bits).to(torch.int16)
    return bits.view(torch.bfloat16)


def chunk_count_for_k(k: int) -> int:
    """Number of K-chunks ("split_k") the format uses for a row length ``k``.

    Restates reference ``utils.py:15-31``: with ``nb = k / 128`` blocks, prefer a chunk of
    ``i`` blocks (``i`` from 32 down to 3) that divides ``nb`` into at most 8 chunks; else the
    smallest ``i`` in 32..128 giving at most 32 chunks; else the largest ``i`` in 32..3 giving at
    most 32 chunks.
    """
    if k % 128 == 0:
        nb = k // 128
        for i in range(32, 2, -1):
            if nb % i == 0 and nb // i <= 8:
                return nb // i
        for i in range(32, 129):
            if nb % i == 0 and nb // i <= 32:
                return nb // i
        for i in range(32, 2, -1):
            if nb % i == 0 and nb // i <= 32:
                return nb // i
    raise RuntimeError(f"Could not find suitable block size for row length {k}")


def get_block_size_n(x: Tensor) -> Tuple[int]:
    """``(split_k,)`` for a ``[M, K]`` weight (reference ``utils.py:15-31``)."""
    try:
        return (chunk_count_for_k(x.size(1)),)
    except RuntimeError:
        raise RuntimeError(f"Could not find suitable block size for shape {x.shape}") from None


def get_model_size(model: nn.Module) -> int:
    """Bytes held by all parameters and buffers (reference ``utils.py:34-42``)."""
    total = 0
    for _, p in model.named_parameters():
        total += p.nelement() * p.element_size()
    for _, b in model.named_buffers():
        total += b.nelement() * b.element_size()
    return total


def print_stats(ori: Tensor, new: nn.Module) -> None:
    ori_size = ori.nelement() * ori.element_size()
    new_size = sum(b.nelement() * b.element_size() for b in new.buffers())
    print(f"ori size = {ori_size / 1024 ** 2:.2f}MiB")
    print(f"new size = {new_size / 1024 ** 2:.2f}MiB")
    print(f"compression ratio = {new_size / ori_size:.2%}")
    print(f"bits = {new_size / ori_size * 16:.2f}")


def shallow_copy_model(model: nn.Module) -> nn.Module:
    """Deep-copy the module tree while sharing every parameter and buffer (reference ``utils.py:55-61``)."""
    memo = {}
    for p in model.parameters():
        memo[id(p)] = p
    for b in model.buffers():
        memo[id(b)] = b
    # derived device data a module keeps outside its buffers (e.g. the folded decode tables of a compressed weight)
    # is shared too: a copy would cost memory and lose what the native library remembers about the original
    for m in model.modules():
        for v in vars(m).values():
            if torch.is_tensor(v):
                memo[id(v)] = v
    return copy.deepcopy(model, memo=memo)
