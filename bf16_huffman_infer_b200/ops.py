"""Thin Python callers of the operator library (same six functions as the reference's
``bf16_huffman_infer/ops.py``, plus the whole-layer encoder passes).

Importing this module loads ``_C`` (the stable-ABI operator library) and, through it,
``libbf16_huffman_b200.so``.  There is no fallback: if the native libraries are missing the
import fails with instructions to build them.
"""
from __future__ import annotations

import os

import torch
from torch import Tensor

_PKG = os.path.dirname(os.path.abspath(__file__))

try:
    from . import _C  # noqa: F401  (registers torch.ops.bf16_huffman_infer.*)
except ImportError as exc:  # pragma: no cover - exercised only on a broken install
    raise ImportError(
        "bf16_huffman_infer_b200: the native libraries are not built "
        f"({exc}). Run `python bf16_huffman_infer_b200/_build.py` (needs nvcc with sm_100a support)."
    ) from exc

_ops = torch.ops.bf16_huffman_infer


def gemv_bf16_huffman(
    A_rem: Tensor, A_exp: Tensor, X: Tensor, Y: Tensor, offsets: Tensor,
    LUT1: Tensor, LUT2: Tensor, LUT3: Tensor, LUT4: Tensor, code_lengths: Tensor,
) -> None:
    _ops.gemv_bf16_huffman.default(A_rem, A_exp, X, Y, offsets, LUT1, LUT2, LUT3, LUT4, code_lengths)


def huffman_encode(data: Tensor, LUT: Tensor, output: Tensor, output_lengths: Tensor) -> None:
    _ops.huffman_encode.default(data, LUT, output, output_lengths)


def huffman_decode(
    A_rem: Tensor, A_exp: Tensor, Y: Tensor, offsets: Tensor,
    LUT1: Tensor, LUT2: Tensor, LUT3: Tensor, LUT4: Tensor, code_lengths: Tensor,
) -> None:
    _ops.huffman_decode.default(A_rem, A_exp, Y, offsets, LUT1, LUT2, LUT3, LUT4, code_lengths)


def gemv_bf16_ans(A_rem: Tensor, A_exp: Tensor, X: Tensor, Y: Tensor, offsets: Tensor, LUT: Tensor) -> None:
    _ops.gemv_bf16_ans.default(A_rem, A_exp, X, Y, offsets, LUT)


def ans_encode(data: Tensor, freq: Tensor, cum: Tensor, output: Tensor, output_lengths: Tensor) -> None:
    _ops.ans_encode.default(data, freq, cum, output, output_lengths)


def ans_decode(A_rem: Tensor, A_exp: Tensor, Y: Tensor, offsets: Tensor, LUT: Tensor) -> None:
    _ops.ans_decode.default(A_rem, A_exp, Y, offsets, LUT)


def set_launch_overlap(on: bool) -> bool:
    """Let consecutive fused kernels overlap (programmatic dependent launch).  Safe whenever the
    weight buffers were not written by a kernel still in flight on the same stream; see
    ``bhi_set_launch_overlap`` in the C header.  Returns the previous setting."""
    return bool(_ops.set_launch_overlap.default(int(bool(on))))


# ---- prepared Huffman tables (folded once per layer instead of inside every launch) -------------------
PREPARED_BYTES = 16384 + 2048


def huffman_prepare(LUT1: Tensor, LUT2: Tensor, LUT3: Tensor, LUT4: Tensor, code_lengths: Tensor, prepared: Tensor) -> None:
    _ops.huffman_prepare.default(LUT1, LUT2, LUT3, LUT4, code_lengths, prepared)


def huffman_table_hint(prepared: Tensor, pair_complete: bool) -> None:
    """Tell the library that no code of the table behind ``prepared`` is longer than 6 bits (a tuning hint for
    the fused kernels' warp layout; results do not depend on it).  See ``bhi_huffman_table_hint``."""
    _ops.huffman_table_hint.default(prepared, int(bool(pair_complete)))


def gemv_bf16_huffman_prepared(A_rem: Tensor, A_exp: Tensor, X: Tensor, Y: Tensor, offsets: Tensor, prepared: Tensor) -> None:
    _ops.gemv_bf16_huffman_prepared.default(A_rem, A_exp, X, Y, offsets, prepared)


def linear_bf16_huffman_prepared(A_rem: Tensor, A_exp: Tensor, X: Tensor, Y: Tensor, offsets: Tensor, prepared: Tensor) -> None:
    """Fused decode + tensor-core product for up to 128 rows of ``X`` (no reference counterpart)."""
    _ops.linear_bf16_huffman_prepared.default(A_rem, A_exp, X, Y, offsets, prepared)


def linear_bf16_ans(A_rem: Tensor, A_exp: Tensor, X: Tensor, Y: Tensor, offsets: Tensor, LUT: Tensor) -> None:
    """Fused decode + tensor-core product for up to 128 rows of ``X`` (no reference counterpart)."""
    _ops.linear_bf16_ans.default(A_rem, A_exp, X, Y, offsets, LUT)


def gemv_bf16_huffman_exchange(A_rem: Tensor, A_exp: Tensor, X: Tensor, offsets: Tensor, prepared: Tensor,
                               peers: Tensor, rank: int, row_base: int, m_total: int) -> None:
    """Row-sharded fused GEMV that stores its results into every rank's output buffer (no reference
    counterpart).  ``peers``: CPU int64 ``[3 * world + 1]`` = output, ready-counter and done-counter
    pointers of every rank, then the local launch counter."""
    _ops.gemv_bf16_huffman_exchange.default(A_rem, A_exp, X, offsets, prepared, peers, rank, row_base, m_total)


def gemv_bf16_ans_exchange(A_rem: Tensor, A_exp: Tensor, X: Tensor, offsets: Tensor, LUT: Tensor,
                           peers: Tensor, rank: int, row_base: int, m_total: int) -> None:
    _ops.gemv_bf16_ans_exchange.default(A_rem, A_exp, X, offsets, LUT, peers, rank, row_base, m_total)


def huffman_decode_prepared(A_rem: Tensor, A_exp: Tensor, Y: Tensor, offsets: Tensor, prepared: Tensor) -> None:
    _ops.huffman_decode_prepared.default(A_rem, A_exp, Y, offsets, prepared)


# ---- whole-layer encoder passes --------------------------------------------------------------------
def huffman_size_pass(W: Tensor, split_k: int, code_lengths: Tensor, words_per_row: Tensor) -> None:
    _ops.huffman_size_pass.default(W, split_k, code_lengths, words_per_row)


def huffman_emit_pass(W: Tensor, split_k: int, code_lengths: Tensor, code_values: Tensor, offsets: Tensor,
                      rem: Tensor, exp: Tensor) -> None:
    _ops.huffman_emit_pass.default(W, split_k, code_lengths, code_values, offsets, rem, exp)


def ans_size_pass(W: Tensor, split_k: int, freq: Tensor, cum: Tensor, words_per_row: Tensor,
                  stream_words: Tensor) -> None:
    _ops.ans_size_pass.default(W, split_k, freq, cum, words_per_row, stream_words)


def ans_emit_pass(W: Tensor, split_k: int, freq: Tensor, cum: Tensor, offsets: Tensor, stream_words: Tensor,
                  rem: Tensor, exp: Tensor) -> None:
    _ops.ans_emit_pass.default(W, split_k, freq, cum, offsets, stream_words, rem, exp)
