"""Host-side rANS model: frequency normalisation and the decode table.

Produces exactly the ``freq`` / ``cum`` / ``decode_lut`` the reference's ``RANSEncoder`` does
(``bf16_huffman_infer/ans.py:5-34`` and the normaliser at ``:42-80``); the device coder and the
CPU oracle consume these tables, so they have to agree to the last count.

Coder conventions (reference ``src/kernel.cu:767-811`` encode, ``:652-683`` decode):
64-bit state, ``precision`` low bits select the slot, 32-bit renormalisation words.
"""
from __future__ import annotations

from collections import Counter
from typing import Dict, List, Mapping, Sequence, Tuple, Union

__all__ = ["RANSEncoder"]


def _scale_counts(counts: Mapping[int, int], target: int) -> Dict[int, int]:
    """Scale positive counts so they sum to ``target`` with every symbol keeping at least 1.

    Same rule as reference ``ans.py:42-80``: round-half-even of ``count * target / total`` (floored
    at 1), then hand out / take back single units cyclically over the symbols ordered by rounding
    error (largest under-estimate first when short, largest over-estimate first when long).
    """
    total = sum(counts.values())
    if total <= 0:
        raise ValueError("sum of frequencies must be positive")
    scaled: Dict[int, int] = {}
    errs: List[Tuple[float, int]] = []
    for sym, c in counts.items():
        if c <= 0:
            raise ValueError(f"frequency of symbol {sym} must be > 0")
        exact = c * target / total
        q = max(int(round(exact)), 1)
        scaled[sym] = q
        errs.append((exact - q, sym))
    have = sum(scaled.values())
    if have < target:
        order = [s for _, s in sorted(errs, reverse=True)]
        while have < target:
            for s in order:
                if have == target:
                    break
                scaled[s] += 1
                have += 1
    elif have > target:
        order = [s for _, s in sorted(errs)]
        while have > target:
            for s in order:
                if have == target:
                    break
                if scaled[s] > 1:
                    scaled[s] -= 1
                    have -= 1
    if sum(scaled.values()) != target:
        raise ValueError("normalisation failed")
    return scaled


class RANSEncoder:
    """Drop-in for the reference class (``ans.py:5-147``): same constructor, attributes and codec."""

    def __init__(self, freq: Union[Mapping[int, int], Sequence[int]], precision: int = 12):
        if precision < 1 or precision > 15:
            raise ValueError("precision must be in [1, 15]")
        if not freq:
            raise ValueError("freq must not be empty")
        if isinstance(freq, list):
            freq = {s: f for s, f in enumerate(freq) if f > 0}
        self.precision = precision
        self.base = 1 << precision
        self.mask = self.base - 1
        table = _scale_counts(freq, self.base)
        self.freq: List[int] = [table.get(s, 0) for s in range(256)]
        self.cum: List[int] = []
        run = 0
        for f in self.freq:
            self.cum.append(run)
            run += f
        # slot -> (symbol, freq[symbol], slot - cum[symbol])
        self.decode_lut: List[Tuple[int, int, int]] = [
            (s, f, j) for s, f in enumerate(self.freq) for j in range(f)
        ]

    @classmethod
    def from_data(cls, data: Sequence[int], precision: int = 12) -> "RANSEncoder":
        return cls(Counter(int(x) for x in data), precision)

    # -- slow single-stream codec, kept for cross-checks (reference ans.py:82-147) ----------
    def compress(self, symbols: Sequence[int]) -> bytes:
        """Encode last-to-first; 32-bit words are appended big-endian, final state as two words."""
        state = self.base
        out = bytearray()
        for sym in reversed([int(x) for x in symbols]):
            f, c = self.freq[sym], self.cum[sym]
            while state >= (f << 32):
                out += (state & 0xFFFFFFFF).to_bytes(4, "big")
                state >>= 32
            q, r = divmod(state, f)
            state = (q << self.precision) + r + c
        for _ in range(2):
            out += (state & 0xFFFFFFFF).to_bytes(4, "big")
            state >>= 32
        return bytes(out)

    def decompress(self, blob: bytes, output_len: int) -> List[int]:
        """Inverse of :meth:`compress`: words are consumed from the end of ``blob``."""
        if output_len == 0:
            return []
        ptr = len(blob)
        state = 0
        out: List[int] = []
        for _ in range(output_len):
            while state < self.base:
                if ptr == 0:
                    raise ValueError("compressed stream is damaged or too short")
                ptr -= 4
                state = (state << 32) | int.from_bytes(blob[ptr:ptr + 4], "big")
            sym, f, r = self.decode_lut[state & self.mask]
            out.append(sym)
            state = f * (state >> self.precision) + r
        return out
