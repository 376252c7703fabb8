"""Host-side builder of the byte-decomposed Huffman tables used by the exponent decoder.

The tables produced here are bit-identical to the ones the reference builds in
``bf16_huffman_infer/huffman.py`` (``LUTHuffmanEncoder.build_lut``, lines 347-361, with the
helpers at lines 40-280), because the compressed exponent plane is only decodable with the
exact code the encoder used.  The algorithm is restated, not transcribed: the tree lives in
flat parent-less arrays, codes are ``(length, value)`` integer pairs with the first path bit in
bit 0, and the conflict scan works on integer masks.  What must be preserved for identical
output is (a) the heap discipline (Python's ``heapq`` with a strict ``<`` on the frequency only,
leaves pushed in ascending symbol order), (b) the left-before-right depth-first numbering of
leaves, which fixes the iteration order of the conflict scan, and (c) the two frequency
perturbation rules (length limit and table-collision repair).

Table semantics (consumed by the CUDA decoders and the CPU oracle):

* a code of ``n`` bits with integer value ``v`` (first path bit = bit 0) is emitted LSB-first;
* ``n <= 8``  : ``LUT1[(v & 0xFF) + i * 2**n] = sym`` for every ``i`` that stays below 256;
* ``8 < n <= 16``: ``LUT2[((v >> 8) & 0xFF) + i * 2**(n-8)] = sym``; likewise ``LUT3`` on byte 2 for
  ``16 < n <= 24`` and ``LUT4`` on byte 3 for ``24 < n <= 32``;
* unfilled entries hold 255; ``code_lengths[sym] = n`` (0 for absent symbols).

A decoder looks at the low four bytes ``b0..b3`` of its bit window and takes the first of
``LUT1[b0], LUT2[b1], LUT3[b2], LUT4[b3]`` that is not 255, then drops ``code_lengths[sym]`` bits
(reference ``src/kernel.cu:354-380``).
"""
from __future__ import annotations

import heapq
from typing import Dict, Iterable, List, Sequence, Tuple, Union

import numpy as np

try:  # torch is optional for the pure table maths
    import torch
except Exception:  # pragma: no cover
    torch = None

SENTINEL = 255
MAX_CODE_BITS = 32

__all__ = ["LUTHuffmanEncoder", "SENTINEL", "MAX_CODE_BITS", "escape_byte_code", "length_limited_code"]


class _HeapItem:
    """Heap entry ordered by frequency alone (ties keep whatever order ``heapq`` gives them)."""

    __slots__ = ("freq", "node")

    def __init__(self, freq: float, node: int):
        self.freq = freq
        self.node = node

    def __lt__(self, other: "_HeapItem") -> bool:
        return self.freq < other.freq


def _huffman_paths(freqs: Dict[int, float]) -> Dict[int, Tuple[int, int]]:
    """Return ``{symbol: (n_bits, value)}`` in depth-first (left first) leaf order.

    ``value`` has the root-side path bit in bit 0 (left edge = 0, right edge = 1).  Follows the
    tree construction of reference ``huffman.py:40-64`` and the traversal of ``:66-82``.
    """
    left: List[int] = []
    right: List[int] = []
    symbol: List[int] = []
    heap: List[_HeapItem] = []
    for sym, f in freqs.items():
        if f > 0:
            left.append(-1)
            right.append(-1)
            symbol.append(sym)
            heapq.heappush(heap, _HeapItem(f, len(symbol) - 1))
    if not heap:
        return {}
    if len(heap) == 1:
        # a lone symbol hangs off the left edge of a synthetic root: one-bit code "0"
        return {symbol[heap[0].node]: (1, 0)}
    while len(heap) > 1:
        a = heapq.heappop(heap)
        b = heapq.heappop(heap)
        left.append(a.node)
        right.append(b.node)
        symbol.append(-1)
        heapq.heappush(heap, _HeapItem(a.freq + b.freq, len(symbol) - 1))
    root = heap[0].node

    out: Dict[int, Tuple[int, int]] = {}
    stack = [(root, 0, 0)]
    while stack:
        node, depth, value = stack.pop()
        if left[node] < 0:
            out[symbol[node]] = (depth, value)
            continue
        # right is pushed first so that left is visited first
        stack.append((right[node], depth + 1, value | (1 << depth)))
        stack.append((left[node], depth + 1, value))
    return out


def _limit_length(freqs: Dict[int, float], max_bits: int) -> Dict[int, float]:
    """Flatten rare symbols until no code is longer than ``max_bits`` (reference ``huffman.py:84-123``)."""
    work = dict(freqs)
    for _ in range(50):
        codes = _huffman_paths(work)
        if not codes:
            return work
        deepest = max(n for n, _ in codes.values())
        if deepest <= max_bits:
            return work
        cands = sorted((s for s, (n, _) in codes.items() if n == deepest), key=lambda s: work[s])
        for s in cands:
            if work[s] > 1:
                work[s] = 1
                break
        else:
            work[cands[0]] = 0.5
    raise AssertionError("length limiting did not converge")


def _table_slots(n_bits: int, value: int) -> Tuple[int, Iterable[int]]:
    """Which byte table a code lands in and the entries it occupies there."""
    level = (n_bits - 1) // 8            # 0..3
    known = n_bits - 8 * level           # significant bits inside that byte, 1..8
    base = (value >> (8 * level)) & 0xFF
    return level, range(base, 256, 1 << known) if known < 8 else (base,)


def _repair_collisions(freqs: Dict[int, float], max_bits: int) -> Dict[int, float]:
    """Perturb frequencies until no two symbols share an entry of the same byte table.

    Mirrors reference ``huffman.py:125-218``: every colliding entry (visited table by table, in
    the order entries were first touched while walking the codes in leaf order) boosts the
    currently most frequent of its claimants by 1.5x, then the code is rebuilt.
    """
    work = _limit_length(dict(freqs), max_bits)
    codes = _huffman_paths(work)
    for _ in range(20):
        claims: List[Dict[int, List[int]]] = [dict() for _ in range(4)]
        for sym, (n, v) in codes.items():
            if n == 0:
                continue
            level, slots = _table_slots(n, v)
            tab = claims[level]
            for slot in slots:
                tab.setdefault(slot, []).append(sym)
        clashes = [syms for tab in claims for syms in tab.values() if len(syms) > 1]
        if not clashes:
            return work
        for syms in clashes:
            winner = max(syms, key=lambda s: work[s])   # first maximal element, as a stable sort would pick
            work[winner] = work[winner] * 1.5
        work = _limit_length(work, max_bits)
        codes = _huffman_paths(work)
    raise AssertionError("table-collision repair did not converge")


# ---- escape-byte builder: an alternative code for the same tables ---------------------------------
# The byte-decomposed tables need every code longer than 8 bits to be recognisable from its SECOND byte
# alone, whatever its first byte was.  The reference reaches that by perturbing frequencies until the
# plain Huffman code happens to satisfy it, which for some histograms lengthens the frequent codes a
# lot.  This builder satisfies the constraint by construction instead: frequent symbols get a
# length-limited (<= 8 bits) optimal code together with ONE escape leaf, padded to exactly 8 bits; all
# the other symbols hang below that escape byte with a second length-limited (<= 8 bits) optimal code,
# so they are told apart by the second byte and no code exceeds 16 bits.  The split point is chosen by
# exhaustive search for the smallest total cost.  The tables it yields have the reference's layout
# and semantics (any decoder of the format reads them); only the code itself differs from the one the
# reference's builder would pick, so the compressed bytes differ too.

def _limited_lengths(weights: Sequence[float], limit: int) -> List[int]:
    """Optimal code lengths with no length above ``limit`` (package-merge); weights need not be sorted."""
    n = len(weights)
    if n == 0:
        return []
    if n == 1:
        return [1]
    assert n <= (1 << limit), "too many symbols for the length limit"
    order = sorted(range(n), key=lambda i: (weights[i], i))
    leaves = [(weights[i], (i,)) for i in order]
    level = list(leaves)
    for _ in range(limit - 1):
        packages = [(level[j][0] + level[j + 1][0], level[j][1] + level[j + 1][1]) for j in range(0, len(level) - 1, 2)]
        level = sorted(leaves + packages, key=lambda t: t[0])      # stable: leaves before packages of equal weight
    lengths = [0] * n
    for _, members in level[: 2 * n - 2]:
        for i in members:
            lengths[i] += 1
    return lengths


def _canonical_paths(lengths: Dict[int, int]) -> Dict[int, str]:
    """Root-first path strings of a canonical prefix code: shorter codes first, then ascending key."""
    paths: Dict[int, str] = {}
    code = 0
    prev = 0
    for key in sorted(lengths, key=lambda k: (lengths[k], k)):
        n = lengths[key]
        code <<= n - prev
        paths[key] = format(code, "b").zfill(n)
        code += 1
        prev = n
    return paths


def escape_byte_code(freqs: Dict[int, float]) -> Dict[int, Tuple[int, int]]:
    """``{symbol: (length, value)}`` (first path bit in bit 0) of the escape-byte code for ``freqs``."""
    syms = sorted(freqs, key=lambda s: (-freqs[s], s))
    n = len(syms)
    if n == 0:
        return {}
    ESC = -1
    best = None
    for top in range(max(1, n - 255), n + 1):
        rest = n - top
        if rest == 1 or top + (1 if rest else 0) > 256:
            continue                                       # a lone escaped symbol is just a 256th leaf: covered by top + 1
        upper = syms[:top] + ([ESC] if rest else [])
        w_upper = [freqs[s] for s in syms[:top]] + ([sum(freqs[s] for s in syms[top:])] if rest else [])
        l_upper = _limited_lengths(w_upper, 8)
        l_lower = _limited_lengths([freqs[s] for s in syms[top:]], 8)
        cost = sum(w * l for w, l in zip(w_upper[:top], l_upper[:top])) + sum(freqs[s] * (8 + l) for s, l in zip(syms[top:], l_lower))
        if best is None or cost < best[0]:
            best = (cost, top, dict(zip(upper, l_upper)), dict(zip(syms[top:], l_lower)))
    _, top, l_upper, l_lower = best
    # canonical order puts the escape leaf last among the leaves of its length (ESC sorts as the largest key below)
    upper_paths = _canonical_paths({(256 if k == ESC else k): v for k, v in l_upper.items()})
    codes: Dict[int, Tuple[int, int]] = {}
    for k, path in upper_paths.items():
        if k != 256:
            codes[k] = (len(path), int(path[::-1], 2))
    if l_lower:
        esc = upper_paths[256].ljust(8, "0")                # pad the escape to a whole byte
        for k, path in _canonical_paths(l_lower).items():
            full = esc + path
            codes[k] = (len(full), int(full[::-1], 2))
    return codes


def length_limited_code(freqs: Dict[int, float], limit: int) -> Dict[int, Tuple[int, int]]:
    """``{symbol: (length, value)}`` of the optimal prefix code whose lengths do not exceed ``limit`` (<= 8).

    Every code fits the first byte table, so the byte-decomposed format holds it as it is.  With
    ``limit = 6`` any two consecutive codes fit a 12-bit window: the fused kernels then resolve two
    symbols with every table lookup and never take their symbol-by-symbol path.  Falls back to the
    escape-byte code when there are more symbols than ``2**limit``.  No counterpart in the reference.
    """
    assert 1 <= limit <= 8
    syms = sorted(freqs)
    if len(syms) > (1 << limit):
        return escape_byte_code(freqs)
    lengths = _limited_lengths([freqs[s] for s in syms], limit)
    paths = _canonical_paths(dict(zip(syms, lengths)))
    return {s: (len(path), int(path[::-1], 2)) for s, path in paths.items()}


class LUTHuffmanEncoder:
    """Drop-in for the reference class of the same name (``huffman.py:23-397``).

    Attributes after :meth:`build_lut`: ``LUT1..LUT4`` and ``code_lengths`` (``uint8[256]``),
    ``huffman_codes`` (``{symbol: str}``; as in the reference the string is the root-to-leaf path
    *reversed*, so ``int(code, 2)`` has the first path bit in bit 0), plus ``code_values``
    (``uint32[256]``, the same integers) for vectorised encoders.
    """

    def __init__(self, max_code_length: int = MAX_CODE_BITS):
        self.max_code_length = max_code_length
        self.huffman_codes: Dict[int, str] = {}
        self.LUT1 = np.full(256, SENTINEL, dtype=np.uint8)
        self.LUT2 = np.full(256, SENTINEL, dtype=np.uint8)
        self.LUT3 = np.full(256, SENTINEL, dtype=np.uint8)
        self.LUT4 = np.full(256, SENTINEL, dtype=np.uint8)
        self.code_lengths = np.zeros(256, dtype=np.uint8)
        self.code_values = np.zeros(256, dtype=np.uint32)

    # -- table construction -------------------------------------------------------------
    def build_lut(self, frequencies: Union[np.ndarray, Sequence[int], "torch.Tensor"], method: str = "reference") -> None:
        """``method='reference'`` reproduces the reference's code exactly; ``'escape'`` builds the
        escape-byte code (same table format, shorter frequent codes when the reference's repair loop
        would have distorted them); ``'limitN'`` (N = 1..8) the optimal code with lengths <= N.  Neither of
        the last two has a counterpart in the reference."""
        if torch is not None and torch.is_tensor(frequencies):
            frequencies = frequencies.cpu().numpy()
        freqs = {i: float(frequencies[i]) for i in range(256) if frequencies[i] > 0}
        if method == "escape":
            self._install(escape_byte_code(freqs))
            return
        if method.startswith("limit"):
            self._install(length_limited_code(freqs, int(method[5:])))
            return
        assert method == "reference", method
        final = _repair_collisions(freqs, self.max_code_length)
        self._install(_huffman_paths(final))

    def _install(self, codes: Dict[int, Tuple[int, int]]) -> None:
        tables = (self.LUT1, self.LUT2, self.LUT3, self.LUT4)
        for t in tables:
            t.fill(SENTINEL)
        self.code_lengths.fill(0)
        self.code_values.fill(0)
        self.huffman_codes = {}
        for sym, (n, v) in codes.items():
            self.code_lengths[sym] = n
            self.code_values[sym] = v
            self.huffman_codes[sym] = format(v, "b").zfill(n) if n else ""
            if n == 0:
                continue
            level, slots = _table_slots(n, v)
            for slot in slots:
                tables[level][slot] = sym

    def build_decomposed_luts(self, codes: Dict[int, str]) -> None:
        """Fill the tables from a ``{symbol: reversed-path string}`` mapping (reference ``huffman.py:220-280``)."""
        self._install({s: (len(c), int(c, 2) if c else 0) for s, c in codes.items()})

    # -- slow single-stream codec, kept for cross-checks ----------------------------------
    @staticmethod
    def encode_to_bitstream(data, codes: Dict[int, str], progress: bool = False) -> str:
        """One stream as a bit string whose *last* character is the first bit (reference ``huffman.py:282-293``)."""
        parts = []
        for s in data:
            s = int(s)
            if s not in codes:
                raise ValueError(f"Byte value {s} not in encoding table")
            parts.append(codes[s][::-1])
        return "".join(parts)[::-1]

    def decode_with_lut(self, bit_string: str, num_elements: int) -> List[int]:
        """Decode a string made by :meth:`encode_to_bitstream` (reference ``huffman.py:295-345``)."""
        total = len(bit_string)
        stream = int(bit_string, 2) if bit_string else 0
        stream |= 0xFFFFFFFF << total            # the reference pads with 32 one-bits past the end
        out: List[int] = []
        pos = 0
        while len(out) < num_elements and pos < total + 32:
            if total + 32 - pos < 8:
                break
            window = (stream >> pos) & 0xFFFFFFFF
            for k, tab in enumerate((self.LUT1, self.LUT2, self.LUT3, self.LUT4)):
                sym = int(tab[(window >> (8 * k)) & 0xFF])
                if sym != SENTINEL:
                    break
            else:
                raise AssertionError("undecodable bit window")
            out.append(sym)
            pos += int(self.code_lengths[sym])
        return out

    def encode(self, data, frequencies):
        """Build tables from ``frequencies`` and encode ``data`` (reference ``huffman.py:364-394``)."""
        if torch is not None and torch.is_tensor(data):
            data = data.cpu().numpy()
        data = np.asarray(data).flatten().astype(np.uint8)
        self.build_lut(frequencies)
        bits = self.encode_to_bitstream(data, self.huffman_codes)
        n = len(data)
        stats = {
            "original_bytes": n,
            "original_bits": 8 * n,
            "compressed_bits": len(bits),
            "compression_ratio": len(bits) / (8 * n) if n else 0,
            "space_saving_percentage": (1 - (len(bits) / (8 * n) if n else 0)) * 100,
            "huffman_codes": dict(self.huffman_codes),
            "average_code_length": len(bits) / n if n else 0,
            "max_code_length": max((len(c) for c in self.huffman_codes.values()), default=0),
            "lut_memory_usage": 4 * 256 + 256,
        }
        return bits, stats

    def decode(self, encoded_bitstring: str, original_length: int) -> List[int]:
        return self.decode_with_lut(encoded_bitstring, original_length)
