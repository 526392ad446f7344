"""Shared helpers of the cost models."""

from __future__ import annotations

from typing import List, Tuple


def split_into_three_powers_of_two(G: int) -> List[Tuple[int, int, int]]:
    """All ``(2^a, 2^b, 2^c)`` with ``a + b + c = log2 G`` (a outer loop, b inner)."""
    if G <= 0 or G & (G - 1):
        raise ValueError("G must be a positive power of 2.")
    n = G.bit_length() - 1
    return [(1 << a, 1 << b, 1 << (n - a - b)) for a in range(n + 1) for b in range(n + 1 - a)]


# axis letter playing each role at layer l % 3
OUTER = ("X", "Z", "Y")
INNER = ("Y", "X", "Z")
DEPTH = ("Z", "Y", "X")
