"""Range bounds for adaptive channel-prefix selection.

Host-side counterparts of the reference's ``src/rns_llm/adaptive.py``
(``signed_capacity`` :9-12, ``minimal_prefix_channels`` :15-41,
``safe_l1_dot_bound`` :44-52), same names and errors.  On the hot path the
bound and the prefix are computed on the device (``rns_select_channels`` in
include/rns_b200.h); these functions serve weight preparation, metadata and
tests.
"""
from __future__ import annotations

from math import prod
from typing import Iterable

from .moduli import validate_moduli


def signed_capacity(moduli: Iterable[int]) -> int:
    """Largest |x| every centred representation over ``moduli`` can hold."""
    return (prod(validate_moduli(moduli)) - 1) // 2


def minimal_prefix_channels(moduli: Iterable[int], absolute_bound: int, *, min_channels: int = 2) -> int:
    """Shortest prefix (>= ``min_channels``) with ``2*bound < prod(prefix)``.

    ``OverflowError`` when the whole set is too small: a result must never wrap
    silently.
    """
    mods = validate_moduli(moduli)
    if absolute_bound < 0:
        raise ValueError("absolute_bound must be non-negative")
    if not 2 <= min_channels <= len(mods):
        raise ValueError("min_channels must be between 2 and len(moduli)")
    product = 1
    for count, modulus in enumerate(mods, 1):
        product *= modulus
        if count >= min_channels and 2 * absolute_bound < product:
            return count
    raise OverflowError(
        f"full moduli set cannot represent bound {absolute_bound}; capacity={signed_capacity(mods)}"
    )


def safe_l1_dot_bound(max_row_l1: int, max_abs_weight: int) -> int:
    """|sum_k a_ik b_kj| <= (max_i sum_k |a_ik|) * max|b| for every output."""
    if max_row_l1 < 0 or max_abs_weight < 0:
        raise ValueError("bounds must be non-negative")
    return int(max_row_l1) * int(max_abs_weight)
