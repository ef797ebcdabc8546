"""Host-side number theory for the RNS linear path.

Everything the device kernels take as constants is produced here: modulus
validation and selection, mixed-radix (Garner) constants, CRT coefficients and
the byte-decomposition modulo table kept for callers of the legacy interface.

Mirrors the public helpers of the reference's ``src/rns_llm/reference.py``
(``validate_moduli`` :11-23, ``crt_constants`` :43-54,
``garner_pairwise_inverses`` :57-67, ``compact_byte_mod_lut`` :70-88,
candidate tables :188-217, ``choose_moduli_for_dot`` :238-265,
``moduli_cost_model`` :268-297) with the same names, arguments and error
behaviour.  The NumPy encoders / decoders of that file are CPU arithmetic, not
constants, and live with the test oracle instead of in this package.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache
from typing import Iterable, Literal, Sequence

import numpy as np

ModuliStrategy = Literal["large_primes", "dense_coprime", "small_primes"]

INT64_MAX = (1 << 63) - 1
MAX_CHANNELS = 10  # channel counts the fused reconstruction accepts (2..10)


def validate_moduli(moduli: Iterable[int]) -> tuple[int, ...]:
    """Return ``moduli`` as a tuple after checking the residue-channel rules.

    Every modulus must lie in [2, 255] so that a centred residue fits a signed
    byte, and the set must be pairwise coprime.  Raises ``ValueError``
    otherwise (same conditions as reference.py:11-23).
    """
    mods = tuple(int(m) for m in moduli)
    if len(mods) == 0:
        raise ValueError("moduli must not be empty")
    for m in mods:
        if not 2 <= m <= 255:
            raise ValueError("every modulus must be in [2, 255]")
    for idx, a in enumerate(mods):
        for b in mods[idx + 1:]:
            if math.gcd(a, b) != 1:
                raise ValueError(f"moduli are not pairwise coprime: {a}, {b}")
    return mods


def _is_prime(n: int) -> bool:
    return n >= 2 and all(n % d for d in range(2, int(n ** 0.5) + 1))


def _primes_between(lo: int, hi: int) -> list[int]:
    return [n for n in range(lo, hi + 1) if _is_prime(n)]


# Candidate orders (reference.py:188-217).  Generated rather than listed:
#   large primes  : the primes in [127, 251], largest first;
#   dense coprime : 255, 253, 247 (composite but mutually coprime with the
#                   primes) merged into the descending primes >= 127, then the
#                   two prime powers 125 and 121;
#   small primes  : every prime in [3, 251], smallest first.
LARGE_PRIME_MODULI: tuple[int, ...] = tuple(reversed(_primes_between(127, 251)))
DENSE_COPRIME_MODULI: tuple[int, ...] = tuple(
    sorted(set(LARGE_PRIME_MODULI) | {255, 253, 247}, reverse=True)
) + (125, 121)
SMALL_PRIME_MODULI: tuple[int, ...] = tuple(_primes_between(3, 251))
HARDWARE_FRIENDLY_MODULI = LARGE_PRIME_MODULI


def candidates_for_strategy(strategy: str) -> tuple[int, ...]:
    table = {
        "large_primes": LARGE_PRIME_MODULI,
        "dense_coprime": DENSE_COPRIME_MODULI,
        "small_primes": SMALL_PRIME_MODULI,
    }
    if strategy not in table:
        raise ValueError(f"unknown moduli strategy: {strategy}")
    return table[strategy]


def dot_product_bound(k: int, max_abs_a: int, max_abs_b: int) -> int:
    """|sum_k a_k b_k| <= k * max|a| * max|b| (reference.py:229-235)."""
    if k <= 0:
        raise ValueError("k must be positive")
    if max_abs_a < 0 or max_abs_b < 0:
        raise ValueError("absolute bounds must be non-negative")
    return int(k) * int(max_abs_a) * int(max_abs_b)


def choose_moduli_for_dot(
    k: int,
    max_abs_a: int,
    max_abs_b: int,
    *,
    candidates: Iterable[int] | None = None,
    strategy: str = "large_primes",
) -> tuple[int, ...]:
    """Greedy prefix of the candidate order whose product exceeds 2*bound.

    Candidates that are not coprime with the ones already taken are skipped.
    ``ValueError`` when the candidates run out first (reference.py:238-265).
    """
    need = 2 * dot_product_bound(k, max_abs_a, max_abs_b) + 1
    pool = tuple(candidates) if candidates is not None else candidates_for_strategy(strategy)
    taken: list[int] = []
    product = 1
    for cand in pool:
        cand = int(cand)
        if not 2 <= cand <= 255 or any(math.gcd(cand, t) != 1 for t in taken):
            continue
        taken.append(cand)
        product *= cand
        if product >= need:
            return tuple(taken)
    raise ValueError(f"candidate moduli cannot cover required range {need}")


def crt_constants(moduli: Iterable[int]) -> tuple[int, tuple[int, ...]]:
    """(P, coefficients) with coefficient_c = (P/m_c) * ((P/m_c)^-1 mod m_c) mod P.

    ``OverflowError`` when P does not fit int64 (reference.py:43-54).
    """
    mods = validate_moduli(moduli)
    product = math.prod(mods)
    if product > INT64_MAX:
        raise OverflowError("product(moduli) must fit signed int64 for this decoder")
    coeffs = []
    for m in mods:
        cofactor = product // m
        coeffs.append(cofactor * pow(cofactor, -1, m) % product)
    return product, tuple(coeffs)


def garner_pairwise_inverses(moduli: Iterable[int]) -> tuple[tuple[int, ...], ...]:
    """Table t with t[j][i] = m_j^-1 mod m_i for j < i, zero elsewhere
    (reference.py:57-67)."""
    mods = validate_moduli(moduli)
    r = len(mods)
    return tuple(
        tuple(pow(mods[j], -1, mods[i]) if j < i else 0 for i in range(r))
        for j in range(r)
    )


def compact_byte_mod_lut(moduli: Iterable[int]) -> np.ndarray:
    """[R,4,256] int16 table: entry [c,p,b] = (b * 256**p) mod m_c
    (reference.py:70-88).  The sm_100a epilogue reduces in registers and never
    reads it; it is produced for callers of the legacy fused entry point."""
    mods = validate_moduli(moduli)
    byte = np.arange(256, dtype=np.int64)
    out = np.empty((len(mods), 4, 256), dtype=np.int16)
    for c, m in enumerate(mods):
        for p in range(4):
            out[c, p] = (byte * pow(256, p, m)) % m
    return out


def moduli_cost_model(
    moduli: Iterable[int],
    *,
    m: int,
    k: int,
    n: int,
    source_element_bytes: int,
    lut_channels: int = 0,
) -> dict[str, int | float]:
    """Byte counts of the plane-materialising pipeline (reference.py:268-297)."""
    mods = validate_moduli(moduli)
    r = len(mods)
    lut_used = min(lut_channels, r)
    full_lut = sum(x * x for x in mods[:lut_channels])
    compact = lut_used * 4 * 256 * 2
    return {
        "channels": r,
        "modulus_product": math.prod(mods),
        "source_inputs_bytes": (m * k + k * n) * source_element_bytes,
        "encoded_inputs_bytes": r * (m * k + k * n),
        "residue_output_bytes": r * m * n,
        "int32_accumulator_bytes": 4 * r * m * n,
        "compact_lut_bytes": compact,
        "full_mul_lut_bytes": full_lut,
        "compact_vs_full_lut_saving": 0.0 if full_lut == 0 else 1.0 - compact / full_lut,
    }


# ---------------------------------------------------------------------------
# Constants of the fused sm_100a epilogue
# ---------------------------------------------------------------------------

def _centre(value: int, modulus: int) -> int:
    """Representative of ``value`` mod ``modulus`` in [-(m-1)//2, m//2]."""
    value %= modulus
    return value - modulus if value > modulus // 2 else value


@dataclass(frozen=True)
class GarnerPlan:
    """Constants of the flattened mixed-radix reconstruction.

    The reference computes digit i with i sequential steps
    ``v = (v - d_j) * inv[j][i] mod m_i`` (csrc/rns_cuda.cu:380-414).  Because
    every intermediate is below 2**24 the same digit is
    ``d_i = (r_i - sum_{j<i} w[i][j] * d_j) * c[i]  mod m_i`` with
    ``w[i][j] = prod_{t<j} m_t mod m_i`` and ``c[i] = (prod_{t<i} m_t)^-1 mod
    m_i`` (both stored centred), which needs one reduction per digit instead of
    i.  ``prefix[i] = prod_{t<i} m_t`` are the mixed-radix place values.
    """

    moduli: tuple[int, ...]
    weights: tuple[tuple[int, ...], ...]   # w[i][j], j < i (0 elsewhere)
    scale: tuple[int, ...]                 # c[i]
    prefix: tuple[int, ...]                # place values, prefix[0] = 1
    product: int


@lru_cache(maxsize=256)
def garner_plan(moduli: Sequence[int]) -> GarnerPlan:
    mods = validate_moduli(moduli)
    r = len(mods)
    prefix = [1] * r
    for i in range(1, r):
        prefix[i] = prefix[i - 1] * mods[i - 1]
    weights = tuple(
        tuple(_centre(prefix[j], mods[i]) if j < i else 0 for j in range(r))
        for i in range(r)
    )
    scale = tuple(
        _centre(pow(prefix[i] % mods[i], -1, mods[i]), mods[i]) if i else 1
        for i in range(r)
    )
    return GarnerPlan(mods, weights, scale, tuple(prefix), prefix[-1] * mods[-1])
