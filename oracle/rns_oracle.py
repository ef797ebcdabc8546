"""CPU restatement of the reference's RNS linear path.  TEST INFRASTRUCTURE ONLY.

This file is the checker the CUDA path is compared with.  Only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import it;
nothing in ``rns_llm_b200`` does.

Parity pins: the functions below are checked against the reference's own NumPy
implementation (imported in the build container) through the golden vectors in
``tests/golden/`` (generator: ``tests/golden/make_golden.py``), and against the
relations the reference's tests assert (``tests/test_reference.py:11-95`` of the
reference).  The reference stores no golden files of its own.

Each function cites the reference code it restates, as path:line inside the
reference project (Nek1tt/rns-llm v0.5).
"""
from __future__ import annotations

from math import gcd, prod
from typing import Iterable, Sequence

import numpy as np

FLT_EPS = np.float32(np.finfo(np.float32).eps)


# ---------------------------------------------------------------------------
# Level 1: the independent integer oracle (docs/CORRECTNESS_GUARDS.md:3-11,
# tests/test_cuda_backend.py:17-18)
# ---------------------------------------------------------------------------
def exact_matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """a[M,K] @ b[K,N] in int64; shares no code with any RNS routine."""
    return np.asarray(a).astype(np.int64) @ np.asarray(b).astype(np.int64)


# ---------------------------------------------------------------------------
# Moduli and constants (src/rns_llm/reference.py:11-23, 43-67)
# ---------------------------------------------------------------------------
def check_moduli(moduli: Iterable[int]) -> tuple[int, ...]:
    mods = tuple(int(m) for m in moduli)
    if not mods:
        raise ValueError("moduli must not be empty")
    if any(not 2 <= m <= 255 for m in mods):
        raise ValueError("every modulus must be in [2, 255]")
    for i in range(len(mods)):
        for j in range(i + 1, len(mods)):
            if gcd(mods[i], mods[j]) != 1:
                raise ValueError(f"moduli are not pairwise coprime: {mods[i]}, {mods[j]}")
    return mods


def pairwise_inverses(moduli: Sequence[int]) -> list[list[int]]:
    """inv[j][i] = m_j^-1 mod m_i for j < i (reference.py:57-67)."""
    mods = check_moduli(moduli)
    r = len(mods)
    return [[pow(mods[j], -1, mods[i]) if j < i else 0 for i in range(r)] for j in range(r)]


def crt_coefficients(moduli: Sequence[int]) -> tuple[int, list[int]]:
    """(P, [(P/m) * ((P/m)^-1 mod m) mod P]) (reference.py:43-54)."""
    mods = check_moduli(moduli)
    p = prod(mods)
    return p, [(p // m) * pow(p // m, -1, m) % p for m in mods]


# ---------------------------------------------------------------------------
# Encoders (reference.py:26-40 for NumPy; csrc/rns_cuda.cu:98-124 for the device
# convention, which differs only at -m/2 of an even modulus)
# ---------------------------------------------------------------------------
def encode_canonical(values: np.ndarray, moduli: Sequence[int]) -> np.ndarray:
    """Residues in [0, m) as uint8 planes [R, *shape] (reference.py:26-29)."""
    mods = check_moduli(moduli)
    v = np.asarray(values, dtype=np.int64)
    return np.stack([np.mod(v, m) for m in mods]).astype(np.uint8)


def encode_centered(values: np.ndarray, moduli: Sequence[int], convention: str = "numpy") -> np.ndarray:
    """Centred residues as int8 planes [R, *shape].

    ``convention="numpy"``: floor-mod then ``r > m//2 -> r - m``
    (reference.py:32-40), so -m/2 of an even modulus becomes +m/2.
    ``convention="device"``: C remainder then fold both sides
    (csrc/rns_cuda.cu:112-122), so -m/2 stays negative.
    """
    mods = check_moduli(moduli)
    v = np.asarray(values, dtype=np.int64)
    planes = []
    for m in mods:
        if convention == "numpy":
            r = np.mod(v, m)
            r = np.where(r > m // 2, r - m, r)
        elif convention == "device":
            r = np.fmod(v, m)  # sign of the dividend, like C '%'
            half = m // 2
            r = np.where(r > half, r - m, np.where(r < -half, r + m, r))
        else:
            raise ValueError(convention)
        planes.append(r.astype(np.int8))
    return np.stack(planes)


# ---------------------------------------------------------------------------
# Decoders (reference.py:91-147; device: csrc/rns_cuda.cu:380-414)
# ---------------------------------------------------------------------------
def decode_crt(residues: np.ndarray, moduli: Sequence[int], signed: bool = True) -> np.ndarray:
    """Chinese-remainder decode of residue planes (reference.py:91-116)."""
    mods = check_moduli(moduli)
    res = np.asarray(residues, dtype=np.int64)
    if res.shape[0] != len(mods):
        raise ValueError("residue channel count does not match moduli")
    p, coeffs = crt_coefficients(mods)
    if p > np.iinfo(np.int64).max:
        raise OverflowError("product(moduli) must fit signed int64 for this decoder")
    out = np.zeros(res.shape[1:], dtype=np.int64)
    for plane, coeff in zip(res, coeffs):
        out = np.mod(out + plane * coeff, p)
    if signed:
        out = np.where(out > p // 2, out - p, out)
    return out


def decode_garner(residues: np.ndarray, moduli: Sequence[int], signed: bool = True) -> np.ndarray:
    """Mixed-radix reconstruction; accepts any representative per channel,
    including raw int32 dot products (reference.py:119-147)."""
    mods = check_moduli(moduli)
    src = np.asarray(residues, dtype=np.int64)
    if src.shape[0] != len(mods):
        raise ValueError("residue channel count does not match moduli")
    inv = pairwise_inverses(mods)
    digits: list[np.ndarray] = []
    for i, m in enumerate(mods):
        d = np.mod(src[i], m)
        for j in range(i):
            d = np.mod((d - digits[j]) * inv[j][i], m)
        digits.append(d)
    total = np.zeros(src.shape[1:], dtype=np.int64)
    place = 1
    for m, d in zip(mods, digits):
        total = total + place * d
        place *= m
    if signed:
        total = np.where(total > place // 2, total - place, total)
    return total


# ---------------------------------------------------------------------------
# GEMMs (reference.py:150-185; device pipeline csrc/rns_cuda.cu:478-523, 442-476)
# ---------------------------------------------------------------------------
def matmul_canonical_planes(a_res: np.ndarray, b_res: np.ndarray, moduli: Sequence[int]) -> np.ndarray:
    """Per-channel product of canonical planes, reduced (reference.py:150-170)."""
    mods = check_moduli(moduli)
    a = np.asarray(a_res, dtype=np.uint8)
    b = np.asarray(b_res, dtype=np.uint8)
    if a.ndim != 3 or b.ndim != 3:
        raise ValueError("expected [R, M, K] and [R, K, N]")
    if a.shape[0] != len(mods) or b.shape[0] != len(mods):
        raise ValueError("residue channel count does not match moduli")
    if a.shape[2] != b.shape[1]:
        raise ValueError("K dimensions do not match")
    return np.stack([
        np.mod(a[c].astype(np.int64) @ b[c].astype(np.int64), m).astype(np.uint8)
        for c, m in enumerate(mods)
    ])


def rns_matmul(a: np.ndarray, b: np.ndarray, moduli: Sequence[int], decode: bool = True) -> np.ndarray:
    """The reference's CPU path: canonical encode, per-channel int64 matmul,
    CRT decode (``rns_matmul_numpy``, reference.py:173-185).  This is the CPU
    baseline that bench.py times."""
    ra = encode_canonical(a, moduli)
    rb = encode_canonical(b, moduli)
    rc = matmul_canonical_planes(ra, rb, moduli)
    return decode_crt(rc, moduli, signed=True) if decode else rc


def channel_sums(a: np.ndarray, b: np.ndarray, moduli: Sequence[int], convention: str = "device") -> np.ndarray:
    """int64 [R,M,N]: the raw per-channel accumulators of the device pipeline
    (centred planes through an exact int8 GEMM, csrc/rns_cuda.cu:478-523)."""
    ra = encode_centered(a, moduli, convention).astype(np.int64)
    rb = encode_centered(b, moduli, convention).astype(np.int64)
    return np.stack([ra[c] @ rb[c] for c in range(len(moduli))])


def rns_matmul_device_pipeline(a: np.ndarray, b: np.ndarray, moduli: Sequence[int],
                               active: int | None = None) -> np.ndarray:
    """encode_centered -> per-channel GEMM -> reduce + Garner + recentre, i.e.
    ``matmul_prepared_fused`` (backends/cuda_backend.py:514-539) on the CPU,
    optionally with only the first ``active`` channels (adaptive prefix,
    backends/cuda_backend.py:573-622)."""
    mods = check_moduli(moduli)
    use = mods if active is None else mods[:active]
    return decode_garner(channel_sums(a, b, use), use, signed=True)


# ---------------------------------------------------------------------------
# Adaptive bound (src/rns_llm/adaptive.py:9-52)
# ---------------------------------------------------------------------------
def signed_capacity(moduli: Sequence[int]) -> int:
    return (prod(check_moduli(moduli)) - 1) // 2


def minimal_prefix_channels(moduli: Sequence[int], absolute_bound: int, min_channels: int = 2) -> int:
    mods = check_moduli(moduli)
    if absolute_bound < 0:
        raise ValueError("absolute_bound must be non-negative")
    if not 2 <= min_channels <= len(mods):
        raise ValueError("min_channels must be between 2 and len(moduli)")
    running = 1
    for count, m in enumerate(mods, start=1):
        running *= m
        if count >= min_channels and 2 * absolute_bound < running:
            return count
    raise OverflowError(f"full moduli set cannot represent bound {absolute_bound}")


def safe_l1_dot_bound(max_row_l1: int, max_abs_weight: int) -> int:
    if max_row_l1 < 0 or max_abs_weight < 0:
        raise ValueError("bounds must be non-negative")
    return int(max_row_l1) * int(max_abs_weight)


def adaptive_channels(a_q: np.ndarray, w_q: np.ndarray, moduli: Sequence[int], min_channels: int = 3) -> tuple[int, int]:
    """(channels, bound) chosen by select_adaptive_variant
    (backends/cuda_backend.py:573-601)."""
    l1 = int(np.abs(np.asarray(a_q, dtype=np.int64)).sum(axis=1).max())
    bound = safe_l1_dot_bound(l1, int(np.abs(np.asarray(w_q, dtype=np.int64)).max()))
    return minimal_prefix_channels(moduli, bound, min_channels), bound


# ---------------------------------------------------------------------------
# Level 2: RNSLinear.forward (src/rns_llm/layers/rns_linear.py:154-166, 183-185,
# 239-241, 264-275), float32 arithmetic in the reference's operation order.
# ---------------------------------------------------------------------------
def symmetric_scale(values: np.ndarray, quant_max: int, axis=None) -> np.ndarray:
    """clamp(max|v| / quant_max, eps_f32) in float32 (rns_linear.py:154-159)."""
    v = np.asarray(values, dtype=np.float32)
    max_abs = np.abs(v).max(axis=axis, keepdims=True).astype(np.float32)
    return np.maximum(max_abs / np.float32(quant_max), FLT_EPS).astype(np.float32)


def quantize(values: np.ndarray, scale: np.ndarray, quant_max: int) -> np.ndarray:
    """clamp(round_half_even(v / scale), +-quant_max) (rns_linear.py:161-166)."""
    v = np.asarray(values, dtype=np.float32)
    q = np.rint((v / scale.astype(np.float32)).astype(np.float32))
    return np.clip(q, -quant_max, quant_max).astype(np.int8 if quant_max <= 127 else np.int16)


def rns_linear_forward(x: np.ndarray, weight: np.ndarray, bias: np.ndarray | None,
                       moduli: Sequence[int], quant_max: int = 127, per_row: bool = False,
                       out_dtype=np.float16) -> dict[str, np.ndarray]:
    """RNSLinear.forward in mode="rns" (rns_linear.py:225-275).

    ``x`` is [..., K] (float16/float32), ``weight`` [N,K], ``bias`` [N] or None.
    The reference scales activations per tensor (rns_linear.py:240 calls
    ``_symmetric_scale(flat)`` with ``dim=None``); ``per_row=True`` is the
    per-token variant this build also offers.  Returns every intermediate so
    that tests can pin each stage.
    """
    lead = x.shape[:-1]
    k = x.shape[-1]
    flat = np.asarray(x).reshape(-1, k).astype(np.float32)
    w32 = np.asarray(weight).astype(np.float32)
    w_scale = symmetric_scale(w32, quant_max, axis=1)            # [N,1]
    w_q = quantize(w32, w_scale, quant_max)                      # [N,K]
    a_scale = symmetric_scale(flat, quant_max, axis=1 if per_row else None)
    a_q = quantize(flat, a_scale, quant_max)                     # [M,K]
    integer = rns_matmul_device_pipeline(a_q, w_q.T, moduli)     # [M,N] int64
    if not np.array_equal(integer, exact_matmul(a_q, w_q.T)):
        raise AssertionError("RNS pipeline disagrees with the int64 oracle")
    out = integer.astype(np.float32) * a_scale.astype(np.float32)
    out = (out * w_scale.reshape(1, -1).astype(np.float32)).astype(np.float32)
    if bias is not None:
        out = (out + np.asarray(bias).astype(np.float32)).astype(np.float32)
    y = out.reshape(*lead, -1).astype(out_dtype)
    return {"y": y, "a_q": a_q, "a_scale": a_scale.reshape(-1), "w_q": w_q,
            "w_scale": w_scale.reshape(-1), "integer": integer}
