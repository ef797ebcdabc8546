"""Host-side constants of the package and the C ABI's host functions against the
reference's golden outputs; the device arithmetic, compiled for the CPU, against
the oracle."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import rns_oracle as O
from rns_llm_b200 import adaptive, moduli as M

C0 = (127, 126, 125, 121)
C4 = (127, 126, 125, 121, 113)
DENSE = (255, 253, 251, 247)
ROOT = Path(__file__).resolve().parent.parent


def test_package_constants_match_reference(golden):
    g = golden("constants")
    for tag, mods in (("c0", C0), ("c4", C4), ("dense", DENSE)):
        product, coeffs = M.crt_constants(mods)
        assert product == int(g[f"{tag}_product"][0])
        assert list(coeffs) == [int(v) for v in g[f"{tag}_crt"]]
        assert np.array_equal(np.array(M.garner_pairwise_inverses(mods)), g[f"{tag}_pairinv"])
        assert np.array_equal(M.compact_byte_mod_lut(mods), g[f"{tag}_lut"])
    for strategy in ("large_primes", "dense_coprime", "small_primes"):
        assert list(M.candidates_for_strategy(strategy)) == [int(v) for v in g[f"cand_{strategy}"]]
        for k, qa in ((64, 127), (768, 127), (4096, 127), (16384, 127), (64, 2047), (768, 2047), (768, 32767)):
            got = M.choose_moduli_for_dot(k, qa, qa, strategy=strategy)
            assert list(got) == [int(v) for v in g[f"choose_{strategy}_{k}_{qa}"]]
    cost = M.moduli_cost_model(C0, m=128, k=768, n=768, source_element_bytes=1, lut_channels=2)
    assert sorted(cost) == list(g["cost_keys"])
    assert [float(cost[key]) for key in sorted(cost)] == list(g["cost_values"])


def test_validate_moduli_errors():
    with pytest.raises(ValueError):
        M.validate_moduli(())
    with pytest.raises(ValueError):
        M.validate_moduli((1, 5))
    with pytest.raises(ValueError):
        M.validate_moduli((256, 5))
    with pytest.raises(ValueError):
        M.validate_moduli((126, 124))
    with pytest.raises(ValueError):
        M.candidates_for_strategy("nope")
    with pytest.raises(ValueError):
        M.choose_moduli_for_dot(10**9, 32767, 32767, strategy="large_primes", candidates=(251, 241))
    with pytest.raises(OverflowError):
        M.crt_constants(M.LARGE_PRIME_MODULI[:9])
    assert M.validate_moduli([127, 126, 125, 121]) == C0


def test_adaptive_host_functions(golden, native):
    g = golden("constants")
    lib = native.load()
    arr = native.moduli_array(C0)
    for bound, expected in zip(g["prefix_bounds"], g["prefix_channels_min2"]):
        c_result = lib.rns_minimal_prefix_channels(arr, 4, int(bound), 2)
        if expected < 0:
            with pytest.raises(OverflowError):
                adaptive.minimal_prefix_channels(C0, int(bound), min_channels=2)
            assert c_result == -native.ERR_OVERFLOW
        else:
            assert adaptive.minimal_prefix_channels(C0, int(bound), min_channels=2) == int(expected)
            assert c_result == int(expected)
    assert adaptive.signed_capacity(C0) == int(g["capacity_c0"][0])
    with pytest.raises(ValueError):
        adaptive.minimal_prefix_channels(C0, 5, min_channels=1)
    with pytest.raises(ValueError):
        adaptive.minimal_prefix_channels(C0, -1)
    with pytest.raises(ValueError):
        adaptive.safe_l1_dot_bound(-1, 3)
    assert adaptive.safe_l1_dot_bound(6362, 127) == 6362 * 127


def test_c_abi_exports_every_declared_symbol(native):
    header = (ROOT / "include" / "rns_b200.h").read_text()
    declared = set(re.findall(r"RNS_API\s+[\w\s\*]+?\b(rns_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(native.SIGNATURES), declared ^ set(native.SIGNATURES)
    lib = C.CDLL(str(native.library_path()))
    for name in declared:
        assert hasattr(lib, name), name
    assert native.load().rns_version() >= 100


def test_c_abi_host_constants(golden, native):
    g = golden("constants")
    lib = native.load()
    for tag, mods in (("c0", C0), ("c4", C4), ("dense", DENSE)):
        r = len(mods)
        recips = (C.c_int64 * r)()
        inv = (C.c_int32 * (r * r))()
        product = C.c_int64()
        native.check(lib.rns_host_constants(native.moduli_array(mods), r, recips, inv, C.byref(product)))
        assert product.value == int(g[f"{tag}_product"][0])
        assert list(recips) == [(1 << 32) // m for m in mods]
        assert np.array_equal(np.array(list(inv)).reshape(r, r), g[f"{tag}_pairinv"])
    with pytest.raises(ValueError):
        native.check(lib.rns_host_constants(native.moduli_array((126, 124)), 2, None, None, None))
    assert "coprime" in native.last_error()
    with pytest.raises(ValueError):
        native.check(lib.rns_host_constants(native.moduli_array((300, 7)), 2, None, None, None))
    with pytest.raises(OverflowError):
        big = M.LARGE_PRIME_MODULI[:9]
        native.check(lib.rns_host_constants(native.moduli_array(big), 9, None, None, None))


def _host_reconstruct(native, sums, mods, active=None):
    sums = np.ascontiguousarray(sums, dtype=np.int32)
    out = np.empty(sums.shape[1], dtype=np.int64)
    native.check(native.load().rns_host_reconstruct(
        sums.ctypes.data, sums.shape[1], native.moduli_array(mods), len(mods),
        len(mods) if active is None else active, out.ctypes.data))
    return out


def test_device_reconstruction_on_host_matches_reference(golden, native):
    g = golden("encode_decode")
    assert np.array_equal(_host_reconstruct(native, g["garner_sums_c0"], C0), g["garner_values_c0"])
    assert np.array_equal(_host_reconstruct(native, g["garner_sums_c4"], C4), g["garner_values_c4"])
    wrap_in = O.encode_centered(g["wrap_inputs_c0"], C0).astype(np.int32)
    assert np.array_equal(_host_reconstruct(native, wrap_in, C0), g["wrap_outputs_c0"])


@pytest.mark.parametrize("mods", [C0, C4, DENSE, (251, 241, 239), (3, 5, 7, 11, 13, 17, 19, 23, 29, 31),
                                  (255, 254, 253, 251, 247, 241, 239), (2, 3), (128, 127, 125, 123, 121)])
def test_device_reconstruction_random(native, mods):
    rng = np.random.default_rng(len(mods) * 1000 + mods[0])
    cap = O.signed_capacity(mods)
    span = min(cap, (1 << 62))
    values = np.concatenate([rng.integers(-span, span + 1, size=20000, dtype=np.int64),
                             np.array([0, 1, -1, cap, -cap, cap // 2, -(cap // 2)], dtype=np.int64)])
    # any int32 representative of each residue, including extreme magnitudes
    sums = np.stack([
        np.mod(values, m) + m * rng.integers(-(2**31) // m + 2, (2**31) // m - 2, size=values.shape)
        for m in mods
    ]).astype(np.int64)
    assert np.all(np.abs(sums) < 2**31)
    got = _host_reconstruct(native, sums.astype(np.int32), mods)
    assert np.array_equal(got, values)
    assert np.array_equal(got, O.decode_garner(sums, mods))
    # prefix (adaptive) reconstruction: small values through the first 2.. channels
    for active in range(2, len(mods) + 1):
        cap_a = O.signed_capacity(mods[:active])
        small = rng.integers(-cap_a, cap_a + 1, size=2000, dtype=np.int64)
        sums_a = np.stack([np.mod(small, m) - m * 7 for m in mods]).astype(np.int32)
        assert np.array_equal(_host_reconstruct(native, sums_a, mods, active), small)


def test_device_reconstruction_wraps_like_reference(native):
    # beyond the capacity both must return the same representative in (-P/2, P/2]
    for mods in (C0, (126, 125), (255, 254, 253), C4):
        p = int(np.prod(np.array(mods, dtype=object)))
        values = np.array([p // 2, p // 2 + 1, -(p // 2), -(p // 2) - 1, p - 1, 1 - p, p // 2 - 1], dtype=object)
        sums = np.stack([np.array([int(v) % m for v in values]) for m in mods]).astype(np.int32)
        expect = O.decode_garner(sums, mods)
        assert np.array_equal(_host_reconstruct(native, sums, mods), expect)


@pytest.mark.parametrize("mods", [C0, C4, DENSE, (86, 87, 89), (254, 255, 253), (128, 127, 125)])
def test_packed_encoder_exhaustive(native, mods):
    values = np.tile(np.arange(-128, 128, dtype=np.int8), 3)[: 256 * 3]
    rng = np.random.default_rng(5)
    rng.shuffle(values)
    out = np.empty((len(mods), values.size), dtype=np.int8)
    native.check(native.load().rns_host_encode_centered_i8(
        values.ctypes.data, values.size, native.moduli_array(mods), len(mods), out.ctypes.data))
    assert np.array_equal(out, O.encode_centered(values, mods, "device"))


def test_reduced_encoder_every_modulus(native):
    """The fused kernel's default encoder: congruent, inside int8, for any moduli;
    within 64 of zero for the moduli just below 128."""
    values = np.arange(-128, 128, dtype=np.int8)
    lib = native.load()
    for start in range(2, 256, 6):
        mods = [m for m in range(start, min(start + 6, 256))]
        # coprimality is not needed by the encoder, but the plan builder checks it: one modulus at a time
        for m in mods:
            pair = (m, m + 1) if m < 255 else (254, 255)
            out = np.empty((2, 256), dtype=np.int8)
            native.check(lib.rns_host_encode_reduced_i8(values.ctypes.data, 256, native.moduli_array(pair), 2,
                                                        out.ctypes.data))
            for c, mod in enumerate(pair):
                assert np.all((out[c].astype(int) - values.astype(int)) % mod == 0), mod
                changed = out[c] != values
                if mod <= 191:
                    assert np.array_equal(changed, (values >= 64) | (values < -64)), mod
                else:
                    assert not changed.any()
    out = np.empty((5, 256), dtype=np.int8)
    native.check(lib.rns_host_encode_reduced_i8(values.ctypes.data, 256, native.moduli_array(C4), 5, out.ctypes.data))
    assert int(np.abs(out.astype(int)).max()) == 64
    exact = O.encode_centered(values, C4, "device").astype(int)
    near = np.abs(np.abs(values.astype(int)) - 64) <= 8
    assert np.array_equal(out.astype(int)[:, ~near], exact[:, ~near])


def test_packed_encoder_rejects_small_moduli(native):
    values = np.zeros(4, dtype=np.int8)
    out = np.empty((2, 4), dtype=np.int8)
    with pytest.raises(ValueError):
        native.check(native.load().rns_host_encode_centered_i8(
            values.ctypes.data, 4, native.moduli_array((85, 127)), 2, out.ctypes.data))
    # the fused kernel's default (one-step reduced) encoder takes any moduli
    assert native.load().rns_linear_fused_supported(native.moduli_array((85, 127)), 2, 64, 64, 64) == 1
    assert native.load().rns_linear_fused_supported(native.moduli_array(C0), 4, 768, 768, 768) == 1
    assert native.load().rns_linear_fused_supported(native.moduli_array(C0), 4, 100, 100, 100) == 0
