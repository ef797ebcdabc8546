"""The oracle (NumPy and C restatements) against the reference's golden outputs
and against the relations the reference's own tests assert."""
import numpy as np
import pytest

from oracle import rns_oracle as O

C0 = (127, 126, 125, 121)
C4 = (127, 126, 125, 121, 113)
DENSE = (255, 253, 251, 247)


def test_constants_match_reference(golden):
    g = golden("constants")
    for tag, mods in (("c0", C0), ("c4", C4), ("dense", DENSE)):
        product, coeffs = O.crt_coefficients(mods)
        assert product == int(g[f"{tag}_product"][0])
        assert coeffs == [int(v) for v in g[f"{tag}_crt"]]
        assert np.array_equal(np.array(O.pairwise_inverses(mods)), g[f"{tag}_pairinv"])
    for bound, expected in zip(g["prefix_bounds"], g["prefix_channels_min2"]):
        if expected < 0:
            with pytest.raises(OverflowError):
                O.minimal_prefix_channels(C0, int(bound), 2)
        else:
            assert O.minimal_prefix_channels(C0, int(bound), 2) == int(expected)
    assert O.signed_capacity(C0) == int(g["capacity_c0"][0])


def test_encoders_match_reference(golden):
    g = golden("encode_decode")
    values = np.arange(-128, 128)
    for tag, mods in (("c0", C0), ("c4", C4), ("dense", DENSE)):
        assert np.array_equal(O.encode_centered(values, mods, "numpy"), g[f"{tag}_centered_all_i8"])
        assert np.array_equal(O.encode_canonical(values, mods), g[f"{tag}_canonical_all_i8"])
    assert np.array_equal(O.encode_centered(g["wide_values"], DENSE), g["wide_centered_dense"])


def test_device_convention_differs_only_at_even_half():
    values = np.arange(-128, 128)
    a = O.encode_centered(values, C0, "numpy").astype(int)
    b = O.encode_centered(values, C0, "device").astype(int)
    diff = np.argwhere(a != b)
    # only modulus 126 (channel 1), only value -63, +63 vs -63
    assert [(int(c), int(values[i])) for c, i in diff] == [(1, -63)]
    assert a[1, 128 - 63] == 63 and b[1, 128 - 63] == -63
    for c, m in enumerate(C0):
        assert np.all((b[c] - values) % m == 0) and np.all(np.abs(b[c]) <= m // 2)


def test_garner_matches_reference_on_raw_sums(golden, c_oracle):
    g = golden("encode_decode")
    assert np.array_equal(O.decode_garner(g["garner_sums_c0"], C0), g["garner_values_c0"])
    assert np.array_equal(O.decode_garner(g["garner_sums_c4"], C4), g["garner_values_c4"])
    assert np.array_equal(c_oracle.garner(g["garner_sums_c0"], C0), g["garner_values_c0"])
    assert np.array_equal(c_oracle.garner(g["garner_sums_c4"], C4), g["garner_values_c4"])
    wrapped = O.decode_garner(O.encode_centered(g["wrap_inputs_c0"], C0), C0)
    assert np.array_equal(wrapped, g["wrap_outputs_c0"])


def test_signed_roundtrip_like_reference_tests():
    # tests/test_reference.py:11-14 and :49-57 of the reference
    mods = (251, 241, 239, 233)
    values = np.arange(-10000, 10001, dtype=np.int64)
    assert np.array_equal(O.decode_crt(O.encode_canonical(values, mods), mods), values)
    rng = np.random.default_rng(123)
    values = rng.integers(-1_000_000, 1_000_001, size=(17, 13), dtype=np.int64)
    assert np.array_equal(O.decode_garner(O.encode_centered(values, DENSE), DENSE), values)


def test_gemm_matches_reference(golden, c_oracle):
    g = golden("gemm")
    a, b = g["small_a"], g["small_b"]
    assert np.array_equal(O.rns_matmul(a, b, C0), g["small_out_c0"])
    assert np.array_equal(O.rns_matmul(a, b, C0, decode=False), g["small_residues_c0"])
    assert np.array_equal(O.exact_matmul(a, b), g["small_out_c0"])
    assert np.array_equal(O.exact_matmul(a, b), g["small_out_legacy"])
    assert np.array_equal(O.rns_matmul_device_pipeline(a, b, C0), g["small_out_c0"])
    got, _ = c_oracle.linear(a, b.T.copy(), C0)
    assert np.array_equal(got, g["small_out_c0"])


def test_config0_checksum(golden, c_oracle):
    g = golden("gemm")
    rng = np.random.default_rng(1000)
    a = rng.integers(-127, 128, size=(128, 768), dtype=np.int64).astype(np.int8)
    b = rng.integers(-127, 128, size=(768, 768), dtype=np.int64).astype(np.int8)
    out = O.exact_matmul(a, b)
    sums = [int(out.sum()), int(np.abs(out).sum()), int(out[0, 0]), int(out[-1, -1])]
    assert sums == [int(v) for v in g["c0_checksum"]]
    assert np.array_equal(out[:4], g["c0_out_rows"])
    got, _ = c_oracle.linear(a, b.T.copy(), C0)
    assert np.array_equal(got, out)
    assert np.array_equal(O.rns_matmul_device_pipeline(a[:16], b, C0), out[:16])


@pytest.mark.parametrize("tag", ["qkv16", "odd"])
def test_rns_linear_forward_matches_reference(golden, c_oracle, tag):
    g = golden("rns_linear")
    res = O.rns_linear_forward(g[f"{tag}_x"], g[f"{tag}_weight"], g[f"{tag}_bias"], C0)
    assert np.array_equal(res["a_q"], g[f"{tag}_a_q"])
    assert np.array_equal(res["w_q"], g[f"{tag}_w_q"])
    assert np.array_equal(res["a_scale"], g[f"{tag}_a_scale"])
    assert np.array_equal(res["w_scale"], g[f"{tag}_w_scale"])
    assert np.array_equal(res["integer"], g[f"{tag}_integer"])
    assert np.array_equal(res["y"].view(np.uint16), g[f"{tag}_y"].view(np.uint16))  # bit-exact fp16
    ints, floats = c_oracle.linear(res["a_q"], res["w_q"], C0, res["a_scale"], res["w_scale"],
                                   g[f"{tag}_bias"].astype(np.float32), want_float=True)
    assert np.array_equal(ints, g[f"{tag}_integer"])
    assert np.array_equal(floats.astype(np.float16).reshape(g[f"{tag}_y"].shape).view(np.uint16),
                          g[f"{tag}_y"].view(np.uint16))


def test_adaptive_bound_is_safe():
    # tests/test_reference.py:84-95 of the reference
    rng = np.random.default_rng(77)
    a = rng.integers(-40, 41, size=(9, 31), dtype=np.int64)
    b = rng.integers(-50, 51, size=(31, 7), dtype=np.int64)
    bound = O.safe_l1_dot_bound(int(np.abs(a).sum(axis=1).max()), int(np.abs(b).max()))
    assert int(np.abs(a @ b).max()) <= bound
    channels, bound2 = O.adaptive_channels(a, b.T, DENSE, 3)
    assert 2 * bound2 < int(np.prod(DENSE[:channels]))


def test_adaptive_prefix_config2():
    rng = np.random.default_rng(1002)
    a_low = rng.integers(-15, 16, size=(128, 768), dtype=np.int64)
    a_full = rng.integers(-127, 128, size=(128, 768), dtype=np.int64)
    w = rng.integers(-127, 128, size=(768, 768), dtype=np.int64)
    assert O.adaptive_channels(a_low, w, C0, 3)[0] == 3
    assert O.adaptive_channels(a_full, w, C0, 3)[0] == 4
    assert np.array_equal(O.rns_matmul_device_pipeline(a_low[:8], w.T, C0, active=3),
                          O.exact_matmul(a_low[:8], w.T))
