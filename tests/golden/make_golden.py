"""Generates tests/golden/*.npz by running the reference's own Python code.

Run in the build container, where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

The reference cannot travel to the GPU machine, so its outputs on seeded
inputs are frozen here and the tests compare the oracle (oracle/rns_oracle.py),
the host-side constants of the package and the CUDA path against them.
Everything stored is produced by reference functions
(src/rns_llm/reference.py, src/rns_llm/adaptive.py, src/rns_llm/rns/*,
RNSLinear._symmetric_scale/_quantize in src/rns_llm/layers/rns_linear.py);
inputs come from seeded generators and are stored next to the outputs.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
MODULI_C0 = (127, 126, 125, 121)
MODULI_C4 = (127, 126, 125, 121, 113)
MODULI_DENSE = (255, 253, 251, 247)


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "src"))
    import torch
    from rns_llm import adaptive, reference
    from rns_llm.layers.rns_linear import RNSLinear
    from rns_llm.rns import matmul as legacy_matmul

    # ---- constants ---------------------------------------------------------
    const = {}
    for tag, mods in (("c0", MODULI_C0), ("c4", MODULI_C4), ("dense", MODULI_DENSE)):
        product, coeffs = reference.crt_constants(mods)
        const[f"{tag}_moduli"] = np.array(mods, dtype=np.int64)
        const[f"{tag}_product"] = np.array([product], dtype=np.int64)
        const[f"{tag}_crt"] = np.array(coeffs, dtype=np.int64)
        const[f"{tag}_pairinv"] = np.array(reference.garner_pairwise_inverses(mods), dtype=np.int64)
        const[f"{tag}_lut"] = reference.compact_byte_mod_lut(mods)
    for strategy in ("large_primes", "dense_coprime", "small_primes"):
        const[f"cand_{strategy}"] = np.array(reference.candidates_for_strategy(strategy), dtype=np.int64)
        for k, qa in ((64, 127), (768, 127), (4096, 127), (16384, 127), (64, 2047), (768, 2047), (768, 32767)):
            const[f"choose_{strategy}_{k}_{qa}"] = np.array(
                reference.choose_moduli_for_dot(k, qa, qa, strategy=strategy), dtype=np.int64)
    bounds = np.array([0, 1, 1000, 808_000, 1_000_124, 1_000_125, 5_000_000, 121_015_124, 121_015_125], dtype=np.int64)
    chosen = []
    for b in bounds:
        try:
            chosen.append(adaptive.minimal_prefix_channels(MODULI_C0, int(b), min_channels=2))
        except OverflowError:
            chosen.append(-1)
    const["prefix_bounds"] = bounds
    const["prefix_channels_min2"] = np.array(chosen, dtype=np.int64)
    const["capacity_c0"] = np.array([adaptive.signed_capacity(MODULI_C0)], dtype=np.int64)
    cost = reference.moduli_cost_model(MODULI_C0, m=128, k=768, n=768, source_element_bytes=1, lut_channels=2)
    const["cost_keys"] = np.array(sorted(cost), dtype="U64")
    const["cost_values"] = np.array([float(cost[key]) for key in sorted(cost)], dtype=np.float64)
    np.savez_compressed(HERE / "constants.npz", **const)

    # ---- encode / decode ---------------------------------------------------
    rng = np.random.default_rng(2024)
    enc = {}
    all_i8 = np.arange(-128, 128, dtype=np.int64)
    for tag, mods in (("c0", MODULI_C0), ("c4", MODULI_C4), ("dense", MODULI_DENSE)):
        enc[f"{tag}_centered_all_i8"] = reference.encode_centered_numpy(all_i8, mods)
        enc[f"{tag}_canonical_all_i8"] = reference.encode_numpy(all_i8, mods)
    wide = rng.integers(-32768, 32768, size=(7, 33), dtype=np.int64)
    enc["wide_values"] = wide
    enc["wide_centered_dense"] = reference.encode_centered_numpy(wide, MODULI_DENSE)
    # raw accumulators (any representative) through the reference Garner decoder
    cap = adaptive.signed_capacity(MODULI_C0)
    values = np.concatenate([
        rng.integers(-cap, cap + 1, size=4000, dtype=np.int64),
        np.array([0, 1, -1, cap, -cap, cap - 1, -cap + 1], dtype=np.int64),
    ])
    sums = np.stack([
        reference.encode_centered_numpy(values, MODULI_C0)[c].astype(np.int64)
        + m * rng.integers(-400_000, 400_001, size=values.shape, dtype=np.int64)
        for c, m in enumerate(MODULI_C0)
    ])
    enc["garner_sums_c0"] = sums.astype(np.int32)
    enc["garner_values_c0"] = reference.decode_garner_numpy(sums, MODULI_C0)
    assert np.array_equal(enc["garner_values_c0"], values)
    # beyond-capacity wrap behaviour of the reference decoder (even product)
    product = int(np.prod(MODULI_C0))
    beyond = np.array([cap + 1, cap + 2, -cap - 1, -cap - 2, product // 2, -(product // 2), product, -product + 5], dtype=np.int64)
    enc["wrap_inputs_c0"] = beyond
    enc["wrap_outputs_c0"] = reference.decode_garner_numpy(
        reference.encode_centered_numpy(beyond, MODULI_C0), MODULI_C0)
    cap5 = adaptive.signed_capacity(MODULI_C4)
    values5 = rng.integers(-cap5, cap5 + 1, size=2000, dtype=np.int64)
    sums5 = np.stack([
        reference.encode_centered_numpy(values5, MODULI_C4)[c].astype(np.int64)
        + m * rng.integers(-500_000, 500_001, size=values5.shape, dtype=np.int64)
        for c, m in enumerate(MODULI_C4)
    ])
    enc["garner_sums_c4"] = sums5.astype(np.int32)
    enc["garner_values_c4"] = reference.decode_garner_numpy(sums5, MODULI_C4)
    assert np.array_equal(enc["garner_values_c4"], values5)
    np.savez_compressed(HERE / "encode_decode.npz", **enc)

    # ---- integer GEMMs -----------------------------------------------------
    gemm = {}
    rng = np.random.default_rng(1000)  # config 0 seed
    a = rng.integers(-127, 128, size=(128, 768), dtype=np.int64).astype(np.int8)
    b = rng.integers(-127, 128, size=(768, 768), dtype=np.int64).astype(np.int8)
    out = reference.rns_matmul_numpy(a, b, MODULI_C0)
    assert np.array_equal(out, a.astype(np.int64) @ b.astype(np.int64))
    gemm["c0_checksum"] = np.array([int(out.sum()), int(np.abs(out).sum()), int(out[0, 0]), int(out[-1, -1])], dtype=np.int64)
    gemm["c0_out_rows"] = out[:4].copy()
    rng = np.random.default_rng(7)
    a = rng.integers(-127, 128, size=(17, 64), dtype=np.int64).astype(np.int8)
    b = rng.integers(-127, 128, size=(64, 20), dtype=np.int64).astype(np.int8)
    gemm["small_a"], gemm["small_b"] = a, b
    gemm["small_out_c0"] = reference.rns_matmul_numpy(a, b, MODULI_C0)
    gemm["small_residues_c0"] = reference.rns_matmul_numpy(a, b, MODULI_C0, decode=False)
    gemm["small_out_legacy"] = legacy_matmul.rns_matmul(a.astype(np.int64), b.astype(np.int64), (251, 241, 239, 233))
    np.savez_compressed(HERE / "gemm.npz", **gemm)

    # ---- RNSLinear forward (quantise / dequantise order) --------------------
    lin = {}
    torch.manual_seed(1001)
    for tag, (m, k, n) in (("qkv16", (16, 768, 96)), ("odd", (5, 64, 24))):
        layer = RNSLinear(k, n, bias=True, moduli=MODULI_C0, mode="rns")
        weight = (torch.randn(n, k) * 0.02).half()
        bias = (torch.randn(n) * 0.1).half()
        x = torch.randn(1, m, k).half()
        w32 = weight.float()
        w_scale = layer._symmetric_scale(w32, dim=1)
        w_q = layer._quantize(w32, w_scale)
        flat = x.reshape(-1, k).float().contiguous()
        a_scale = layer._symmetric_scale(flat)
        a_q = layer._quantize(flat, a_scale)
        integer = reference.rns_matmul_numpy(a_q.numpy(), w_q.numpy().T.copy(), MODULI_C0)
        result = torch.from_numpy(integer).float()
        y = result * a_scale * w_scale.squeeze(1).unsqueeze(0)
        y = y + bias.float()
        y = y.reshape(1, m, n).to(x.dtype)
        lin[f"{tag}_x"] = x.numpy()
        lin[f"{tag}_weight"] = weight.numpy()
        lin[f"{tag}_bias"] = bias.numpy()
        lin[f"{tag}_a_q"] = a_q.numpy()
        lin[f"{tag}_a_scale"] = a_scale.numpy().reshape(-1)
        lin[f"{tag}_w_q"] = w_q.numpy()
        lin[f"{tag}_w_scale"] = w_scale.numpy().reshape(-1)
        lin[f"{tag}_integer"] = integer
        lin[f"{tag}_y"] = y.numpy()
    np.savez_compressed(HERE / "rns_linear.npz", **lin)
    for name in ("constants", "encode_decode", "gemm", "rns_linear"):
        print(name, (HERE / f"{name}.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of Nek1tt/rns-llm v0.5>")
    main(sys.argv[1])
