"""Plane-level entry points on the GPU against the oracle; the cases of the
reference's tests/test_cuda_backend.py, seeded."""
import numpy as np
import pytest
import torch

from oracle import rns_oracle as O

pytestmark = pytest.mark.gpu

C0 = (127, 126, 125, 121)
DENSE = (255, 253, 251, 247)


@pytest.fixture(scope="module")
def backend():
    from rns_llm_b200.backends import CudaRNSBackend
    return CudaRNSBackend()


def dev(arr):
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


@pytest.mark.parametrize("dtype,lo,hi", [(np.int8, -128, 128), (np.int16, -32768, 32768), (np.int32, -10**6, 10**6)])
def test_encode_centered_device_convention(backend, dtype, lo, hi):
    rng = np.random.default_rng(11)
    values = rng.integers(lo, hi, size=(37, 53)).astype(dtype)
    for mods in (C0, DENSE, (3, 5, 7, 11, 13)):
        got = backend.encode_centered(dev(values), mods).cpu().numpy()
        assert np.array_equal(got, O.encode_centered(values, mods, "device"))


def test_encode_canonical(backend):
    values = np.arange(-128, 128, dtype=np.int8).reshape(16, 16)
    got = backend.encode(dev(values), C0).cpu().numpy()
    assert np.array_equal(got, O.encode_canonical(values, C0))
    with pytest.raises(ValueError):
        backend.encode(dev(values.astype(np.int16)), C0)


@pytest.mark.parametrize("kernel", ["scalar", "dp4a", "dp4a_safe", "auto", "cublas"])
def test_matmul_wide_int8(backend, kernel):
    rng = np.random.default_rng(21)
    shape = (32, 64, 32) if kernel == "cublas" else (17, 64, 20)
    a = rng.integers(-127, 128, size=shape[:2]).astype(np.int8)
    b = rng.integers(-127, 128, size=shape[1:]).astype(np.int8)
    from rns_llm_b200.moduli import choose_moduli_for_dot
    mods = choose_moduli_for_dot(64, 127, 127)
    got = backend.matmul_wide(dev(a), dev(b), mods, kernel=kernel).cpu().numpy()
    assert np.array_equal(got, O.exact_matmul(a, b))


def test_wide_int12_exactness_and_fused_garner(backend):
    from rns_llm_b200.moduli import choose_moduli_for_dot
    rng = np.random.default_rng(22)
    a = rng.integers(-2047, 2048, size=(24, 64)).astype(np.int16)
    b = rng.integers(-2047, 2048, size=(64, 32)).astype(np.int16)
    mods = choose_moduli_for_dot(64, 2047, 2047, strategy="dense_coprime")
    exact = O.exact_matmul(a, b)
    assert np.array_equal(backend.matmul_wide(dev(a), dev(b), mods).cpu().numpy(), exact)
    prepared = backend.prepare_weight(dev(b), mods)
    assert prepared.kernel == "cublas"
    for lut_channels in (0, 1, 2):
        ws = backend.create_workspace(device=torch.device("cuda"), channels=len(mods), m=24, n=32)
        got = backend.matmul_prepared_fused(dev(a), prepared, lut_channels=lut_channels, workspace=ws)
        assert got.data_ptr() == ws.output.data_ptr()
        assert np.array_equal(got.cpu().numpy(), exact)
    assert np.array_equal(backend.matmul_prepared(dev(a), prepared).cpu().numpy(), exact)


def test_canonical_planes_gemm(backend):
    rng = np.random.default_rng(23)
    a = rng.integers(-127, 128, size=(13, 29)).astype(np.int8)
    b = rng.integers(-127, 128, size=(29, 17)).astype(np.int8)
    mods = (251, 241, 239, 233)
    ra, rb = backend.encode(dev(a), mods), backend.encode(dev(b), mods)
    for kernel in ("auto", "naive", "tiled", "tiled_safe"):
        got = backend.matmul_residues(ra, rb, mods, kernel=kernel).cpu().numpy()
        assert np.array_equal(got, O.rns_matmul(a, b, mods, decode=False))
    decoded = backend.decode(backend.matmul_residues(ra, rb, mods), mods).cpu().numpy()
    assert np.array_equal(decoded, O.exact_matmul(a, b))


def test_garner_decoder_matches_crt_decoder(backend):
    rng = np.random.default_rng(24)
    a = rng.integers(-127, 128, size=(32, 64)).astype(np.int8)
    b = rng.integers(-127, 128, size=(64, 32)).astype(np.int8)
    ra, rb = backend.encode_centered(dev(a), DENSE), backend.encode_centered(dev(b), DENSE)
    residues = backend.matmul_centered_residues(ra, rb, DENSE, kernel="cublas")
    old = backend.decode(residues, DENSE)
    new = backend.decode_garner(residues, DENSE)
    assert torch.equal(old, new)
    assert np.array_equal(new.cpu().numpy(), O.exact_matmul(a, b))


def test_garner_on_golden_values(backend, golden):
    g = golden("encode_decode")
    for tag, mods in (("c0", C0), ("c4", (127, 126, 125, 121, 113))):
        values = g[f"garner_values_{tag}"]
        planes = O.encode_centered(values, mods, "device")
        got = backend.decode_garner(dev(planes), mods).cpu().numpy()
        assert np.array_equal(got, values)
    wrap = O.encode_centered(g["wrap_inputs_c0"], C0, "device")
    assert np.array_equal(backend.decode_garner(dev(wrap), C0).cpu().numpy(), g["wrap_outputs_c0"])


def test_plane_level_errors(backend):
    a = torch.zeros((4, 8, 16), dtype=torch.int8, device="cuda")
    b = torch.zeros((4, 16, 6), dtype=torch.int8, device="cuda")
    with pytest.raises(ValueError):
        backend.matmul_centered_fused(a, b, C0)                       # N % 4 != 0
    with pytest.raises(ValueError):
        backend.matmul_centered_fused(a, b[:, :8].contiguous(), C0)   # K mismatch
    with pytest.raises(ValueError):
        backend.matmul_centered_residues(a, b, C0[:3])                # moduli count
    with pytest.raises(ValueError):
        backend.matmul_centered_residues(a.cpu(), b, C0)              # device
    with pytest.raises(ValueError):
        backend.matmul_centered_residues(a.transpose(1, 2), b, C0)    # contiguity
    with pytest.raises(ValueError):
        backend.encode_centered(torch.zeros(4, device="cuda"), C0)    # dtype
    with pytest.raises(ValueError):
        backend.encode_centered(torch.zeros(4, dtype=torch.int8, device="cuda"), (126, 124))
    ws = backend.create_workspace(device=a.device, channels=4, m=9, n=8)
    b8 = torch.zeros((4, 16, 8), dtype=torch.int8, device="cuda")
    with pytest.raises(ValueError):
        backend.matmul_centered_fused(a, b8, C0, workspace=ws)        # workspace shape
