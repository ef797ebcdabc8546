"""Sources wider than int8 (quant_bits 12 / 16 of the reference's RNSLinear,
src/rns_llm/layers/rns_linear.py:45-46, 96-98; tests/test_cuda_backend.py:49-58, 73-94) on the
tensor cores: residue planes of the activations from the quantiser, cached residue planes of the
weight (rns_linear_args.w_channel_stride), the two-CTA kernel with one int8 MMA per channel.

Level 1: reconstructed integers bit-exact against the int64 oracle.  Level 2: the module's
outputs bit-equal to the oracle's restatement of RNSLinear.forward with the same quant_max.
"""
import numpy as np
import pytest
import torch

from oracle import rns_oracle as O
from rns_llm_b200.reference import choose_moduli_for_dot
from tests.test_gpu_pair import tiled_plane_offsets

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    from rns_llm_b200.backends import CudaRNSBackend
    return CudaRNSBackend()


def wide_int(backend, a, w_kn, mods, out_dtype=torch.int64):
    """a int16 [M,K] x w int16 [K,N] through prepare_weight's packed planes and host-tiled
    activation planes."""
    from rns_llm_b200 import _native as N
    lib = N.load()
    m, k = a.shape
    rows = int(lib.rns_pair_tile_rows(len(mods), k))
    assert rows == {4: 64, 5: 48, 6: 32}[len(mods)]
    prepared = backend.prepare_weight(torch.from_numpy(w_kn).cuda(), mods)
    assert prepared.weight_planes_packed is not None and prepared.weight_plane_stride % 16 == 0
    nbytes = int(lib.rns_packed_planes_bytes(m, k, len(mods), rows))
    host = np.full(nbytes, 55, dtype=np.int8)                   # pad rows / columns hold junk
    planes = O.encode_centered(a, mods, "device")               # [R, M, K]
    host[tiled_plane_offsets(m, k, len(mods), rows)] = np.moveaxis(planes, 0, 2)
    out = torch.full((m, w_kn.shape[1]), -7, dtype=out_dtype, device="cuda")
    backend._launch_fused(prepared=prepared, m=m, a=None, a_planes=torch.from_numpy(host).cuda(), a_packed=True,
                          out=out, a_tile_rows=rows, weight_planes=True)
    torch.cuda.synchronize()
    backend.check_status()
    return out.cpu().numpy()


@pytest.mark.parametrize("bits,strategy", [(12, "dense_coprime"), (12, "large_primes"), (16, "dense_coprime"),
                                           (16, "large_primes")])
@pytest.mark.parametrize("m,k,n", [(256, 512, 256), (300, 1024, 260), (130, 528, 1000), (1300, 576, 2000)])
def test_wide_exact_integers(backend, bits, strategy, m, k, n):
    qmax = (1 << (bits - 1)) - 1
    mods = choose_moduli_for_dot(k, qmax, qmax, strategy=strategy)
    assert len(mods) == (5 if bits == 12 else 6)
    rng = np.random.default_rng(bits + m + k + n)
    a = rng.integers(-qmax, qmax + 1, size=(m, k)).astype(np.int16)
    w = rng.integers(-qmax, qmax + 1, size=(k, n)).astype(np.int16)
    a[0, :] = qmax; a[1, :] = -qmax; w[:, 0] = qmax; w[:, 1] = -qmax      # the largest dot products
    assert np.array_equal(wide_int(backend, a, w, mods), O.exact_matmul(a, w))


def test_wide_four_channels(backend):
    """Nine-bit sources at K = 512 fit four channels: the third per-channel-weight form."""
    qmax, m, k, n = 255, 384, 512, 300
    mods = choose_moduli_for_dot(k, qmax, qmax, strategy="large_primes")
    assert len(mods) == 4
    rng = np.random.default_rng(4)
    a = rng.integers(-qmax, qmax + 1, size=(m, k)).astype(np.int16)
    w = rng.integers(-qmax, qmax + 1, size=(k, n)).astype(np.int16)
    assert np.array_equal(wide_int(backend, a, w, mods), O.exact_matmul(a, w))


@pytest.mark.parametrize("bits", [12, 16])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("per_row", [False, True])
def test_wide_linear_forward_matches_oracle(backend, bits, dtype, per_row):
    from rns_llm_b200.layers import RNSLinear
    torch.manual_seed(bits + int(per_row))
    m, k, n = 600, 1024, 392
    layer = RNSLinear(k, n, backend=backend, mode="rns", quant_bits=bits,
                      activation_scale="row" if per_row else "tensor").to(dtype).cuda().eval()
    x = torch.randn(3, m // 3, k).to(dtype)
    np_dtype = np.float16 if dtype == torch.float16 else np.float32
    res = O.rns_linear_forward(x.float().numpy(), layer.weight.detach().float().cpu().numpy(),
                               layer.bias.detach().float().cpu().numpy(), layer.moduli,
                               quant_max=layer.quant_max, per_row=per_row, out_dtype=np_dtype)
    backend.reset_stats()
    with torch.no_grad():
        y = layer(x.cuda())
    torch.cuda.synchronize()
    backend.check_status()
    assert layer._prepared_weight.weight_planes_packed is not None
    assert np.array_equal(layer._weight_scale.cpu().numpy(), res["w_scale"])        # the weight side, stage by stage
    w_planes = layer._prepared_weight.residues.cpu().numpy()                        # [R, K, N]
    assert np.array_equal(w_planes, O.encode_centered(res["w_q"].T, layer.moduli, "device"))
    assert backend.stats_snapshot()[f"fused_gemm_channels_{len(layer.moduli)}"] == 1
    assert y.shape == (3, m // 3, n)
    assert np.array_equal(y.cpu().numpy(), res["y"])


def test_wide_few_rows_stay_on_the_plane_pipeline(backend):
    from rns_llm_b200.layers import RNSLinear
    torch.manual_seed(3)
    layer = RNSLinear(1024, 64, backend=backend, mode="rns", quant_bits=16).cuda().eval()
    x = torch.randn(8, 1024, device="cuda")
    with torch.no_grad():
        y = layer(x)
    ref = torch.nn.functional.linear(x, layer.weight, layer.bias)
    assert float((y - ref).abs().max()) < 1e-3
    assert not backend.supports_wide_forward(layer._prepared_weight, 8)
    backend.check_status()


def test_wide_quantiser_refuses_integer_output(backend):
    from rns_llm_b200 import _native as N
    lib = N.load()
    x = torch.randn(128, 512, device="cuda", dtype=torch.float16)
    q = torch.empty(128 * 512, dtype=torch.int8, device="cuda")
    scale = torch.empty(1, device="cuda")
    scratch = torch.zeros(16, dtype=torch.int8, device="cuda")
    rc = lib.rns_quantize_activations_tiled(x.data_ptr(), N.F16, 128, 512, 512, 0, 0, 0, 2047,
                                            N.moduli_array((251, 241, 239, 233, 229)), 5, q.data_ptr(), None, 1, 0,
                                            scale.data_ptr(), None, scratch.data_ptr(), None, 0, 0,
                                            torch.cuda.current_stream().cuda_stream)
    assert rc != N.OK
