"""The one-launch few-token kernel (rns_linear_small) through the C ABI: exact integers on
int8 activations, bit-exact dequantised outputs on floating activations (per-tensor and
per-row scales) against the oracle, refusal outside its range."""
import numpy as np
import pytest
import torch

from oracle import rns_oracle as O

pytestmark = pytest.mark.gpu

C0 = (127, 126, 125, 121)
C4 = (127, 126, 125, 121, 113)


@pytest.fixture(scope="module")
def backend():
    from rns_llm_b200.backends import CudaRNSBackend
    return CudaRNSBackend()


def representative(exact, mods):
    """What an RNS with these moduli returns for `exact`: the residue class modulo
    P = prod(mods) in (-P/2, P/2] (csrc/rns_cuda.cu:380-414 of the reference); the exact value
    itself whenever it fits the capacity."""
    product = int(np.prod([int(m) for m in mods], dtype=object))
    wrapped = np.mod(exact, product)
    return np.where(wrapped > product // 2, wrapped - product, wrapped)


def call_small(backend, x, w_q, mods, *, x_type, per_row=False, col_scale=None, bias=None, out_dtype=torch.int64):
    from rns_llm_b200 import _native as N
    from rns_llm_b200.backends.cuda_backend import _OUT_TYPES
    lib = N.load()
    prepared = backend.prepare_weight_nk(w_q, mods)
    m, k = x.shape
    out = torch.full((m, w_q.shape[0]), -7, dtype=out_dtype, device="cuda")
    assert lib.rns_linear_small_supported(m, k, len(mods)) == 1
    N.check(lib.rns_linear_small(x.data_ptr(), x_type, m, k, x.stride(0), 1 if per_row else 0,
                                 prepared.weight_packed.data_ptr(), w_q.shape[0], N.moduli_array(mods), len(mods),
                                 None if col_scale is None else col_scale.data_ptr(),
                                 None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0),
                                 _OUT_TYPES[out_dtype], torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("mods", [(127, 125), C0, C4, (255, 253, 251, 247)])
@pytest.mark.parametrize("m,k,n", [(1, 768, 2304), (16, 768, 768), (4, 64, 20), (17, 256, 33), (32, 1536, 100),
                                   (3, 16, 8), (5, 80, 9), (2, 144, 24)])
def test_small_kernel_exact_integers(backend, mods, m, k, n):
    rng = np.random.default_rng(m * 31 + k + n + len(mods))
    a = rng.integers(-128, 128, size=(m, k)).astype(np.int8)
    w = rng.integers(-128, 128, size=(n, k)).astype(np.int8)
    from rns_llm_b200 import _native as N
    expect = representative(O.exact_matmul(a, w.T), mods)       # (127, 125) cannot hold these products: wraps
    if N.load().rns_linear_small_supported(m, k, len(mods)) == 1:
        got = call_small(backend, torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda(), mods, x_type=-1)
        assert np.array_equal(got.cpu().numpy(), expect)
    else:
        # the residues of all tokens do not fit the kernel's shared memory: the backend takes another route
        assert len(mods) * k * 16 > 96 * 1024
    # and through the backend entry the reference exposes (matmul_prepared_fused picks this kernel)
    prepared = backend.prepare_weight_nk(torch.from_numpy(w).cuda(), mods)
    assert np.array_equal(backend.matmul_prepared_fused(torch.from_numpy(a).cuda(), prepared).cpu().numpy(), expect)
    backend.check_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("per_row", [False, True])
@pytest.mark.parametrize("m,k,n", [(1, 768, 2304), (16, 768, 96), (19, 256, 136), (32, 80, 40)])
def test_small_kernel_dequantised_outputs(backend, dtype, per_row, m, k, n):
    from rns_llm_b200 import _native as N
    torch.manual_seed(m + k + n)
    x = torch.randn(m, k).to(dtype)
    weight = (torch.randn(n, k) * 0.05).to(dtype)
    bias = torch.randn(n).to(dtype)
    np_dtype = {torch.float16: np.float16, torch.float32: np.float32}.get(dtype, np.float32)
    res = O.rns_linear_forward(x.float().numpy(), weight.float().numpy(), bias.float().numpy(), C0,
                               per_row=per_row, out_dtype=np_dtype)
    w_q, w_scale, _ = backend.quantize_weight(weight.cuda())
    x_type = {torch.float16: N.F16, torch.bfloat16: N.BF16, torch.float32: N.F32}[dtype]
    y = call_small(backend, x.cuda(), w_q, C0, x_type=x_type, per_row=per_row, col_scale=w_scale,
                   bias=bias.float().cuda(), out_dtype=dtype)
    if dtype == torch.bfloat16:
        assert torch.equal(y.cpu(), torch.from_numpy(res["y"]).to(torch.bfloat16))
    else:
        assert np.array_equal(y.cpu().numpy(), res["y"])
    # the module path takes the same kernel
    y2 = backend.linear_forward(x.cuda(), backend.prepare_weight_nk(w_q, C0), w_scale, bias.float().cuda(),
                                per_row=per_row)
    assert torch.equal(y2, y)
    backend.check_status()


def test_small_kernel_refuses_what_it_does_not_cover(backend):
    from rns_llm_b200 import _native as N
    lib = N.load()
    assert lib.rns_linear_small_supported(33, 768, 4) == 0
    assert lib.rns_linear_small_supported(4, 8192, 4) == 0          # residues would not fit shared memory
    assert lib.rns_linear_small_supported(4, 72, 4) == 0            # K % 16 != 0
    assert lib.rns_linear_small_supported(4, 768, 7) == 0
    x = torch.zeros((33, 64), dtype=torch.int8, device="cuda")
    code = lib.rns_linear_small(x.data_ptr(), -1, 33, 64, 64, 0, x.data_ptr(), 8, N.moduli_array(C0), 4, None, None,
                                x.data_ptr(), 8, N.OUT_INT64, None)
    assert code == N.ERR_UNSUPPORTED
    assert lib.rns_linear_small(None, -1, 1, 64, 64, 0, None, 8, N.moduli_array(C0), 4, None, None, None, 8,
                                N.OUT_INT64, None) == N.ERR_INVALID_ARGUMENT


# ---------------------------------------------------------------------------
# Few tokens on large weights: the weight-streaming kernel (rns_linear_stream)
# ---------------------------------------------------------------------------
def call_stream(backend, a_q, w_q, mods, *, row_scale=None, per_row=False, col_scale=None, bias=None,
                out_dtype=torch.int64):
    from rns_llm_b200 import _native as N
    from rns_llm_b200.backends.cuda_backend import _OUT_TYPES
    lib = N.load()
    prepared = backend.prepare_weight_nk(w_q, mods)
    m, k = a_q.shape
    assert lib.rns_linear_stream_supported(m, k, len(mods)) == 1
    out = torch.full((m, w_q.shape[0]), -7, dtype=out_dtype, device="cuda")
    N.check(lib.rns_linear_stream(a_q.data_ptr(), m, k, a_q.stride(0),
                                  None if row_scale is None else row_scale.data_ptr(), 1 if per_row else 0,
                                  prepared.weight_packed.data_ptr(), w_q.shape[0], N.moduli_array(mods), len(mods),
                                  None if col_scale is None else col_scale.data_ptr(),
                                  None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0),
                                  _OUT_TYPES[out_dtype], torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("mods", [C0, C4, (255, 253, 251, 247), (127, 126, 125)])
@pytest.mark.parametrize("m,k,n", [(1, 4096, 520), (7, 2048, 96), (16, 3072, 768), (32, 4112, 100), (33, 1040, 40),
                                   (64, 512, 264), (3, 16, 8), (17, 528, 33)])
def test_stream_kernel_exact_integers(backend, mods, m, k, n):
    rng = np.random.default_rng(m * 7 + k + n + len(mods))
    a = rng.integers(-128, 128, size=(m, k)).astype(np.int8)
    w = rng.integers(-128, 128, size=(n, k)).astype(np.int8)
    expect = representative(O.exact_matmul(a, w.T), mods)
    got = call_stream(backend, torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda(), mods)
    assert np.array_equal(got.cpu().numpy(), expect)
    backend.check_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("per_row", [False, True])
@pytest.mark.parametrize("m,k,n,mods", [(1, 4096, 1024, C0), (8, 3072, 768, C0), (32, 16384, 136, C4), (19, 2064, 40, C0),
                                        (4, 4096, 4096, C0)])
def test_few_tokens_on_large_weights_match_the_oracle(backend, dtype, per_row, m, k, n, mods):
    """linear_forward for at most 32 tokens on a K the one-launch kernel cannot hold: quantiser +
    the weight-streaming kernel (weights below 2^23 values; the last shape is above and takes the
    two-CTA kernel), bit-equal to the oracle's forward."""
    from rns_llm_b200 import _native as N
    assert N.load().rns_linear_small_supported(m, k, len(mods)) == 0
    torch.manual_seed(m + k + n)
    x = torch.randn(m, k).to(dtype)
    weight = (torch.randn(n, k) * 0.05).to(dtype)
    bias = torch.randn(n).to(dtype)
    np_dtype = {torch.float16: np.float16, torch.float32: np.float32}.get(dtype, np.float32)
    res = O.rns_linear_forward(x.float().numpy(), weight.float().numpy(), bias.float().numpy(), mods,
                               per_row=per_row, out_dtype=np_dtype)
    w_q, w_scale, _ = backend.quantize_weight(weight.cuda())
    prepared = backend.prepare_weight_nk(w_q, mods)
    y = backend.linear_forward(x.cuda(), prepared, w_scale, bias.float().cuda(), per_row=per_row)
    torch.cuda.synchronize()
    backend.check_status()
    if dtype == torch.bfloat16:
        assert torch.equal(y.cpu(), torch.from_numpy(res["y"]).to(torch.bfloat16))
    else:
        assert np.array_equal(y.cpu().numpy(), res["y"])
    # the same call through the two-CTA kernel (what served it before) gives the same bits
    from rns_llm_b200.backends import cuda_backend as CB
    saved, CB.STREAM_MAX_ROWS = CB.STREAM_MAX_ROWS, 0
    try:
        other = backend.linear_forward(x.cuda(), prepared, w_scale, bias.float().cuda(), per_row=per_row)
    finally:
        CB.STREAM_MAX_ROWS = saved
    assert torch.equal(y, other)
