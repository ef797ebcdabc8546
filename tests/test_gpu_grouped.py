"""Grouped multi-head integer products (QK^T and PV of attention) in one launch:
`CudaRNSBackend.matmul_grouped` against the int64 oracle, problem by problem.  The reference
lists the grouped kernel as open work (docs/OPTIMIZATIONS_V04.md:49) and times the shapes of one
head through its plane pipeline (benchmarks/benchmark_attention.py:107-113); the exactness bar is
the same as for every other entry: reconstructed integers bit-equal to the int64 product."""
import numpy as np
import pytest
import torch

from oracle import rns_oracle as O

pytestmark = pytest.mark.gpu

C0 = (127, 126, 125, 121)
C4 = (127, 126, 125, 121, 113)
C6 = (127, 126, 125, 121, 113, 109)


@pytest.fixture(scope="module")
def backend():
    from rns_llm_b200.backends import CudaRNSBackend
    return CudaRNSBackend()


def grouped_exact(a, b_nk):
    return np.einsum("gmk,gnk->gmn", a.astype(np.int64), b_nk.astype(np.int64))


@pytest.mark.parametrize("mods,groups,m,k,n", [
    (C0, 6, 128, 64, 128),        # scores of six heads: T = 128, head_dim = 64 (one K block)
    (C0, 5, 200, 64, 200),        # ragged T: the rows are padded to whole token tiles
    (C0, 3, 256, 256, 64),        # P V: K = T, N = head_dim
    (C0, 24, 512, 64, 512),       # more tiles than resident clusters
    (C0, 7, 130, 80, 72),         # K % 64 != 0, N % 128 != 0, odd group count
    (C4, 4, 192, 1024, 136),      # five channels (96-token tiles), long K
    (C6, 3, 128, 128, 64),        # six channels (64-token tiles)
    (C0, 1, 256, 64, 256),        # a single problem through the grouped entry
])
def test_grouped_products_are_exact(backend, mods, groups, m, k, n):
    rng = np.random.default_rng(groups * 1000 + m + k + n)
    a = rng.integers(-128, 128, size=(groups, m, k)).astype(np.int8)
    b = rng.integers(-128, 128, size=(groups, n, k)).astype(np.int8)
    exact = grouped_exact(a, b)
    assert np.abs(exact).max() <= O.signed_capacity(mods)
    got = backend.matmul_grouped(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), mods)
    torch.cuda.synchronize()
    backend.check_status()
    assert got.shape == (groups, m, n)
    assert np.array_equal(got.cpu().numpy(), exact)
    if len(mods) == 4:
        got32 = backend.matmul_grouped(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), mods,
                                       out_dtype=torch.int32)
        assert np.array_equal(got32.cpu().numpy(), exact.astype(np.int32))


def test_attention_scores_and_values_of_all_heads(backend):
    """Q K^T and P V of a batch of heads as two grouped launches, each equal to the per-head
    integer products (what benchmarks/benchmark_attention.py:107-113 shapes one head of)."""
    rng = np.random.default_rng(12)
    batch, heads, tokens, head_dim = 2, 12, 256, 64
    g = batch * heads
    q = rng.integers(-127, 128, size=(g, tokens, head_dim)).astype(np.int8)
    k = rng.integers(-127, 128, size=(g, tokens, head_dim)).astype(np.int8)
    v = rng.integers(-127, 128, size=(g, tokens, head_dim)).astype(np.int8)
    scores = backend.matmul_grouped(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), C0)
    assert np.array_equal(scores.cpu().numpy(), grouped_exact(q, k))
    probs = torch.softmax(scores.float() / (127.0 * 127.0 * head_dim ** 0.5), dim=-1)
    p_q = torch.clamp(torch.round(probs * 127.0), 0, 127).to(torch.int8)             # [G, T, T]
    v_t = torch.from_numpy(np.ascontiguousarray(v.transpose(0, 2, 1))).cuda()          # V^T: [G, d, T]
    context = backend.matmul_grouped(p_q, v_t, C0)
    assert np.array_equal(context.cpu().numpy(),
                          np.einsum("gts,gsd->gtd", p_q.cpu().numpy().astype(np.int64), v.astype(np.int64)))
    backend.check_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_grouped_scaled_floating_outputs(backend, dtype):
    rng = np.random.default_rng(5)
    groups, m, k, n = 12, 256, 64, 264
    a = rng.integers(-127, 128, size=(groups, m, k)).astype(np.int8)
    b = rng.integers(-127, 128, size=(groups, n, k)).astype(np.int8)
    scale = np.float32(0.0123 * 0.0456 / 8.0)
    got = backend.matmul_grouped(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), C0, out_dtype=dtype,
                                 scale=float(scale))
    expect = (grouped_exact(a, b).astype(np.float32) * scale).astype(np.float32)
    expect = expect.astype(np.float16) if dtype == torch.float16 else expect
    assert np.array_equal(got.cpu().numpy(), expect)
    backend.check_status()


def test_grouped_arguments_are_checked(backend):
    a = torch.zeros((2, 128, 64), dtype=torch.int8, device="cuda")
    with pytest.raises(ValueError):
        backend.matmul_grouped(a, torch.zeros((2, 100, 64), dtype=torch.int8, device="cuda"), C0)   # N % 8
    with pytest.raises(ValueError):
        backend.matmul_grouped(a, torch.zeros((3, 128, 64), dtype=torch.int8, device="cuda"), C0)   # group counts
    with pytest.raises(ValueError):
        backend.matmul_grouped(a, torch.zeros((2, 128, 64), dtype=torch.int8, device="cuda"), (127, 126, 125))
    with pytest.raises(ValueError):
        backend.matmul_grouped(a.float(), torch.zeros((2, 128, 64), dtype=torch.int8, device="cuda"), C0)
    with pytest.raises(ValueError):      # a floating output needs its scale
        backend.matmul_grouped(a, torch.zeros((2, 128, 64), dtype=torch.int8, device="cuda"), C0,
                               out_dtype=torch.float16)
