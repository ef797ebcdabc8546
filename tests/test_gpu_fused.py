"""The fused tcgen05 path through the C ABI against the oracle: bit-exact
integers, bit-exact dequantised fp16 (the oracle follows the reference's fp32
operation order, so the 1e-3 relative tolerance of the specification is met
with zero error), quantiser, adaptive prefix, continuous batching, streams."""
import numpy as np
import pytest
import torch

from oracle import rns_oracle as O

pytestmark = pytest.mark.gpu

C0 = (127, 126, 125, 121)
C4 = (127, 126, 125, 121, 113)
REL_TOL = 1e-3  # north-star tolerance for dequantised outputs


@pytest.fixture(scope="module")
def backend():
    from rns_llm_b200.backends import CudaRNSBackend
    return CudaRNSBackend()


def dev(arr):
    return torch.from_numpy(np.ascontiguousarray(arr)).cuda()


def packed_act_offsets(m, k, channels):
    """Byte offsets of element (row, col, channel) in the packed activation layout
    (include/rns_b200.h): [M/128][K/64][channels][128][64] with 16-byte chunks of a
    row XORed by (row >> 1) & 3."""
    rows = np.arange(m)[:, None, None]
    cols = np.arange(k)[None, :, None]
    ch = np.arange(channels)[None, None, :]
    kblocks = (k + 63) // 64
    tile = ((rows >> 7) * kblocks + (cols >> 6)) * channels + ch
    r, c = rows & 127, cols & 63
    inner = r * 64 + ((((c >> 4) ^ ((r >> 1) & 3)) << 4) | (c & 15))
    return tile * 8192 + inner


def fused_int(backend, a, w_nk, mods, *, planes=False, packed=False, plain_weight=False, tile_n=0, tile_k=0,
              out_dtype=torch.int64, active=None, pair_mode=2, exact_residues=False, **tuning):
    """Direct call of rns_linear_fused on a [M,K] int8 and w [N,K] int8.
    planes: activations as centred planes; packed: activations in the packed tile
    layout; plain_weight: weight through the tensor map instead of the packed copy."""
    w_dev = dev(w_nk)
    prepared = backend.prepare_weight_nk(w_dev, mods)
    assert prepared.kernel == "tcgen05"
    m, k = a.shape
    out = torch.full((m, w_nk.shape[0]), -7, dtype=out_dtype, device="cuda")
    a_dev = dev(a)
    kwargs = dict(prepared=prepared, m=m, out=out, tile_n=tile_n, tile_k=tile_k, active=active,
                  plain_weight=w_dev if plain_weight else None, pair_mode=pair_mode,
                  exact_residues=exact_residues, **tuning)
    if planes and packed:
        from rns_llm_b200 import _native as N
        buf = torch.empty(int(N.load().rns_packed_activation_bytes(m, k, len(mods))), dtype=torch.int8, device="cuda")
        N.check(N.load().rns_encode_planes_packed(a_dev.data_ptr(), m, k, k, N.moduli_array(mods), len(mods),
                                                  buf.data_ptr(), torch.cuda.current_stream().cuda_stream))
        backend._launch_fused(a=None, a_planes=buf, a_packed=True, **kwargs)
    elif planes:
        backend._launch_fused(a=None, a_planes=backend.encode_centered(a_dev, mods), **kwargs)
    elif packed:
        host = np.zeros(((m + 255) // 256) * 256 * ((k + 63) // 64) * 64, dtype=np.int8)
        host[packed_act_offsets(m, k, 1)[:, :, 0]] = a
        backend._launch_fused(a=dev(host), a_planes=None, a_packed=True, **kwargs)
    else:
        backend._launch_fused(a=a_dev, a_planes=None, **kwargs)
    torch.cuda.synchronize()
    backend.check_status()
    return out.cpu().numpy()


# pair_mode=1: two CTAs per 256-row tile (tcgen05 cta_group::2); 0: one CTA per tile
MODES = [dict(pair_mode=0), dict(planes=True, pair_mode=0), dict(packed=True, pair_mode=0),
         dict(planes=True, packed=True, pair_mode=0), dict(plain_weight=True, pair_mode=0),
         dict(planes=True, plain_weight=True, pair_mode=0),
         dict(pair_mode=1), dict(planes=True, packed=True, pair_mode=1), dict(packed=True, pair_mode=1),
         dict(planes=True, plain_weight=True, pair_mode=1),
         dict(pair_mode=0, exact_residues=True), dict(packed=True, pair_mode=1, exact_residues=True)]


def rand_i8(rng, shape, lo=-127, hi=127):
    return rng.integers(lo, hi + 1, size=shape).astype(np.int8)


def test_config0_bit_exact(backend, golden):
    rng = np.random.default_rng(1000)
    a = rng.integers(-127, 128, size=(128, 768), dtype=np.int64).astype(np.int8)
    b = rng.integers(-127, 128, size=(768, 768), dtype=np.int64).astype(np.int8)
    exact = O.exact_matmul(a, b)
    g = golden("gemm")
    assert [int(exact.sum()), int(np.abs(exact).sum()), int(exact[0, 0]), int(exact[-1, -1])] == \
        [int(v) for v in g["c0_checksum"]]
    w = np.ascontiguousarray(b.T)
    for mode in MODES:
        assert np.array_equal(fused_int(backend, a, w, C0, **mode), exact), mode
    assert np.array_equal(fused_int(backend, a, w, C0, out_dtype=torch.int32), exact.astype(np.int32))
    # the backend entry point the reference exposes
    prepared = backend.prepare_weight(dev(b), C0)
    got = backend.matmul_prepared_fused(dev(a), prepared, lut_channels=2)
    assert got.dtype == torch.int64 and np.array_equal(got.cpu().numpy(), exact)


@pytest.mark.parametrize("m,k,n", [(1, 64, 16), (17, 64, 20), (5, 128, 33), (128, 768, 96),
                                   (129, 256, 130), (300, 1024, 260), (256, 4096, 256)])
@pytest.mark.parametrize("mode", range(len(MODES)))
def test_shapes_ragged_and_deep(backend, m, k, n, mode):
    rng = np.random.default_rng(m * 7 + k + n)
    a, w = rand_i8(rng, (m, k), -128, 127), rand_i8(rng, (n, k), -128, 127)
    assert np.array_equal(fused_int(backend, a, w, C0, **MODES[mode]), O.exact_matmul(a, w.T))


@pytest.mark.parametrize("mods", [(127, 125), (127, 126, 125), C0, C4])
def test_tensor_memory_operand_variant(backend, mods):
    """variant=2: the weight tile is the MMA's tensor-memory operand, encoded by the
    worker warps with tcgen05.st; activations are packed planes.  Odd and even numbers
    of K blocks, ragged M and N, every token-tile width the channel count allows."""
    rng = np.random.default_rng(len(mods) + 77)
    cap = O.signed_capacity(mods)
    for m, k, n in [(64, 64, 128), (100, 192, 200), (300, 1024, 260), (256, 320, 256), (513, 2048, 130)]:
        a, w = rand_i8(rng, (m, k), -128, 127), rand_i8(rng, (n, k), -128, 127)
        exact = O.exact_matmul(a, w.T)
        expect = exact if np.abs(exact).max() <= cap else \
            O.decode_garner(np.stack([exact % q for q in mods]), mods)
        widths = [0, 32] + ([64] if len(mods) <= 4 else []) + ([128] if len(mods) <= 2 else [])
        for tile_t in widths:
            got = fused_int(backend, a, w, mods, planes=True, packed=True, variant=2, tile_n=tile_t)
            assert np.array_equal(got, expect), (m, k, n, tile_t)
    with pytest.raises(Exception):   # plain (unpacked) activations are not a variant-2 input
        fused_int(backend, a, w, mods, variant=2)


@pytest.mark.parametrize("mods", [C0, C4])
def test_fixed_configuration_kernels(backend, mods):
    """Packed planes, every channel active, default knobs and the full-width tile select
    the instantiations with compile-time ring parameters (single-CTA tiles: weights read
    straight from global memory by the encoder threads; pair tiles for four channels).
    Ragged rows and columns, K from 8 blocks up."""
    rng = np.random.default_rng(len(mods) * 31)
    tile = 128 if len(mods) <= 4 else 96
    for m, k, n in [(300, 1024, 260), (129, 512, 130), (256, 4096, 200), (640, 576, 96),
                    (640, 528, 728), (520, 1040, 360), (200, 2064, 256)]:   # K ending in a part block
        a, w = rand_i8(rng, (m, k), -128, 127), rand_i8(rng, (n, k), -128, 127)
        exact = O.exact_matmul(a, w.T)
        for pair in ([0, 1] if len(mods) <= 4 else [0]):
            got = fused_int(backend, a, w, mods, planes=True, packed=True, pair_mode=pair, tile_n=tile)
            assert np.array_equal(got, exact), (m, k, n, pair)
        # packed int8 activations: both operands encoded from global memory, no bulk copies
        got = fused_int(backend, a, w, mods, packed=True, pair_mode=0, tile_n=tile)
        assert np.array_equal(got, exact), (m, k, n, "int8 activations")


@pytest.mark.parametrize("tuning", [dict(sub_blocks=1), dict(sub_blocks=2), dict(sub_blocks=4),
                                    dict(sub_blocks=2, enc_stages=2), dict(enc_groups=1, enc_stages=1),
                                    dict(enc_groups=2, enc_stages=3), dict(enc_groups=4, enc_stages=4),
                                    dict(enc_groups=4, enc_stages=2, sub_blocks=3)])
@pytest.mark.parametrize("mode", [0, 2, 3, 6, 7, 8])
def test_pipeline_tuning_knobs(backend, tuning, mode):
    """K blocks per stage, operand-ring depth and encoder groups only change the
    schedule: odd K-block counts (tail stages) and ragged edges stay bit-exact."""
    rng = np.random.default_rng(sum(tuning.values()) + mode)
    for m, k, n in [(130, 64 * 7, 72), (257, 64 * 18, 260)]:
        a, w = rand_i8(rng, (m, k), -128, 127), rand_i8(rng, (n, k), -128, 127)
        assert np.array_equal(fused_int(backend, a, w, C0, **MODES[mode], **tuning), O.exact_matmul(a, w.T)), (m, k, n)


@pytest.mark.parametrize("tile_n", [16, 32, 48, 64, 96, 128])
@pytest.mark.parametrize("tile_k", [64, 128])
def test_tile_shapes(backend, tile_n, tile_k):
    rng = np.random.default_rng(tile_n + tile_k)
    mods = (127, 125)  # two channels leave room for every tile shape
    a, w = rand_i8(rng, (140, 512)), rand_i8(rng, (200, 512))
    exact = O.exact_matmul(a, w.T)
    # two moduli hold +-7937: compare modulo P through the oracle's reconstruction
    expect = O.decode_garner(np.stack([exact % 127, exact % 125]), mods)
    # tile_k = 128 exists for plain (tensor-map) operands only
    assert np.array_equal(fused_int(backend, a, w, mods, tile_n=tile_n, tile_k=tile_k, plain_weight=True,
                                    pair_mode=0), expect)
    if tile_k == 64:
        for mode in MODES[:4] + (MODES[6:] if tile_n % 32 == 0 else []):
            assert np.array_equal(fused_int(backend, a, w, mods, tile_n=tile_n, **mode), expect), mode


@pytest.mark.parametrize("mods", [(127, 125), (127, 126, 125), C0, C4, (127, 126, 125, 121, 113, 109),
                                  (255, 253, 251, 247), (127, 125, 123, 121, 119, 113, 109, 107),
                                  (3, 5, 7, 11, 13, 17, 19, 23), (191, 193, 85, 64)])
def test_channel_counts(backend, mods):
    rng = np.random.default_rng(len(mods))
    k = 16384 if mods == C4 else 256
    a, w = rand_i8(rng, (40, k)), rand_i8(rng, (72, k))
    exact = O.exact_matmul(a, w.T)
    cap = O.signed_capacity(mods)
    if np.abs(exact).max() <= cap:
        expect = exact
    else:
        expect = O.decode_garner(np.stack([exact % m for m in mods]), mods)
    single_fold = min(mods) >= 86
    for mode in MODES:
        if mode.get("exact_residues") and not single_fold:
            continue
        assert np.array_equal(fused_int(backend, a, w, mods, **mode), expect), mode


def test_genuine_residues_reach_the_tensor_core(backend):
    """With the product of the moduli far below the true dot products the result
    must be the wrapped value of the residue arithmetic, not the plain integer
    product: evidence that every channel multiplies residues."""
    rng = np.random.default_rng(99)
    mods = (127, 113)
    a, w = rand_i8(rng, (64, 1024)), rand_i8(rng, (64, 1024))
    exact = O.exact_matmul(a, w.T)
    assert np.abs(exact).max() > O.signed_capacity(mods)
    expect = O.rns_matmul_device_pipeline(a, w.T, mods)
    got = fused_int(backend, a, w, mods)
    assert np.array_equal(got, expect) and not np.array_equal(got, exact)


@pytest.mark.parametrize("tag", ["qkv16", "odd"])
def test_linear_forward_matches_reference_golden(backend, golden, tag):
    g = golden("rns_linear")
    x = dev(g[f"{tag}_x"])
    weight = dev(g[f"{tag}_weight"])
    bias = dev(g[f"{tag}_bias"])
    w_q, w_scale, max_abs = backend.quantize_weight(weight)
    assert np.array_equal(w_q.cpu().numpy(), g[f"{tag}_w_q"])
    assert np.array_equal(w_scale.cpu().numpy(), g[f"{tag}_w_scale"])
    assert int(max_abs.item()) == int(np.abs(g[f"{tag}_w_q"].astype(np.int32)).max())
    prepared = backend.prepare_weight_nk(w_q, C0)
    flat = x.reshape(-1, x.shape[-1])
    y = backend.linear_forward(flat, prepared, w_scale, bias.float())
    torch.cuda.synchronize()
    backend.check_status()
    expect = g[f"{tag}_y"].reshape(y.shape)
    got = y.cpu().numpy()
    assert np.array_equal(got.view(np.uint16), expect.view(np.uint16))
    denom = np.maximum(np.abs(expect.astype(np.float32)), 1e-3)
    assert float(np.max(np.abs(got.astype(np.float32) - expect.astype(np.float32)) / denom)) <= REL_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("per_row", [False, True])
@pytest.mark.parametrize("m", [3, 700])
def test_linear_forward_dtypes_and_scales(backend, dtype, per_row, m):
    torch.manual_seed(5)
    k, n = 256, 136
    x = torch.randn(m, k).to(dtype)
    weight = (torch.randn(n, k) * 0.05).to(dtype)
    bias = torch.randn(n).to(dtype)
    np_dtype = {torch.float16: np.float16, torch.float32: np.float32}.get(dtype, np.float32)
    res = O.rns_linear_forward(x.float().numpy(), weight.float().numpy(), bias.float().numpy(), C0,
                               per_row=per_row, out_dtype=np_dtype)
    w_q, w_scale, _ = backend.quantize_weight(weight.cuda())
    assert np.array_equal(w_q.cpu().numpy(), res["w_q"])
    prepared = backend.prepare_weight_nk(w_q, C0)
    y = backend.linear_forward(x.cuda(), prepared, w_scale, bias.float().cuda(), per_row=per_row)
    torch.cuda.synchronize()
    backend.check_status()
    if dtype == torch.bfloat16:
        expect = torch.from_numpy(res["y"]).to(torch.bfloat16)
        assert torch.equal(y.cpu(), expect)
    else:
        assert np.array_equal(y.cpu().numpy(), res["y"])


def test_quantizer_outputs(backend):
    rng = np.random.default_rng(31)
    x = (rng.standard_normal((37, 192)) * 3).astype(np.float16)
    x[5, 7] = 0.0
    from rns_llm_b200 import _native as N
    lib = N.load()
    xd = dev(x)
    exp = {}
    for per_row in (0, 1):
        q = torch.empty((37, 192), dtype=torch.int8, device="cuda")
        planes = torch.empty((4, 37, 192), dtype=torch.int8, device="cuda")
        scale = torch.empty(37 if per_row else 1, dtype=torch.float32, device="cuda")
        l1 = torch.empty(1, dtype=torch.int32, device="cuda")
        scratch = torch.empty(4, dtype=torch.int32, device="cuda")
        N.check(lib.rns_quantize_activations(xd.data_ptr(), N.F16, 37, 192, 192, 0, 0, per_row, 127,
                                             N.moduli_array(C0), 4, q.data_ptr(), planes.data_ptr(), 0,
                                             scale.data_ptr(), l1.data_ptr(), scratch.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        exp_scale = O.symmetric_scale(x.astype(np.float32), 127, axis=1 if per_row else None)
        exp_q = O.quantize(x.astype(np.float32), exp_scale, 127)
        assert np.array_equal(scale.cpu().numpy(), exp_scale.reshape(-1))
        assert np.array_equal(q.cpu().numpy(), exp_q)
        assert np.array_equal(planes.cpu().numpy(), O.encode_centered(exp_q, C0, "device"))
        assert int(l1.item()) == int(np.abs(exp_q.astype(np.int64)).sum(axis=1).max())
        exp[per_row] = exp_q
    # packed tile layouts, and the two-launch per-tensor path (M*K > 128 Ki elements)
    big = (rng.standard_normal((300, 512)) * 2).astype(np.float16)
    for values, per_row in ((x, 0), (big, 0), (big, 1)):
        m, k = values.shape
        vd = dev(values)
        qp = torch.zeros(int(lib.rns_packed_activation_bytes(m, k, 1)), dtype=torch.int8, device="cuda")
        pp = torch.zeros(int(lib.rns_packed_activation_bytes(m, k, 4)), dtype=torch.int8, device="cuda")
        scale = torch.empty(m if per_row else 1, dtype=torch.float32, device="cuda")
        scratch = torch.empty(4, dtype=torch.int32, device="cuda")
        N.check(lib.rns_quantize_activations(vd.data_ptr(), N.F16, m, k, k, 0, 0, per_row, 127,
                                             N.moduli_array(C0), 4, qp.data_ptr(), pp.data_ptr(), 1,
                                             scale.data_ptr(), None, scratch.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        exp_scale = O.symmetric_scale(values.astype(np.float32), 127, axis=1 if per_row else None)
        exp_q = O.quantize(values.astype(np.float32), exp_scale, 127)
        assert np.array_equal(scale.cpu().numpy(), exp_scale.reshape(-1))
        assert np.array_equal(qp.cpu().numpy()[packed_act_offsets(m, k, 1)[:, :, 0]], exp_q)
        got_planes = pp.cpu().numpy()[packed_act_offsets(m, k, 4)]            # [M,K,4]
        # packed planes only feed the tensor cores: one-step reduced residues (x - m for
        # x >= 64, x + m for x < -64), the same encoder as the in-kernel one
        reduced = np.empty((4, m * k), dtype=np.int8)
        flat = np.ascontiguousarray(exp_q.reshape(-1))
        N.check(lib.rns_host_encode_reduced_i8(flat.ctypes.data, flat.size, N.moduli_array(C0), 4, reduced.ctypes.data))
        assert np.array_equal(got_planes.transpose(2, 0, 1), reduced.reshape(4, m, k))
        for c, mod in enumerate(C0):
            assert np.all((reduced[c].astype(int) - flat.astype(int)) % mod == 0)
    zeros = torch.zeros((4, 64), dtype=torch.float16, device="cuda")
    wq, ws, _ = backend.quantize_weight(zeros)
    assert float(ws[0]) == float(np.finfo(np.float32).eps) and int(wq.abs().max()) == 0


@pytest.mark.parametrize("m", [5, 200, 1100])
@pytest.mark.parametrize("per_row", [False, True])
def test_linear_forward_reads_gathered_column_blocks(backend, m, per_row):
    """A [G, M, K/G] activation (what an all-gather of G column shards leaves) gives the
    same bits as the plain [M, K] matrix it stands for: single-CTA quantiser, the
    two-launch one, and the residue-plane path of many-token calls."""
    torch.manual_seed(m)
    g, k, n = 4, 1024, 264
    blocks = torch.randn(g, m, k // g, dtype=torch.float16, device="cuda")
    plain = blocks.permute(1, 0, 2).reshape(m, k).contiguous()
    weight = (torch.randn(n, k, device="cuda") * 0.05).half()
    w_q, w_scale, _ = backend.quantize_weight(weight)
    prepared = backend.prepare_weight_nk(w_q, C0)
    y_plain = backend.linear_forward(plain, prepared, w_scale, None, per_row=per_row).clone()
    y_blocks = backend.linear_forward(blocks, prepared, w_scale, None, per_row=per_row)
    torch.cuda.synchronize()
    backend.check_status()
    assert torch.equal(y_plain, y_blocks)
    expect = O.rns_linear_forward(plain.cpu().numpy(), weight.cpu().numpy(), None, C0, per_row=per_row)["y"]
    assert np.array_equal(y_blocks.cpu().numpy().view(np.uint16), expect.view(np.uint16))


def test_quantizer_ties_and_near_ties(backend):
    """Values whose quotient by the scale sits on or within a few ulp of a half-integer:
    the reciprocal-product shortcut may not be trusted there and the division is redone.
    float32 input, so that the near-ties are as near as float32 allows."""
    from rns_llm_b200 import _native as N
    lib = N.load()
    rng = np.random.default_rng(77)
    m, k = 320, 512
    for absmax in (127.0, 100.0, 3.3, 1e-3):
        scale = np.float32(absmax) / np.float32(127)
        halves = rng.integers(-127, 127, size=(m, k)).astype(np.float32) + np.float32(0.5)
        x = (halves * scale).astype(np.float32)
        nudge = rng.integers(-3, 4, size=(m, k))
        for _ in range(3):   # up to three ulp either side, a third of the values untouched
            step = np.sign(nudge).astype(np.float32)
            x = np.where(nudge != 0, np.nextafter(x, x + step).astype(np.float32), x)
            nudge = nudge - np.sign(nudge)
        x[0, 0] = absmax; x[1, 1] = -absmax
        xd = torch.from_numpy(x).cuda()
        for per_row in (0, 1):
            q = torch.empty((m, k), dtype=torch.int8, device="cuda")
            scale_out = torch.empty(m if per_row else 1, dtype=torch.float32, device="cuda")
            scratch = torch.empty(4, dtype=torch.int32, device="cuda")
            N.check(lib.rns_quantize_activations(xd.data_ptr(), N.F32, m, k, k, 0, 0, per_row, 127,
                                                 N.moduli_array(C0), 4, q.data_ptr(), None, 0,
                                                 scale_out.data_ptr(), None, scratch.data_ptr(),
                                                 torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            exp_scale = O.symmetric_scale(x, 127, axis=1 if per_row else None)
            assert np.array_equal(scale_out.cpu().numpy(), exp_scale.reshape(-1))
            assert np.array_equal(q.cpu().numpy(), O.quantize(x, exp_scale, 127)), (absmax, per_row)


def test_adaptive_prefix_selected_on_device(backend):
    rng = np.random.default_rng(1002)
    a_low = rand_i8(rng, (128, 768), -15, 15)
    a_full = rand_i8(rng, (128, 768))
    w_kn = rand_i8(rng, (768, 768))
    adaptive = backend.prepare_weight_adaptive(dev(w_kn), C0, min_channels=3)
    assert adaptive.max_abs_weight == 127 and sorted(adaptive.variants) == [3, 4]
    backend.reset_stats()
    out_low, meta_low = backend.matmul_prepared_adaptive_fused(dev(a_low), adaptive, return_metadata=True)
    out_full, meta_full = backend.matmul_prepared_adaptive_fused(dev(a_full), adaptive, return_metadata=True)
    assert np.array_equal(out_low.cpu().numpy(), O.exact_matmul(a_low, w_kn))
    assert np.array_equal(out_full.cpu().numpy(), O.exact_matmul(a_full, w_kn))
    exp_low = O.adaptive_channels(a_low, w_kn.T, C0, 3)
    exp_full = O.adaptive_channels(a_full, w_kn.T, C0, 3)
    assert (meta_low["channels"], meta_low["bound"]) == exp_low and exp_low[0] == 3
    assert (meta_full["channels"], meta_full["bound"]) == exp_full and exp_full[0] == 4
    assert meta_low["bound"] <= meta_low["capacity"] == O.signed_capacity(C0[:3])
    stats = backend.stats_snapshot()
    assert stats["adaptive_selections"] == 2
    assert stats["adaptive_channels_3"] == 1 and stats["adaptive_channels_4"] == 1
    backend.check_status()
    # host-synchronising selection kept with the reference's signature
    variant, bound = backend.select_adaptive_variant(dev(a_low), adaptive)
    assert len(variant.moduli) == 3 and bound == exp_low[1]


def test_adaptive_runs_under_graph_capture(backend):
    """No host synchronisation on the adaptive path: it can be captured."""
    rng = np.random.default_rng(41)
    a_low = dev(rand_i8(rng, (16, 256), -8, 8))
    w_kn = rand_i8(rng, (256, 64), -40, 40)
    adaptive = backend.prepare_weight_adaptive(dev(w_kn), C0, min_channels=3)
    ws = {4: backend.create_workspace(device=a_low.device, channels=4, m=16, n=64)}
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        backend.matmul_prepared_adaptive_fused(a_low, adaptive, workspace_by_channels=ws)  # warm the arena
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = backend.matmul_prepared_adaptive_fused(a_low, adaptive, workspace_by_channels=ws)
        out.zero_()
        graph.replay()
        stream.synchronize()
    assert np.array_equal(out.cpu().numpy(), O.exact_matmul(a_low.cpu().numpy(), w_kn))


def test_adaptive_overflow_sets_status(backend):
    rng = np.random.default_rng(43)
    mods = (127, 113)
    a = dev(rand_i8(rng, (8, 1024)))
    w_kn = dev(rand_i8(rng, (1024, 32)))
    adaptive = backend.prepare_weight_adaptive(w_kn, mods, min_channels=2)
    backend.matmul_prepared_adaptive_fused(a, adaptive)
    with pytest.raises(OverflowError):
        backend.check_status()
    backend.check_status()  # cleared


def test_continuous_batch_matches_independent_requests(backend):
    rng = np.random.default_rng(1002)
    weight_kn = rand_i8(rng, (768, 768))
    prepared = backend.prepare_weight(dev(weight_kn), C0)
    for rows in ((1,), (1, 1), (1, 1, 1, 1), (1, 3, 5, 2)):
        requests = [rand_i8(rng, (r, 768)) for r in rows]
        ws = backend.create_request_batch_workspace(device=torch.device("cuda"), dtype=torch.int8,
                                                    rows_per_request=rows, k=768, channels=4, n=768)
        backend.reset_stats()
        merged = backend.matmul_prepared_fused_requests([dev(r) for r in requests], prepared,
                                                        workspace=ws, clone_outputs=True)
        for request, actual in zip(requests, merged):
            independent = backend.matmul_prepared_fused(dev(request), prepared)
            assert torch.equal(actual, independent)
            assert np.array_equal(actual.cpu().numpy(), O.exact_matmul(request, weight_kn))
        stats = backend.stats_snapshot()
        assert stats["continuous_batch_calls"] == 1 and stats["continuous_batch_requests"] == len(rows)
    with pytest.raises(ValueError):
        backend.matmul_prepared_fused_requests([], prepared)
    with pytest.raises(ValueError):
        backend.create_request_batch_workspace(device=torch.device("cuda"), dtype=torch.int8,
                                               rows_per_request=[1, 0], k=768, channels=4, n=768)


def test_streams_have_private_scratch(backend):
    rng = np.random.default_rng(51)
    weight = (torch.randn(96, 512) * 0.03).half().cuda()
    w_q, w_scale, _ = backend.quantize_weight(weight)
    prepared = backend.prepare_weight_nk(w_q, C0)
    streams = [torch.cuda.Stream() for _ in range(4)]
    xs = [torch.randn(24 + 8 * i, 512).half().cuda() for i in range(4)]
    torch.cuda.synchronize()
    outs = [None] * 4
    for _ in range(5):
        for i, s in enumerate(streams):
            with torch.cuda.stream(s):
                outs[i] = backend.linear_forward(xs[i], prepared, w_scale, None)
    torch.cuda.synchronize()
    backend.check_status()
    for i in range(4):
        expect = O.rns_linear_forward(xs[i].cpu().numpy(), weight.cpu().numpy(), None, C0)["y"]
        assert np.array_equal(outs[i].cpu().numpy(), expect)
    assert len(backend.arena.streams()) >= 4


def test_fused_argument_errors(backend):
    from rns_llm_b200 import _native as N
    a = torch.zeros((8, 64), dtype=torch.int8, device="cuda")
    w = torch.zeros((16, 64), dtype=torch.int8, device="cuda")
    prepared = backend.prepare_weight_nk(w, C0)
    out = torch.zeros((8, 16), dtype=torch.int64, device="cuda")
    with pytest.raises(ValueError):
        backend._launch_fused(prepared=prepared, m=8, a=a, a_planes=None, out=out, tile_n=24)
    with pytest.raises(ValueError):
        backend._launch_fused(prepared=prepared, m=8, a=a, a_planes=None, out=out, tile_k=32)
    with pytest.raises(ValueError):
        backend.matmul_prepared_fused(a[:, :48].contiguous(), prepared)
    with pytest.raises(ValueError):
        backend.matmul_prepared_fused(a, prepared, lut_channels=3)
    # K not a multiple of 16 or small moduli: served by the plane-level pipeline, still exact
    rng = np.random.default_rng(61)
    a2, b2 = rand_i8(rng, (9, 20)), rand_i8(rng, (20, 12))
    prepared2 = backend.prepare_weight(dev(b2), C0)
    assert prepared2.kernel == "cublas"
    assert np.array_equal(backend.matmul_prepared_fused(dev(a2), prepared2).cpu().numpy(), O.exact_matmul(a2, b2))
    # more than eight channels: plane-level pipeline as well
    many = (3, 5, 7, 11, 13, 17, 19, 23, 29)
    a3, b3 = rand_i8(rng, (6, 64)), rand_i8(rng, (64, 8))
    prepared3 = backend.prepare_weight(dev(b3), many)
    assert prepared3.kernel != "tcgen05"
    assert np.array_equal(backend.matmul_prepared_fused(dev(a3), prepared3).cpu().numpy(), O.exact_matmul(a3, b3))
    # exactly centred in-kernel residues need every modulus >= 86
    small = backend.prepare_weight_nk(dev(np.ascontiguousarray(b3.T)), (3, 5, 7, 11, 13, 17, 19, 23))
    with pytest.raises(ValueError):
        backend._launch_fused(prepared=small, m=6, a=dev(a3), a_planes=None,
                              out=torch.zeros((6, 8), dtype=torch.int64, device="cuda"), exact_residues=True)
    assert N.load().rns_linear_fused(None, None) == N.ERR_INVALID_ARGUMENT


def test_full_size_against_independent_int_gemm(backend, c_oracle):
    """Configuration-4 layer shapes: too large for the CPU oracle in full, so the
    whole output is compared with torch._int_mm (cuBLAS int8 -> int32, an
    independent exact GEMM) and a sample of rows with the C oracle."""
    torch.manual_seed(1004)
    for (m, k, n, mods) in ((4096, 4096, 4096, C0), (1024, 16384, 1024, C4)):
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda")
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda")
        prepared = backend.prepare_weight_nk(w, mods)
        got = backend.matmul_prepared_fused(a, prepared)
        expect = torch._int_mm(a, w.t())
        assert torch.equal(got, expect.to(torch.int64))
        rows = [0, 1, m // 2, m - 1]
        sample, _ = c_oracle.linear(a[rows].cpu().numpy(), w.cpu().numpy(), mods)
        assert np.array_equal(got[rows].cpu().numpy(), sample)
        # linearity: (a + a2) W = a W + a2 W for operands that stay inside int8
        a_half = torch.div(a, 2, rounding_mode="trunc").to(torch.int8)
        rest = (a - a_half).to(torch.int8)
        both = backend.matmul_prepared_fused(a_half, prepared).clone() + \
            backend.matmul_prepared_fused(rest, prepared)
        assert torch.equal(both, got)
    backend.check_status()


def test_weight_pack_roundtrip_and_residues(backend):
    rng = np.random.default_rng(71)
    for n, k in ((20, 64), (384, 128), (500, 208)):
        w = rand_i8(rng, (n, k), -128, 127)
        prepared = backend.prepare_weight_nk(dev(w), C0)
        from rns_llm_b200 import _native as N
        assert prepared.weight_packed.numel() == N.load().rns_packed_weight_bytes(n, k) == \
            ((n + 383) // 384) * 384 * ((k + 63) // 64) * 64
        assert np.array_equal(prepared.weight_nk.cpu().numpy(), w)
        # planes are derived on request, in the reference's [R,K,N] shape
        assert np.array_equal(prepared.residues.cpu().numpy(), O.encode_centered(w.T, C0, "device"))


def _torch_linear_reference(x_plain, w_q, w_scale, bias):
    """Per-tensor quantisation, exact int8 GEMM through torch._int_mm and the reference's
    fp32 dequantisation order (layers/rns_linear.py:239-241, 264, 272-275), all on the GPU."""
    flat = x_plain.float()
    amax = flat.abs().amax()
    s_a = torch.clamp(amax / torch.full_like(amax, 127.0), min=float(np.finfo(np.float32).eps))
    a_q = torch.clamp(torch.round(flat / s_a), -127, 127).to(torch.int8)
    acc = torch._int_mm(a_q, w_q.t())
    y = acc.float() * s_a * w_scale[None, :]
    if bias is not None:
        y = y + bias[None, :]
    return y.to(x_plain.dtype), acc


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("name,k,n,mods,groups", [("qkv", 4096, 12288, C0, 3), ("out_proj", 4096, 4096, C0, 1),
                                                  ("fc1", 4096, 16384, C0, 1), ("fc2", 16384, 4096, C4, 1)])
def test_rank_local_problems_of_a_sharded_stack(backend, world, name, k, n, mods, groups):
    """What one rank of a 4- or 8-way column-sharded OPT-6.7B-shaped layer runs, on one GPU:
    M = 4096 tokens, N / world output features, the activation read from a gathered
    [G, M, K/G] tensor (for out_proj: a column-group view of a wider gathered tensor, as the
    q block of a fused QKV output), the result written into slot `rank` of a [G, M, N/G]
    buffer, for the first and the last rank.  Checked bit for bit against the same call on
    the plain [M, K] matrix into a fresh tensor, and that against torch._int_mm + fp32
    dequantisation (exact integers; 1e-3 relative on the fp16 outputs)."""
    from rns_llm_b200.parallel import group_view, shard_tensor

    m = 4096
    torch.manual_seed(world * 100 + k // 1024 + n // 1024)
    if name == "out_proj":
        wide = torch.randn(world, m, 3 * k // world, dtype=torch.float16, device="cuda")
        blocks = group_view(wide, 3, 0)                          # strided view, [G, M, K/G]
    else:
        blocks = torch.randn(world, m, k // world, dtype=torch.float16, device="cuda")
    plain = blocks.permute(1, 0, 2).reshape(m, k).contiguous()
    full_w = (torch.randn(n, k, device="cuda") * (1.0 / k ** 0.5)).half()
    full_b = (torch.randn(n, device="cuda") * 0.01).float()
    for rank in (0, world - 1):
        weight = shard_tensor(full_w, world, rank, groups).contiguous()
        bias = shard_tensor(full_b, world, rank, groups).contiguous()
        w_q, w_scale, _ = backend.quantize_weight(weight)
        prepared = backend.prepare_weight_nk(w_q, mods)
        local_n = n // world
        gathered = torch.full((world, m, local_n), float("nan"), dtype=torch.float16, device="cuda")
        backend.linear_forward(blocks, prepared, w_scale, bias, out=gathered[rank])
        fresh = backend.linear_forward(plain, prepared, w_scale, bias)
        torch.cuda.synchronize()
        backend.check_status()
        assert torch.equal(gathered[rank], fresh), (name, world, rank)
        others = [r for r in range(world) if r != rank]
        assert bool(torch.isnan(gathered[others]).all())          # nothing written outside the slot
        expect, _ = _torch_linear_reference(plain, w_q, w_scale, bias)
        diff = (fresh.float() - expect.float()).abs()
        assert float((diff / expect.float().abs().clamp_min(1e-3)).max()) <= REL_TOL
        # the integer path on the same shard, bit-exact against the independent int8 GEMM
        a_q = torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda")
        got = backend.matmul_prepared_fused(a_q, prepared)
        assert torch.equal(got, torch._int_mm(a_q, w_q.t()).to(torch.int64)), (name, world, rank)
    backend.check_status()


@pytest.mark.parametrize("k", [16, 80, 144])
def test_k_tails_inside_the_last_64_byte_block(backend, k):
    """K is a multiple of 16 but not of 64: the packed layouts pad the last K block, the
    quantiser does not write the pad columns of the activation side, and the result must
    not depend on what an earlier, larger call left in the same scratch."""
    from rns_llm_b200 import _native as N

    rng = np.random.default_rng(k)
    for m in (7, 130):
        a, w = rand_i8(rng, (m, k), -128, 127), rand_i8(rng, (40, k), -128, 127)
        exact = O.exact_matmul(a, w.T)
        for mode in MODES:
            assert np.array_equal(fused_int(backend, a, w, C0, **mode), exact), (m, mode)
    torch.manual_seed(k)
    n = 72
    weight = (torch.randn(n, k, device="cuda") * 0.1).half()
    bias = torch.randn(n, device="cuda").float()
    w_q, w_scale, _ = backend.quantize_weight(weight)
    prepared = backend.prepare_weight_nk(w_q, C0)
    lib = N.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for m in (9, 600):                       # in-kernel residues, and residue planes
        # dirty the arena and the static array with a larger problem first
        big = torch.randn(1024, 256, dtype=torch.float16, device="cuda") * 50
        big_w, big_s, _ = backend.quantize_weight((torch.randn(64, 256, device="cuda")).half())
        big_p = backend.prepare_weight_nk(big_w, C0)
        backend.linear_forward(big, big_p, big_s, None)
        sink = torch.empty((1024, 64), dtype=torch.float16, device="cuda")
        N.check(lib.rns_linear_static(big.data_ptr(), N.F16, 1024, 256, 256, big_p.weight_packed.data_ptr(), 64,
                                      N.moduli_array(C0), 4, big_s.data_ptr(), None, sink.data_ptr(), 64,
                                      N.OUT_F16, status.data_ptr(), stream))
        x = torch.randn(m, k, dtype=torch.float16, device="cuda")
        expect = O.rns_linear_forward(x.cpu().numpy(), weight.cpu().numpy(), bias.cpu().numpy(), C0)["y"]
        y = backend.linear_forward(x, prepared, w_scale, bias)
        assert np.array_equal(y.cpu().numpy().view(np.uint16), expect.view(np.uint16)), m
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        N.check(lib.rns_linear_static(x.data_ptr(), N.F16, m, k, k, prepared.weight_packed.data_ptr(), n,
                                      N.moduli_array(C0), 4, w_scale.data_ptr(), bias.data_ptr(), got.data_ptr(), n,
                                      N.OUT_F16, status.data_ptr(), stream))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert np.array_equal(got.cpu().numpy().view(np.uint16), expect.view(np.uint16)), m
    backend.check_status()


def test_channel_sum_overflow_is_refused(backend):
    """K beyond 131071 could wrap an int32 channel sum: the C ABI refuses it."""
    from rns_llm_b200 import _native as N
    args = N.LinearArgs()
    args.m, args.n, args.k, args.channels = 16, 16, 131072, 4
    for i, mod in enumerate(C0):
        args.moduli[i] = mod
    dummy = torch.zeros(64, dtype=torch.int8, device="cuda")
    args.d_a = dummy.data_ptr(); args.d_w = dummy.data_ptr(); args.d_out = dummy.data_ptr()
    args.lda = args.ldw = 131072; args.ldo = 16; args.out_type = N.OUT_INT64
    assert N.load().rns_linear_fused(args, None) == N.ERR_OVERFLOW
