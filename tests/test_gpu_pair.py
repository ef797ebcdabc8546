"""The two-CTA feature-major kernel (rns_linear_args.variant 3) through the C ABI:
exact integers against the int64 oracle on ragged shapes, the dequantised outputs of
linear_forward against the oracle's fp32 operation order, and the absmax word that lets
a layer stack skip the quantiser's own pass over the activations."""
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


def tiled_plane_offsets(m, k, channels, tile_rows):
    """Byte offset of (row, col, channel) in [M_pad/rows][K_pad/64][channels][rows][64]
    with 16-byte chunks of a row XORed by (row_in_tile >> 1) & 3 (include/rns_b200.h)."""
    rows = np.arange(m)[:, None, None]
    cols = np.arange(k)[None, :, None]
    ch = np.arange(channels)[None, None, :]
    kblocks = (k + 63) // 64
    tile = ((rows // tile_rows) * kblocks + (cols >> 6)) * channels + ch
    r, c = rows % tile_rows, cols & 63
    inner = r * 64 + ((((c >> 4) ^ ((r >> 1) & 3)) << 4) | (c & 15))
    return tile * (tile_rows * 64) + inner


def pair_int(backend, a, w_nk, mods, out_dtype=torch.int64, variant=0, active=None):
    from rns_llm_b200 import _native as N
    lib = N.load()
    m, k = a.shape
    rows = int(lib.rns_pair_tile_rows(len(mods), k))
    assert rows in (64, 48)
    nbytes = int(lib.rns_packed_planes_bytes(m, k, len(mods), rows))
    assert nbytes == -(-m // (2 * rows)) * 2 * rows * -(-k // 64) * 64 * len(mods)
    host = np.full(nbytes, 77, dtype=np.int8)                   # pad rows / columns hold junk
    planes = O.encode_centered(a, mods, "device")               # [R, M, K]
    if active is not None:
        planes[active:] = 99                                     # channels beyond the prefix: never read
    host[tiled_plane_offsets(m, k, len(mods), rows)] = np.moveaxis(planes, 0, 2)
    w_dev = torch.from_numpy(np.ascontiguousarray(w_nk)).cuda()
    prepared = backend.prepare_weight_nk(w_dev, mods)
    out = torch.full((m, w_nk.shape[0]), -7, dtype=out_dtype, device="cuda")
    backend._launch_fused(prepared=prepared, m=m, a=None, a_planes=torch.from_numpy(host).cuda(), a_packed=True,
                          out=out, a_tile_rows=rows, variant=variant,
                          active=None if active is None else torch.tensor([active], dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    backend.check_status()
    return out.cpu().numpy()


@pytest.mark.parametrize("variant", [0, 3, 4])   # 0 resolves to 4 (int8 weights as every channel's operand); 3 encodes
@pytest.mark.parametrize("mods", [C0, C4])
@pytest.mark.parametrize("m,k,n", [(128, 512, 256), (300, 1024, 260), (97, 528, 130), (700, 2048, 700),
                                   (1024, 4096, 512), (260, 576, 1000), (1300, 576, 2000)])
def test_pair_kernel_exact_integers(backend, mods, m, k, n, variant):
    rng = np.random.default_rng(m + k + n + len(mods))
    a = rng.integers(-128, 128, size=(m, k)).astype(np.int8)
    w = rng.integers(-128, 128, size=(n, k)).astype(np.int8)
    exact = O.exact_matmul(a, w.T)
    assert np.array_equal(pair_int(backend, a, w, mods, variant=variant), exact)
    if len(mods) == 4:
        assert np.array_equal(pair_int(backend, a, w, mods, torch.int32, variant=variant), exact.astype(np.int32))


@pytest.mark.parametrize("mods", [C0, C4])
@pytest.mark.parametrize("m,k,n", [(300, 512, 260), (1300, 576, 2000)])
def test_pair_kernel_channel_prefix(backend, mods, m, k, n):
    """d_active_channels: only the leading channels are loaded, multiplied and reconstructed.
    Operand ranges are chosen so that the products fit the prefix's capacity; the planes of
    the unused channels hold junk, to show that nothing reads them."""
    rng = np.random.default_rng(m + k + len(mods))
    for active in range(2, len(mods) + 1):
        capacity = (int(np.prod([int(v) for v in mods[:active]], dtype=object)) - 1) // 2
        a_max = 1 if active == 2 else (15 if active == 3 else 127)
        w_max = min(127, capacity // (k * a_max))
        assert w_max >= 1
        a = rng.integers(-a_max, a_max + 1, size=(m, k)).astype(np.int8)
        w = rng.integers(-w_max, w_max + 1, size=(n, k)).astype(np.int8)
        exact = O.exact_matmul(a, w.T)
        assert np.abs(exact).max() <= capacity
        assert np.array_equal(pair_int(backend, a, w, mods, active=active), exact), active


@pytest.mark.parametrize("mods,k", [(C0, 4096), (C4, 16384)])
def test_pair_kernel_extreme_magnitudes(backend, mods, k):
    """Every product at its largest magnitude and one sign: the channel sums of the kernel that
    feeds raw int8 weights reach K * 64 * 128 (K * 128 * 128 could not occur: the activation
    side is always a reduced residue), far inside int32; the integers stay exact."""
    m, n = 256, 256
    for a_val, w_val in ((-128, -128), (127, -128), (64, -128), (-65, 127), (63, 127)):
        a = np.full((m, k), a_val, dtype=np.int8)
        w = np.full((n, k), w_val, dtype=np.int8)
        a[::7, ::5] = -a_val if a_val != -128 else 127           # a few sign changes so that rows differ
        exact = O.exact_matmul(a, w.T)
        if np.abs(exact).max() > (int(np.prod([int(v) for v in mods], dtype=object)) - 1) // 2:
            continue                                             # beyond the moduli set's capacity
        assert np.array_equal(pair_int(backend, a, w, mods), exact)


@pytest.mark.parametrize("mods", [C0, C4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("per_row", [False, True])
def test_pair_kernel_linear_forward_matches_oracle(backend, mods, dtype, per_row):
    torch.manual_seed(11 + len(mods))
    m, k, n = 600, 1024, 392
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


def test_absmax_word_feeds_the_next_quantiser(backend):
    """The epilogue's max |y| equals the tensor's absmax as the next layer computes it, and
    a quantiser given that word (alone, or as the maximum of several words) produces the
    same bits as one that scans the activations itself."""
    torch.manual_seed(5)
    m, k, n = 1024, 1024, 768
    x = torch.randn(m, k, dtype=torch.float16, device="cuda")
    w1 = (torch.randn(n, k, device="cuda") * 0.05).half()
    w2 = (torch.randn(512, n, device="cuda") * 0.05).half()
    q1, s1, _ = backend.quantize_weight(w1)
    q2, s2, _ = backend.quantize_weight(w2)
    p1, p2 = backend.prepare_weight_nk(q1, C0), backend.prepare_weight_nk(q2, C0)
    words = torch.zeros(8, dtype=torch.int32, device="cuda")
    y1 = backend.linear_forward(x, p1, s1, None, absmax_out=words.data_ptr())
    torch.cuda.synchronize()
    got = words[:1].view(torch.float32).item()
    assert got == float(y1.float().abs().max())
    plain = backend.linear_forward(y1, p2, s2, None).clone()
    given = backend.linear_forward(y1, p2, s2, None, absmax_in=(words.data_ptr(), 1, 0)).clone()
    assert torch.equal(plain, given)
    # several parts: the maximum counts (smaller words elsewhere must not matter)
    words[2] = torch.tensor([0.25], dtype=torch.float32).view(torch.int32).item()
    words[4] = 0
    spread = backend.linear_forward(y1, p2, s2, None, absmax_in=(words.data_ptr(), 3, 2))
    assert torch.equal(plain, spread)
    backend.check_status()
    with pytest.raises(ValueError):
        backend.linear_forward(x[:64], p1, s1, None, absmax_out=words.data_ptr())


def test_sharded_layers_pass_the_absmax_on(backend):
    """A chain of column-sharded layers (one rank, so no process group is needed) gives the
    same bits whether the second layer scans its input for the absmax or takes the word the
    first layer's epilogue left behind; a column-group view does not carry the word."""
    from rns_llm_b200.parallel import ColumnShardedRNSLinear, GatheredActivation, group_view

    torch.manual_seed(21)
    m, k = 1024, 1024
    x = torch.randn(m, k, dtype=torch.float16, device="cuda")
    w1 = (torch.randn(1536, k, device="cuda") * 0.04).half()
    w2 = (torch.randn(768, 1536, device="cuda") * 0.04).half()
    w3 = (torch.randn(640, 512, device="cuda") * 0.04).half()
    l1 = ColumnShardedRNSLinear(w1, None, backend=backend, moduli=C0, rank=0, world=1, groups=3)
    l2 = ColumnShardedRNSLinear(w2, None, backend=backend, moduli=C0, rank=0, world=1)
    l3 = ColumnShardedRNSLinear(w3, None, backend=backend, moduli=C0, rank=0, world=1)
    y1 = l1(x)
    assert isinstance(y1, GatheredActivation) and y1.absmax_words is not None and y1.absmax_words[1] == 1
    y2 = l2(y1)                                   # takes the word
    y2_plain = l2(y1.as_subclass(torch.Tensor))   # scans the activations itself
    torch.cuda.synchronize()
    assert torch.equal(y2.as_subclass(torch.Tensor), y2_plain.as_subclass(torch.Tensor))
    q = group_view(y1, 3, 0)
    assert not isinstance(q, GatheredActivation)
    y3 = l3(q)
    expect = O.rns_linear_forward(q.permute(1, 0, 2).reshape(m, 512).cpu().numpy(), w3.cpu().numpy(), None, C0)["y"]
    assert np.array_equal(y3[0].cpu().numpy().view(np.uint16), expect.view(np.uint16))
    expect2 = O.rns_linear_forward(y1[0].cpu().numpy(), w2.cpu().numpy(), None, C0)["y"]
    assert np.array_equal(y2[0].cpu().numpy().view(np.uint16), expect2.view(np.uint16))
    backend.check_status()


@pytest.mark.parametrize("m,k,n,mods", [(640, 1024, 520, C0), (600, 1024, 384, C4), (645, 512, 260, C0),
                                        (1027, 768, 1024, C0)])
def test_output_copies_and_absmax_hand_over(backend, m, k, n, mods):
    """The epilogue's fan-out, on one GPU: buffers of this process stand in for the other
    ranks' memory.  Every copy receives exactly what `out` receives, and the finished
    absmax word (written by the last CTA to contribute) equals max |y|.  The shapes take
    the row-wide staged stores (full 128-feature blocks, row stride a multiple of 8), the
    lane-pair stores (ragged last block; stride 260) and ragged token tiles."""
    torch.manual_seed(31)
    x = torch.randn(m, k, dtype=torch.float16, device="cuda")
    weight = (torch.randn(n, k, device="cuda") * 0.05).half()
    bias = torch.randn(n, device="cuda").float()
    w_q, w_scale, _ = backend.quantize_weight(weight)
    prepared = backend.prepare_weight_nk(w_q, mods)
    plain = backend.linear_forward(x, prepared, w_scale, bias).clone()
    for copies in (1, 3, 7):
        out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        peers = [torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda") for _ in range(copies)]
        words = torch.zeros(2, dtype=torch.int32, device="cuda")
        peer_words = torch.full((copies, 4), -1, dtype=torch.int32, device="cuda")
        backend.linear_forward(x, prepared, w_scale, bias, out=out, absmax_out=words.data_ptr(),
                               out_copies=[p.data_ptr() for p in peers],
                               absmax_copies=[peer_words[i].data_ptr() for i in range(copies)])
        torch.cuda.synchronize()
        assert torch.equal(out, plain)
        for p in peers:
            assert torch.equal(p, plain)
        expect = float(plain.float().abs().max())
        assert words[:1].view(torch.float32).item() == expect
        assert int(words[1]) == 148 or int(words[1]) > 0            # every CTA counted itself
        for i in range(copies):
            assert peer_words[i, :1].view(torch.float32).item() == expect
            assert int(peer_words[i, 1]) == -1                       # only the word itself is handed over
    backend.check_status()
    with pytest.raises(ValueError):
        backend.linear_forward(x[:64], prepared, w_scale, bias, out_copies=[plain.data_ptr()])


def test_adaptive_many_token_calls_take_the_two_cta_kernel(backend):
    """Adaptive layers with many tokens: the prefix is chosen on the device as always (metadata,
    counters), the two-CTA kernel computes only that prefix, and the outputs are those of the
    non-adaptive layer bit for bit (every sufficient prefix reconstructs the same integer)."""
    from rns_llm_b200.layers import RNSLinear
    torch.manual_seed(17)
    m, k, n = 640, 1024, 384
    plain = RNSLinear(k, n, backend=backend, mode="rns", moduli=C0).half().cuda().eval()
    adaptive = RNSLinear(k, n, backend=backend, mode="rns", moduli=C0, adaptive_channels=True,
                         adaptive_min_channels=3).half().cuda().eval()
    adaptive.load_state_dict(plain.state_dict())
    x = torch.randn(m, k, dtype=torch.float16, device="cuda") * 0.02
    x[0, 0] = 1.0                                   # one large value: small quantised rows, a three-channel bound
    backend.reset_stats()
    with torch.no_grad():
        y_plain = plain(x)
        y_adaptive = adaptive(x)
    torch.cuda.synchronize()
    backend.check_status()
    assert torch.equal(y_plain, y_adaptive)
    meta = adaptive.last_adaptive_metadata
    assert meta is not None and int(meta["channels"]) in (3, 4) and int(meta["bound"]) <= int(meta["capacity"])
    res = O.rns_linear_forward(x.float().cpu().numpy(), plain.weight.detach().float().cpu().numpy(),
                               plain.bias.detach().float().cpu().numpy(), C0, out_dtype=np.float16)
    expect_channels, expect_bound = O.adaptive_channels(res["a_q"], res["w_q"], C0, 3)
    assert int(meta["channels"]) == expect_channels and int(meta["bound"]) == expect_bound
    assert np.array_equal(y_adaptive.cpu().numpy(), res["y"])
    assert backend.stats_snapshot()["adaptive_selections"] == 1


@pytest.mark.parametrize("mods,min_channels", [(C0, 3), (C4, 3)])
def test_adaptive_integer_entry_with_many_tokens(backend, mods, min_channels):
    """matmul_prepared_adaptive_fused at M >= 512: tiled planes from int8 activations, the
    prefix chosen on the device, the two-CTA kernel computing only that prefix."""
    rng = np.random.default_rng(77 + len(mods))
    m, k, n = 700, 768, 520
    w_kn = rng.integers(-127, 128, size=(k, n)).astype(np.int8)
    adaptive = backend.prepare_weight_adaptive(torch.from_numpy(w_kn).cuda(), mods, min_channels=min_channels)
    backend.reset_stats()
    seen = set()
    for a_max in (3, 40, 127):
        a = rng.integers(-a_max, a_max + 1, size=(m, k)).astype(np.int8)
        out, meta = backend.matmul_prepared_adaptive_fused(torch.from_numpy(a).cuda(), adaptive, return_metadata=True)
        assert np.array_equal(out.cpu().numpy(), O.exact_matmul(a, w_kn)), a_max
        expect = O.adaptive_channels(a, w_kn.T, mods, min_channels)
        assert (meta["channels"], meta["bound"]) == expect
        seen.add(expect[0])
    assert len(seen) >= 2                                        # more than one prefix length was exercised
    backend.check_status()
    # the non-adaptive integer entry takes the same kernel
    full = backend.prepare_weight(torch.from_numpy(w_kn).cuda(), mods)
    a = rng.integers(-127, 128, size=(m, k)).astype(np.int8)
    assert np.array_equal(backend.matmul_prepared_fused(torch.from_numpy(a).cuda(), full).cpu().numpy(),
                          O.exact_matmul(a, w_kn))
