"""Host-side routing between the kernels (no GPU): which calls the backend sends to the one-launch
kernel, the weight-streaming kernel, the general kernel and the two-CTA kernel, and the host-only
entry points of the C ABI that the decision reads."""
import pytest

from rns_llm_b200 import _native as N

C0 = (127, 126, 125, 121)


@pytest.fixture(scope="module")
def lib():
    return N.load()


@pytest.fixture(scope="module")
def router(lib):
    """A backend object without a device: only the routing helper and the library are used."""
    from rns_llm_b200.backends.cuda_backend import CudaRNSBackend
    backend = object.__new__(CudaRNSBackend)
    backend._lib = lib
    return backend


def test_tile_rows_of_the_two_cta_kernel(lib):
    assert lib.rns_pair_tile_rows(4, 4096) == 64
    assert lib.rns_pair_tile_rows(5, 16384) == 48
    assert lib.rns_pair_tile_rows(6, 1024) == 32
    assert lib.rns_pair_tile_rows(3, 4096) == 0           # channel counts it does not cover
    assert lib.rns_pair_tile_rows(7, 4096) == 0
    assert lib.rns_pair_tile_rows(4, 256) == 0            # K below 512
    assert lib.rns_pair_tile_rows(4, 520) == 0            # K % 16 != 0
    # planes are padded to whole token tiles of 2 * tile_rows rows and whole 64-byte K blocks
    assert lib.rns_packed_planes_bytes(4096, 4096, 4, 64) == 4096 * 4096 * 4
    assert lib.rns_packed_planes_bytes(130, 528, 5, 48) == 192 * 576 * 5
    assert lib.rns_packed_planes_bytes(1, 512, 6, 32) == 64 * 512 * 6


def test_few_token_kernels_say_what_they_cover(lib):
    assert lib.rns_linear_small_supported(1, 768, 4) == 1
    assert lib.rns_linear_small_supported(32, 1536, 4) == 1
    assert lib.rns_linear_small_supported(33, 768, 4) == 0          # more than 32 tokens
    assert lib.rns_linear_small_supported(8, 3072, 4) == 0          # residues of a token block exceed shared memory
    assert lib.rns_linear_small_supported(8, 1536, 5) == 0
    assert lib.rns_linear_stream_supported(8, 3072, 4) == 1
    assert lib.rns_linear_stream_supported(64, 16384, 5) == 1
    assert lib.rns_linear_stream_supported(65, 4096, 4) == 0
    assert lib.rns_linear_stream_supported(8, 4096, 6) == 0         # static shared memory: up to five channels
    assert lib.rns_linear_stream_supported(8, 4104, 4) == 0         # K % 16 != 0
    assert lib.rns_linear_stream_supported(8, 131088, 4) == 0       # int32 channel sums could overflow


@pytest.mark.parametrize("m,k,n,channels,rows", [
    (4096, 4096, 12288, 4, 64),      # the layer stack
    (4096, 16384, 4096, 5, 48),
    (512, 1024, 1024, 6, 32),
    (320, 768, 2304, 4, 64),         # from 320 rows on, whatever the weight
    (319, 768, 2304, 4, 0),          # below: small weights stay on the general kernel
    (48, 768, 2304, 4, 0),
    (48, 4096, 4096, 4, 64),         # large weights (K * N >= 2^23): from 33 rows on
    (33, 4096, 2048, 4, 64),
    (33, 4096, 2047 // 8 * 8, 4, 0),
    (8, 768, 2304, 4, 0),            # few tokens that the one-launch kernel takes
    (8, 4096, 12288, 4, 64),         # few tokens it cannot hold, large weight
    (4096, 4096, 4096, 3, 0),        # channel counts and K the two-CTA kernel does not cover
    (4096, 256, 4096, 4, 0),
])
def test_which_calls_take_the_two_cta_kernel(router, m, k, n, channels, rows):
    assert router._pair_tile_rows(m, k, n, channels) == rows


def test_thresholds_are_the_documented_ones():
    from rns_llm_b200.backends import cuda_backend as CB
    assert (CB.PLANES_MIN_ROWS, CB.PAIR_MIN_ROWS, CB.PAIR_LARGE_WEIGHT, CB.STREAM_MAX_ROWS, CB.WIDE_MIN_ROWS) == (
        512, 320, 1 << 23, 32, 128)
