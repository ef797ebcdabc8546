"""The allocation-free entry point rns_linear_static against the ordinary path.

It serves hosts that bind the C ABI directly and cannot allocate device memory on
the request path (a C/C++ serving loop that owns no allocator): its scratch is a
fixed array inside the library.  Two calls in a row, with different inputs, must
give bit for bit what backend.linear_forward gives (this suite's tolerance for the
dequantised path is exact equality), whether this file runs alone or last.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

C0 = (127, 126, 125, 121)


def test_static_scratch_entry_matches_arena_path_twice():
    from rns_llm_b200 import _native as N
    from rns_llm_b200.backends import CudaRNSBackend

    backend = CudaRNSBackend()
    lib = N.load()
    torch.manual_seed(77)
    k, n = 768, 2304
    weight = (torch.randn(n, k, device="cuda") * 0.02).half()
    bias = (torch.randn(n, device="cuda") * 0.02).float()
    w_q, w_scale, _ = backend.quantize_weight(weight)
    prepared = backend.prepare_weight_nk(w_q, C0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.rns_static_scratch_bytes() == 8 << 20

    for step, m in enumerate((16, 200)):          # second call: other shape, other data, same array
        x = (torch.randn(m, k, device="cuda") * (1.0 + step)).half()
        expect = backend.linear_forward(x, prepared, w_scale, bias)
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        N.check(lib.rns_linear_static(x.data_ptr(), N.F16, m, k, k, prepared.weight_packed.data_ptr(), n,
                                      N.moduli_array(C0), 4, w_scale.data_ptr(), bias.data_ptr(),
                                      got.data_ptr(), n, N.OUT_F16, status.data_ptr(), stream))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(got, expect)
    backend.check_status()

    # beyond the built-in array: refused with a clear error, nothing launched
    too_many_rows = (8 << 20) // 768 + 512
    with pytest.raises(ValueError) as err:
        N.check(lib.rns_linear_static(x.data_ptr(), N.F16, too_many_rows, k, k, prepared.weight_packed.data_ptr(), n,
                                      N.moduli_array(C0), 4, w_scale.data_ptr(), bias.data_ptr(),
                                      got.data_ptr(), n, N.OUT_F16, status.data_ptr(), stream))
    assert "scratch" in str(err.value)

    # bad arguments are refused before anything is queued (NULL moduli, K % 16 != 0)
    for bad in (dict(moduli=None), dict(k=772)):
        kk = bad.get("k", k)
        mods = bad.get("moduli", N.moduli_array(C0))
        code = lib.rns_linear_static(x.data_ptr(), N.F16, 16, kk, kk, prepared.weight_packed.data_ptr(), n,
                                     mods, 4, w_scale.data_ptr(), bias.data_ptr(),
                                     got.data_ptr(), n, N.OUT_F16, status.data_ptr(), stream)
        assert code in (N.ERR_INVALID_ARGUMENT, N.ERR_UNSUPPORTED)
