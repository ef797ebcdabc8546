"""Module-level behaviour that needs no GPU: the fused-QKV proxy/cache protocol
in mode="torch" (as tests/test_qkv_fusion.py of the reference), constructor
validation, the arena, and that the product path refuses to run without CUDA."""
import pytest
import torch
from torch import nn

from rns_llm_b200.layers import CachedRNSQKV, RNSLinear, RNSQKVProjection, install_opt_qkv_fusion


def make_linears(dtype=torch.float32):
    torch.manual_seed(123)
    return tuple(nn.Linear(16, 16, bias=True, dtype=dtype).eval() for _ in range(3))


def test_torch_qkv_fusion_matches_three_linears():
    q, k, v = make_linears()
    fused = RNSQKVProjection.from_linears(q, k, v, mode="torch").eval()
    x = torch.randn(2, 5, 16)
    for left, right in zip(fused(x), (q(x), k(x), v(x))):
        torch.testing.assert_close(left, right, rtol=1e-6, atol=2e-7)
    assert fused.compute_count == 1
    assert fused.split_sizes == (16, 16, 16)


def test_cached_qkv_computes_once_for_three_projection_calls():
    q, k, v = make_linears()
    projection = RNSQKVProjection.from_linears(q, k, v, mode="torch").eval()
    coordinator = CachedRNSQKV(projection).eval()
    q_proxy, k_proxy, v_proxy = coordinator.slices()
    x = torch.randn(2, 5, 16)
    actual = (q_proxy(x), k_proxy(x), v_proxy(x))
    assert projection.compute_count == 1
    assert coordinator.cache_misses == 1 and coordinator.cache_hits == 2
    for left, right in zip(actual, (q(x), k(x), v(x))):
        torch.testing.assert_close(left, right, rtol=1e-6, atol=2e-7)
    _ = q_proxy(x), k_proxy(x), v_proxy(x)
    assert projection.compute_count == 2
    # the same slice twice in a row is a new logical call
    _ = q_proxy(x), q_proxy(x)
    assert projection.compute_count == 4
    with pytest.raises(ValueError):
        coordinator.forward_slice(x, 3)


class DummyAttention(nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj = make_linears()

    def forward(self, x):
        return self.q_proj(x), self.k_proj(x), self.v_proj(x)


def test_proxy_installation_preserves_outputs_and_registers_parameters_once():
    attention = DummyAttention().eval()
    x = torch.randn(2, 3, 16)
    expected = attention(x)
    projection = RNSQKVProjection.from_linears(
        attention.q_proj, attention.k_proj, attention.v_proj, mode="torch").eval()
    coordinator = CachedRNSQKV(projection).eval()
    attention.rns_qkv = coordinator
    attention.q_proj, attention.k_proj, attention.v_proj = coordinator.slices()
    for left, right in zip(attention(x), expected):
        torch.testing.assert_close(left, right, rtol=1e-6, atol=2e-7)
    assert projection.compute_count == 1
    names = [name for name, _ in attention.named_parameters()]
    assert sorted(names) == ["rns_qkv.projection.combined.bias", "rns_qkv.projection.combined.weight"]


def test_install_rejects_non_linear_projections():
    attention = DummyAttention()
    attention.q_proj = nn.Identity()
    with pytest.raises(TypeError):
        install_opt_qkv_fusion(attention, backend=None)


def test_from_linears_validation():
    q, k, v = make_linears()
    with pytest.raises(TypeError):
        RNSQKVProjection.from_linears(q, k, nn.Identity(), mode="torch")
    with pytest.raises(ValueError):
        RNSQKVProjection.from_linears(q, k, nn.Linear(8, 16), mode="torch")
    with pytest.raises(ValueError):
        RNSQKVProjection.from_linears(q, k, nn.Linear(16, 16, bias=False), mode="torch")
    with pytest.raises(ValueError):
        RNSQKVProjection(RNSLinear(16, 48), (16, 16, 8))


def test_rns_linear_constructor_and_modes():
    with pytest.raises(ValueError):
        RNSLinear(8, 8, quant_bits=7)
    with pytest.raises(ValueError):
        RNSLinear(8, 8, lut_channels=3)
    with pytest.raises(ValueError):
        RNSLinear(8, 8, moduli=(126, 124))
    with pytest.raises(ValueError):
        RNSLinear(8, 8, activation_scale="column")
    layer = RNSLinear(768, 8, quant_bits=8)
    assert layer.moduli == (255, 253, 251, 247)   # dense_coprime default of the reference
    assert RNSLinear(768, 8, moduli=(127, 126, 125, 121)).moduli == (127, 126, 125, 121)
    assert layer.quant_max == 127 and layer.quant_dtype == torch.int8
    assert RNSLinear(8, 8, quant_bits=12).quant_dtype == torch.int16
    layer.mode = "rns"
    with pytest.raises(RuntimeError):
        layer(torch.randn(2, 768))           # training mode
    layer.eval()
    with pytest.raises(RuntimeError):
        layer(torch.randn(2, 768))           # no backend
    layer.backend = object()
    with pytest.raises(RuntimeError):
        layer(torch.randn(2, 768))           # CPU weights: there is no CPU fallback
    layer.mode = "bogus"
    with pytest.raises(ValueError):
        layer(torch.randn(2, 768))
    src = nn.Linear(12, 6)
    copy = RNSLinear.from_linear(src, mode="torch")
    x = torch.randn(3, 12)
    torch.testing.assert_close(copy(x), src(x))
    assert set(copy.state_dict()) == {"weight", "bias"}


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_backend_fails_loudly_without_cuda():
    from rns_llm_b200.backends import CudaRNSBackend
    with pytest.raises(RuntimeError):
        CudaRNSBackend()


def test_reference_alias_module():
    from rns_llm_b200 import reference
    assert reference.choose_moduli_for_dot(64, 127, 127) == (251, 241, 239)
    assert reference.validate_moduli([3, 5]) == (3, 5)
