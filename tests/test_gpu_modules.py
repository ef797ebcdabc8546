"""RNSLinear / fused QKV modules on the GPU: the checks of the reference's
benchmarks/benchmark_qkv_fusion.py:80-84 (fused output bit-equal to three
separate layers) and of scripts/evaluate_ppl.py:212-217 (the fused kernel
really ran), on configuration-1 shapes."""
import numpy as np
import pytest
import torch
from torch import nn

from oracle import rns_oracle as O

pytestmark = pytest.mark.gpu

C0 = (127, 126, 125, 121)


@pytest.fixture(scope="module")
def backend():
    from rns_llm_b200.backends import CudaRNSBackend
    return CudaRNSBackend()


def qkv_linears(hidden=768, dtype=torch.float16):
    torch.manual_seed(1001)
    layers = []
    for _ in range(3):
        layer = nn.Linear(hidden, hidden, bias=True, device="cuda", dtype=dtype).eval()
        with torch.no_grad():
            layer.weight.normal_(0, 0.02)
            layer.bias.normal_(0, 0.02)
        layers.append(layer)
    return layers


@pytest.mark.parametrize("tokens", [1, 16, 128, 256])
@pytest.mark.parametrize("activation_scale", ["tensor", "row"])
def test_fused_qkv_bit_equals_three_layers(backend, tokens, activation_scale):
    from rns_llm_b200.layers import RNSLinear, RNSQKVProjection
    originals = qkv_linears()
    separate = [RNSLinear.from_linear(l, backend=backend, mode="rns", moduli=C0,
                                      activation_scale=activation_scale).eval() for l in originals]
    fused = RNSQKVProjection.from_linears(*originals, backend=backend, mode="rns", moduli=C0,
                                          activation_scale=activation_scale).eval()
    x = torch.randn(1, tokens, 768, device="cuda", dtype=torch.float16)
    backend.reset_stats()
    outs = fused(x)
    assert backend.stats_snapshot()["fused_gemm_calls"] == 1
    for got, layer, orig in zip(outs, separate, originals):
        expect = layer(x)
        assert got.shape == (1, tokens, 768) and got.dtype == torch.float16
        assert torch.equal(got, expect)
        res = O.rns_linear_forward(x.cpu().numpy(), orig.weight.detach().cpu().numpy(),
                                   orig.bias.detach().cpu().numpy(), C0,
                                   per_row=activation_scale == "row")
        assert np.array_equal(expect.cpu().numpy(), res["y"])
        # and it is a faithful int8 approximation of the fp16 layer
        ref = orig(x).detach().float()
        assert float((expect.float() - ref).abs().max()) < 0.05
    backend.check_status()


def test_installed_fusion_in_attention_like_module(backend):
    from rns_llm_b200.layers import install_opt_qkv_fusion

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.k_proj, self.v_proj = qkv_linears(256)

        def forward(self, h):
            return self.q_proj(h), self.k_proj(h), self.v_proj(h)

    attention = Attention().eval()
    h = torch.randn(2, 7, 256, device="cuda", dtype=torch.float16)
    expected = [t.float() for t in attention(h)]
    coordinator = install_opt_qkv_fusion(attention, backend=backend, moduli=C0)
    backend.reset_stats()
    got = attention(h)
    assert coordinator.projection.compute_count == 1
    assert coordinator.cache_misses == 1 and coordinator.cache_hits == 2
    assert backend.stats_snapshot()["fused_gemm_calls"] == 1
    for g, e in zip(got, expected):
        assert float((g.detach().float() - e.detach()).abs().max()) < 0.05
    # default moduli of the reference installer: dense_coprime -> (255,253,251,247)
    attention2 = Attention().eval()
    c2 = install_opt_qkv_fusion(attention2, backend=backend)
    assert c2.projection.combined.moduli == (255, 253, 251)   # hidden 256: three moduli cover 2*256*127^2
    for g, e in zip(attention2(h), expected):
        assert float((g.detach().float() - e.detach()).abs().max()) < 0.05


def test_weight_cache_follows_in_place_updates(backend):
    from rns_llm_b200.layers import RNSLinear
    layer = RNSLinear(128, 48, backend=backend, mode="rns", moduli=C0).cuda().half().eval()
    x = torch.randn(5, 128, device="cuda", dtype=torch.float16)
    y1 = layer(x)
    cached = layer._prepared_weight
    assert layer(x).data_ptr() != 0 and layer._prepared_weight is cached
    # the cached weight is the packed int8 matrix: N padded to 384, K to 64, one byte per value
    assert layer._weight_residues.dtype == torch.int8 and layer._weight_residues.numel() == 384 * 128
    assert torch.equal(cached.weight_nk, backend.quantize_weight(layer.weight.detach())[0])
    with torch.no_grad():
        layer.weight.mul_(2.0)
    y2 = layer(x)
    assert layer._prepared_weight is not cached
    res = O.rns_linear_forward(x.cpu().numpy(), layer.weight.detach().cpu().numpy(),
                               layer.bias.detach().cpu().numpy(), C0)
    assert np.array_equal(y2.cpu().numpy(), res["y"]) and not torch.equal(y1, y2)
    layer.clear_weight_cache()
    assert layer._prepared_weight is None
    assert torch.equal(layer(x), y2)


def test_adaptive_module(backend):
    from rns_llm_b200.layers import RNSLinear
    torch.manual_seed(3)
    layer = RNSLinear(768, 768, backend=backend, mode="rns", moduli=C0, adaptive_channels=True,
                      adaptive_min_channels=3).cuda().half().eval()
    plain = RNSLinear(768, 768, backend=backend, mode="rns", moduli=C0).cuda().half().eval()
    plain.load_state_dict(layer.state_dict())
    # a few large outliers make most rows quantise to small integers -> 3 channels suffice
    x = torch.randn(128, 768, device="cuda", dtype=torch.float16)
    x[0, 0] = 40.0
    y = layer(x)
    assert torch.equal(y, plain(x))
    meta = layer.last_adaptive_metadata
    assert meta["channels"] == 3 and meta["bound"] <= meta["capacity"]
    x_full = torch.rand(128, 768, device="cuda", dtype=torch.float16) * 2 - 1
    assert torch.equal(layer(x_full), plain(x_full))
    assert layer.last_adaptive_metadata["channels"] == 4
    backend.check_status()


def test_wide_quant_bits_use_plane_pipeline(backend):
    from rns_llm_b200.layers import RNSLinear
    torch.manual_seed(9)
    layer = RNSLinear(64, 32, backend=backend, mode="rns", quant_bits=12).cuda().eval()
    x = torch.randn(6, 64, device="cuda")
    y = layer(x)
    ref = torch.nn.functional.linear(x, layer.weight, layer.bias)
    assert float((y - ref).abs().max()) < 5e-3
    assert layer._prepared_weight.kernel == "cublas"


def test_opt_decoder_layer_with_rns_attention(backend):
    """A randomly initialised OPT decoder layer (transformers) with q/k/v fused
    and out_proj replaced, as scripts/evaluate_ppl.py:53-94 of the reference."""
    transformers = pytest.importorskip("transformers")
    from rns_llm_b200.layers import RNSLinear, install_opt_qkv_fusion
    config = transformers.OPTConfig(vocab_size=512, hidden_size=768, num_hidden_layers=2,
                                    num_attention_heads=12, ffn_dim=3072, max_position_embeddings=128)
    torch.manual_seed(1003)
    model = transformers.OPTForCausalLM(config).half().cuda().eval()
    ids = torch.randint(0, 512, (2, 16), device="cuda")
    with torch.no_grad():
        base = model(ids).logits.float()
    for layer in model.model.decoder.layers:
        install_opt_qkv_fusion(layer.self_attn, backend=backend, moduli=C0)
        layer.self_attn.out_proj = RNSLinear.from_linear(layer.self_attn.out_proj, backend=backend,
                                                         mode="rns", moduli=C0).eval()
    backend.reset_stats()
    with torch.no_grad():
        logits = model(ids).logits.float()
        generated = model.generate(ids, max_new_tokens=4, do_sample=False)
    stats = backend.stats_snapshot()
    assert stats["fused_gemm_calls"] >= 4
    assert generated.shape == (2, 20)
    rel = float((logits - base).abs().max() / base.abs().max())
    assert rel < 0.05, rel
    backend.check_status()


class _ExactInt8Linear(torch.nn.Module):
    """Test twin of an RNS linear in plain torch: the reference's quantisation
    (layers/rns_linear.py:154-166, 183-184, 239-241), an exact int64 matrix product in
    place of the RNS GEMM, and its fp32 dequantisation order (:264, 272-275)."""

    def __init__(self, weight, bias):
        super().__init__()
        w = weight.detach().float()
        eps = torch.finfo(torch.float32).eps
        # Division by a TENSOR: on CUDA torch turns a division by a Python scalar into a
        # multiplication by its reciprocal, which rounds differently in the last place for
        # some values; the kernels (and torch on the CPU, where the golden vectors come
        # from) divide.
        amax = w.abs().amax(dim=1, keepdim=True)
        self.scale = torch.clamp(amax / torch.full_like(amax, 127.0), min=eps)
        self.wq = torch.clamp(torch.round(w / self.scale), -127, 127).to(torch.int64)
        self.bias = None if bias is None else bias.detach().float()

    def forward(self, x):
        flat = x.reshape(-1, x.shape[-1]).float()
        amax = flat.abs().amax()
        s_a = torch.clamp(amax / torch.full_like(amax, 127.0), min=torch.finfo(torch.float32).eps)
        xq = torch.clamp(torch.round(flat / s_a), -127, 127).to(torch.int64)
        acc = (xq.cpu() @ self.wq.cpu().t()).to(x.device)         # exact: int64 on the host
        y = acc.float() * s_a * self.scale.reshape(1, -1)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*x.shape[:-1], -1).to(x.dtype)


@pytest.mark.parametrize("tokens", [24, 520])
def test_opt125m_shaped_model_with_rns_attention_and_ffn(backend, tokens):
    """The 12-layer OPT-125m-shaped model of configuration 3 (smaller vocabulary to keep the
    test light) with every attention block (fused q|k|v + out_proj) and every FFN linear
    (fc1, fc2) replaced through the library's model-level helpers.  Its logits equal, bit
    for bit, those of a twin whose linears are exact int8 products in plain torch, and stay
    within a bound of the fp16 model's."""
    transformers = pytest.importorskip("transformers")
    import copy
    from rns_llm_b200.integration import find_parent, replace_opt_attention_blocks, replace_selected_linears

    config = transformers.OPTConfig(vocab_size=2048, hidden_size=768, num_hidden_layers=12, num_attention_heads=12,
                                    ffn_dim=3072, max_position_embeddings=1024, word_embed_proj_dim=768)
    torch.manual_seed(1003)
    base = transformers.OPTForCausalLM(config).half().cuda().eval()
    ids = torch.randint(0, 2048, (2, tokens // 2), device="cuda")
    rns = copy.deepcopy(base)
    replaced, coordinators = replace_opt_attention_blocks(rns, backend=backend, moduli=C0)
    replaced += replace_selected_linears(rns, backend=backend, patterns=("fc1", "fc2"), moduli=C0)
    assert len(replaced) == 12 * 4 and len(coordinators) == 12
    twin = copy.deepcopy(base)
    for layer in twin.model.decoder.layers:
        attn = layer.self_attn
        w = torch.cat([attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight], dim=0)
        b = torch.cat([attn.q_proj.bias, attn.k_proj.bias, attn.v_proj.bias], dim=0)
        fused = _ExactInt8Linear(w, b)
        for index, name in enumerate(("q_proj", "k_proj", "v_proj")):
            # the fused projection quantises the activation once; each slice is a column block
            setattr(attn, name, _Slice(fused, index, 768))
        attn.out_proj = _ExactInt8Linear(attn.out_proj.weight, attn.out_proj.bias)
        layer.fc1 = _ExactInt8Linear(layer.fc1.weight, layer.fc1.bias)
        layer.fc2 = _ExactInt8Linear(layer.fc2.weight, layer.fc2.bias)
    backend.reset_stats()
    with torch.no_grad():
        want = base(ids).logits.float()
        got = rns(ids).logits.float()
        exact = twin(ids).logits.float()
    backend.check_status()
    assert backend.stats_snapshot()["fused_gemm_calls"] == 12 * 4
    assert all(c.projection.compute_count == 1 for c in coordinators)
    assert torch.equal(got, exact)
    assert float((got - want).norm() / want.norm()) < 0.05


class _Slice(torch.nn.Module):
    def __init__(self, fused, index, width):
        super().__init__()
        self.fused, self.index, self.width = fused, index, width

    def forward(self, x):
        return self.fused(x)[..., self.index * self.width:(self.index + 1) * self.width]
