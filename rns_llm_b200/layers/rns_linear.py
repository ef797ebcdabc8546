"""RNSLinear: inference-only drop-in for ``nn.Linear`` on the RNS backend.

Constructor, class methods, attributes and error behaviour follow the
reference's ``src/rns_llm/layers/rns_linear.py`` (:27-152, 225-275).  What
``forward`` does in ``mode="rns"`` is numerically the same recipe

    s_w[n] = max(max_k |W[n,k]| / qmax, eps)        Wq = clamp(rint(W / s_w))
    s_a    = max(max |x| / qmax, eps)               Aq = clamp(rint(x / s_a))
    y      = dtype( f32(Aq @ Wq^T) * s_a * s_w[n] + bias[n] )

but runs as a quantiser launch plus ONE fused GEMM launch: residues of Aq and
Wq are formed inside the GEMM, the per-channel int32 sums never leave the SM,
and the epilogue reconstructs, recentres and dequantises.  The cached weight is
Wq itself in the [out,in] layout, one byte per value for any channel count.
"""
from __future__ import annotations

from typing import Iterable

import torch
from torch import nn
from torch.nn import functional as F

from ..backends import PreparedAdaptiveRNSWeight, PreparedRNSWeight, RNSWorkspace
from ..moduli import choose_moduli_for_dot, validate_moduli


class RNSLinear(nn.Module):
    def __init__(
        self,
        in_features: int,
        out_features: int,
        *,
        bias: bool = True,
        backend=None,
        moduli: Iterable[int] | None = None,
        moduli_strategy: str = "dense_coprime",
        mode: str = "torch",
        kernel: str = "auto",
        quant_bits: int = 8,
        fused: bool = True,
        lut_channels: int = 2,
        adaptive_channels: bool = False,
        adaptive_min_channels: int = 3,
        activation_scale: str = "tensor",
    ) -> None:
        super().__init__()
        if quant_bits not in (8, 12, 16):
            raise ValueError("quant_bits must be 8, 12 or 16")
        if lut_channels not in (0, 1, 2):
            raise ValueError("lut_channels must be 0, 1 or 2")
        if activation_scale not in ("tensor", "row"):
            raise ValueError("activation_scale must be 'tensor' or 'row'")
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.backend = backend
        self.mode = mode
        self.kernel = kernel
        self.quant_bits = int(quant_bits)
        self.fused = bool(fused)
        # Accepted and validated for interface compatibility; the sm_100a
        # epilogue reduces in registers and reads no table.
        self.lut_channels = int(lut_channels)
        self.moduli_strategy = moduli_strategy
        self.adaptive_channels = bool(adaptive_channels)
        self.adaptive_min_channels = int(adaptive_min_channels)
        # "tensor": one scale for the whole activation, as the reference;
        # "row": one scale per token row.
        self.activation_scale = activation_scale

        qmax = self.quant_max
        chosen = tuple(moduli) if moduli is not None else choose_moduli_for_dot(
            self.in_features, qmax, qmax, strategy=moduli_strategy)
        self.moduli = validate_moduli(chosen)

        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self.register_buffer("_weight_scale", torch.empty(0), persistent=False)
        self.register_buffer("_weight_residues", torch.empty(0, dtype=torch.int8), persistent=False)
        self._reset_cache_fields()
        self.reset_parameters()

    # ------------------------------------------------------------------
    @property
    def quant_max(self) -> int:
        return (1 << (self.quant_bits - 1)) - 1

    @property
    def quant_dtype(self) -> torch.dtype:
        return torch.int8 if self.quant_bits == 8 else torch.int16

    def _reset_cache_fields(self) -> None:
        self._prepared_weight_version: int | None = None
        self._prepared_bias_version: int | None = None
        self._prepared_weight: PreparedRNSWeight | None = None
        self._adaptive_prepared_weight: PreparedAdaptiveRNSWeight | None = None
        self._bias_f32: torch.Tensor | None = None
        self._workspace_by_rows: dict[tuple[int, int, int], RNSWorkspace] = {}
        self.last_adaptive_metadata = None

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        if self.bias is not None:
            bound = 1 / self.in_features ** 0.5
            nn.init.uniform_(self.bias, -bound, bound)
        self.clear_weight_cache()

    def clear_weight_cache(self) -> None:
        self._weight_scale = torch.empty(0, device=self.weight.device)
        self._weight_residues = torch.empty(0, dtype=torch.int8, device=self.weight.device)
        self._reset_cache_fields()

    @classmethod
    def from_linear(cls, layer: nn.Linear, *, backend=None, moduli: Iterable[int] | None = None,
                    moduli_strategy: str = "dense_coprime", mode: str = "torch", kernel: str = "auto",
                    quant_bits: int = 8, fused: bool = True, lut_channels: int = 2,
                    adaptive_channels: bool = False, adaptive_min_channels: int = 3,
                    activation_scale: str = "tensor") -> "RNSLinear":
        result = cls(
            layer.in_features, layer.out_features, bias=layer.bias is not None, backend=backend,
            moduli=moduli, moduli_strategy=moduli_strategy, mode=mode, kernel=kernel,
            quant_bits=quant_bits, fused=fused, lut_channels=lut_channels,
            adaptive_channels=adaptive_channels, adaptive_min_channels=adaptive_min_channels,
            activation_scale=activation_scale,
        ).to(device=layer.weight.device, dtype=layer.weight.dtype)
        result.weight.data.copy_(layer.weight.data)
        if layer.bias is not None and result.bias is not None:
            result.bias.data.copy_(layer.bias.data)
        return result

    # Same arithmetic as the reference's helpers (rns_linear.py:154-166); used for
    # sources wider than 8 bits, which take the plane-level pipeline.
    def _symmetric_scale(self, values: torch.Tensor, dim=None) -> torch.Tensor:
        max_abs = values.detach().abs().amax(dim=dim, keepdim=True)
        # Tensor divisor: with a Python scalar torch's CUDA kernel multiplies by the rounded
        # reciprocal, which differs from the IEEE quotient (what the reference computes on the
        # CPU and the quantiser kernels compute) in the last bit for some inputs.
        return torch.clamp(max_abs / torch.full_like(max_abs, float(self.quant_max)),
                           min=torch.finfo(torch.float32).eps)

    def _quantize(self, values: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        return torch.clamp(torch.round(values / scale), -self.quant_max, self.quant_max).to(self.quant_dtype)

    # ------------------------------------------------------------------
    @torch.no_grad()
    def prepare_weight(self) -> None:
        """Quantise (and cache) the weight; redone when ``weight`` is modified in
        place (rns_linear.py:168-204)."""
        if self.backend is None:
            raise RuntimeError("RNSLinear requires a backend in mode='rns'")
        if not self.weight.is_cuda:
            raise RuntimeError("RNSLinear currently expects CUDA weights")
        version = self.weight._version
        if self._prepared_weight_version == version and self._prepared_weight is not None:
            return
        backend = self.backend
        if self.quant_bits == 8:
            weight = self.weight.detach()
            if weight.stride(1) != 1:
                weight = weight.contiguous()
            w_q, scale, max_abs = backend.quantize_weight(weight, self.quant_max)
            prepared = backend.prepare_weight_nk(w_q, self.moduli)
            adaptive = None
            if self.adaptive_channels:
                adaptive = backend._adaptive_from_full(prepared, int(max_abs.item()),
                                                       self.adaptive_min_channels)
        else:
            w32 = self.weight.float()
            scale2d = self._symmetric_scale(w32, dim=1)
            quantized_b = self._quantize(w32, scale2d).transpose(0, 1).contiguous()
            scale = scale2d.squeeze(1)
            adaptive = None
            if self.adaptive_channels:
                adaptive = backend.prepare_weight_adaptive(quantized_b, self.moduli,
                                                           min_channels=self.adaptive_min_channels)
                prepared = adaptive.variants[len(self.moduli)]
            else:
                prepared = backend.prepare_weight(quantized_b, self.moduli)
        self._weight_scale = scale.to(self.weight.device)
        # The reference exposes the cached planes here; this build caches the
        # quantised matrix itself when the tensor-core kernel serves the layer.
        self._weight_residues = (prepared.weight_packed if prepared.weight_packed is not None
                                 else prepared.residues)
        self._prepared_weight = prepared
        self._adaptive_prepared_weight = adaptive
        self._prepared_weight_version = version
        self._workspace_by_rows = {}

    def _bias_float(self) -> torch.Tensor | None:
        if self.bias is None:
            return None
        version = self.bias._version
        if self._bias_f32 is None or self._prepared_bias_version != version:
            self._bias_f32 = self.bias.detach().float().contiguous()
            self._prepared_bias_version = version
        return self._bias_f32

    def _workspace(self, rows: int, channels: int | None = None) -> RNSWorkspace:
        """Workspace per (rows, channels, stream) as the reference (rns_linear.py:
        206-223); only the plane-level pipeline (wide sources) needs one."""
        assert self._prepared_weight is not None
        channels = len(self.moduli) if channels is None else int(channels)
        stream = torch.cuda.current_stream(self.weight.device)
        key = (int(rows), int(channels), int(stream.cuda_stream))
        cached = self._workspace_by_rows.get(key)
        if cached is None:
            cached = self.backend.create_workspace(device=self.weight.device, channels=channels,
                                                   m=rows, n=self.out_features)
            self._workspace_by_rows[key] = cached
        return cached

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if self.mode == "torch":
            return F.linear(inputs, self.weight, self.bias)
        if self.mode != "rns":
            raise ValueError(f"unknown mode: {self.mode}")
        if self.training:
            raise RuntimeError("RNSLinear is inference-only; call eval()")
        if self.backend is None:
            raise RuntimeError("RNSLinear mode='rns' requires a backend")
        self.prepare_weight()
        prepared = self._prepared_weight
        assert prepared is not None
        lead = inputs.shape[:-1]
        flat = inputs.reshape(-1, self.in_features)

        if prepared.kernel == "tcgen05" and self.fused and self.quant_bits == 8:
            if flat.stride(-1) != 1 or flat.dtype not in (torch.float16, torch.bfloat16, torch.float32):
                flat = flat.contiguous() if flat.dtype in (torch.float16, torch.bfloat16, torch.float32) \
                    else flat.float().contiguous()
            result = self.backend.linear_forward(
                flat, prepared, self._weight_scale, self._bias_float(),
                per_row=self.activation_scale == "row",
                adaptive=self._adaptive_prepared_weight,
                return_metadata=self.adaptive_channels,
            )
            if self.adaptive_channels:
                result, self.last_adaptive_metadata = result
            return result.reshape(*lead, self.out_features).to(inputs.dtype)

        if (self.quant_bits != 8 and self.fused and not self.adaptive_channels
                and self.backend.supports_wide_forward(prepared, flat.shape[0])):
            # 12/16-bit sources with enough rows: quantiser -> residue planes -> the two-CTA
            # tensor-core kernel with the weight's cached residue planes.
            if flat.stride(-1) != 1 or flat.dtype not in (torch.float16, torch.bfloat16, torch.float32):
                flat = flat.contiguous() if flat.dtype in (torch.float16, torch.bfloat16, torch.float32) \
                    else flat.float().contiguous()
            result = self.backend.linear_forward_wide(
                flat, prepared, self._weight_scale, self._bias_float(), quant_max=self.quant_max,
                per_row=self.activation_scale == "row")
            return result.reshape(*lead, self.out_features).to(inputs.dtype)

        # Wide sources (12/16-bit) with few rows, or shapes outside the tensor-core kernel:
        # the reference's plane-level pipeline, op for op (rns_linear.py:239-275).
        flat = flat.float().contiguous()
        scale_dim = 1 if self.activation_scale == "row" else None
        activation_scale = self._symmetric_scale(flat, dim=scale_dim)
        quantized_a = self._quantize(flat, activation_scale).contiguous()
        if self.adaptive_channels:
            assert self._adaptive_prepared_weight is not None
            workspaces = {c: self._workspace(flat.shape[0], c) for c in self._adaptive_prepared_weight.variants}
            integer_result, metadata = self.backend.matmul_prepared_adaptive_fused(
                quantized_a, self._adaptive_prepared_weight, lut_channels=self.lut_channels,
                workspace_by_channels=workspaces, return_metadata=True)
            self.last_adaptive_metadata = metadata
            integer_result = integer_result.float()
        elif self.fused and prepared.kernel in ("cublas", "tcgen05"):
            integer_result = self.backend.matmul_prepared_fused(
                quantized_a, prepared, lut_channels=self.lut_channels,
                workspace=self._workspace(flat.shape[0])).float()
        else:
            integer_result = self.backend.matmul_prepared(quantized_a, prepared, kernel=self.kernel).float()
        output = integer_result * activation_scale * self._weight_scale.unsqueeze(0)
        if self.bias is not None:
            output = output + self.bias.float()
        return output.reshape(*lead, self.out_features).to(inputs.dtype)
