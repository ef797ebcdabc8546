"""Model-level replacement of nn.Linear layers by RNS linears.

The reference keeps these recipes in a script (scripts/evaluate_ppl.py:20-94 of the
reference): attention blocks get one fused q|k|v projection plus, optionally, an RNS
``out_proj``; any other linear (the FFN's ``fc1`` / ``fc2``) is swapped by name pattern.
Here they are library functions with the same behaviour and an optional ``moduli``
argument (the reference always derives moduli from ``moduli_strategy``).
"""
from __future__ import annotations

from typing import Iterable, Sequence

from torch import nn

from .layers import RNSLinear, install_opt_qkv_fusion


def find_parent(model: nn.Module, dotted_name: str) -> tuple[nn.Module, str]:
    """The module that owns ``dotted_name`` and the attribute under which it holds it."""
    parent = model
    parts = dotted_name.split(".")
    for part in parts[:-1]:
        parent = getattr(parent, part)
    return parent, parts[-1]


def replace_opt_attention_blocks(model: nn.Module, *, backend, blocks: int | None = None, quant_bits: int = 8,
                                 include_out_proj: bool = True, adaptive_channels: bool = False,
                                 moduli: Iterable[int] | None = None,
                                 moduli_strategy: str = "dense_coprime") -> tuple[list[str], list[nn.Module]]:
    """Fuses q/k/v of the first ``blocks`` attention modules (every module that has
    ``q_proj``, ``k_proj`` and ``v_proj`` linears; all of them when ``blocks`` is None)
    and, with ``include_out_proj``, replaces their ``out_proj``.  Returns the names of
    what was replaced and the fused-QKV coordinators, whose ``compute_count`` a caller
    checks to make sure the RNS path really ran (scripts/evaluate_ppl.py:53-94, 212-217)."""
    candidates = [(name, module) for name, module in model.named_modules()
                  if all(isinstance(getattr(module, attr, None), nn.Linear) for attr in ("q_proj", "k_proj", "v_proj"))]
    if blocks is not None:
        candidates = candidates[:blocks]
    replaced: list[str] = []
    coordinators: list[nn.Module] = []
    for name, attention in candidates:
        coordinators.append(install_opt_qkv_fusion(attention, backend=backend, quant_bits=quant_bits,
                                                   moduli_strategy=moduli_strategy, lut_channels=2,
                                                   adaptive_channels=adaptive_channels, moduli=moduli))
        replaced.append(f"{name}.qkv_fused")
        if include_out_proj:
            if not isinstance(attention.out_proj, nn.Linear):
                raise TypeError(f"{name}.out_proj is not nn.Linear")
            attention.out_proj = RNSLinear.from_linear(attention.out_proj, backend=backend, mode="rns",
                                                       quant_bits=quant_bits, fused=True, lut_channels=2,
                                                       moduli=moduli, moduli_strategy=moduli_strategy,
                                                       adaptive_channels=adaptive_channels).eval()
            replaced.append(f"{name}.out_proj")
    return replaced, coordinators


def replace_selected_linears(model: nn.Module, *, backend, patterns: Sequence[str], max_layers: int | None = None,
                             quant_bits: int = 8, adaptive_channels: bool = False,
                             moduli: Iterable[int] | None = None,
                             moduli_strategy: str = "dense_coprime") -> list[str]:
    """Replaces the first ``max_layers`` nn.Linear modules whose qualified name contains one
    of ``patterns`` (e.g. ("fc1", "fc2") for an OPT feed-forward block) by RNS linears
    (scripts/evaluate_ppl.py:20-50).  A layer whose K needs more moduli than the given set
    covers gets its own set through ``moduli_strategy`` when ``moduli`` is None."""
    candidates = [(name, module) for name, module in model.named_modules()
                  if isinstance(module, nn.Linear) and any(pattern in name for pattern in patterns)]
    if max_layers is not None:
        candidates = candidates[:max_layers]
    replaced = []
    for name, layer in candidates:
        parent, attribute = find_parent(model, name)
        setattr(parent, attribute, RNSLinear.from_linear(layer, backend=backend, mode="rns", quant_bits=quant_bits,
                                                         fused=True, lut_channels=2, moduli=moduli,
                                                         moduli_strategy=moduli_strategy,
                                                         adaptive_channels=adaptive_channels).eval())
        replaced.append(name)
    return replaced
