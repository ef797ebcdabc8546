from .rns_linear import RNSLinear
from .rns_qkv import (
    CachedRNSQKV,
    InstalledQKVFusion,
    RNSQKVProjection,
    install_opt_qkv_fusion,
)

__all__ = [
    "RNSLinear",
    "RNSQKVProjection",
    "CachedRNSQKV",
    "InstalledQKVFusion",
    "install_opt_qkv_fusion",
]
