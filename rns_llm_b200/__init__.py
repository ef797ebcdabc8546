"""B200-native RNS linear path with the module and backend interface of
Nek1tt/rns-llm (``RNSLinear``, fused QKV, ``CudaRNSBackend``)."""
from .backends import (
    CudaRNSBackend,
    PreparedAdaptiveRNSWeight,
    PreparedRNSWeight,
    RNSRequestBatchWorkspace,
    RNSWorkspace,
    cuda_extension_available,
)
from .layers import (
    CachedRNSQKV,
    RNSLinear,
    RNSQKVProjection,
    install_opt_qkv_fusion,
)

__all__ = [
    "CudaRNSBackend",
    "PreparedRNSWeight",
    "PreparedAdaptiveRNSWeight",
    "RNSWorkspace",
    "RNSRequestBatchWorkspace",
    "cuda_extension_available",
    "RNSLinear",
    "RNSQKVProjection",
    "CachedRNSQKV",
    "install_opt_qkv_fusion",
]
