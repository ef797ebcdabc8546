from .cuda_backend import (
    AdaptiveMetadata,
    CudaRNSBackend,
    PreparedAdaptiveRNSWeight,
    PreparedRNSWeight,
    RNSRequestBatchWorkspace,
    RNSWorkspace,
    cuda_extension_available,
)

__all__ = [
    "AdaptiveMetadata",
    "CudaRNSBackend",
    "PreparedRNSWeight",
    "PreparedAdaptiveRNSWeight",
    "RNSWorkspace",
    "RNSRequestBatchWorkspace",
    "cuda_extension_available",
]
