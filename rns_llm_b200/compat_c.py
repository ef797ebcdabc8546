"""Stand-in for the reference's compiled module ``rns_llm._C`` over librns_b200.so.

The reference's ``CudaRNSBackend`` calls six functions of its pybind11 module
(csrc/bindings.cpp:45-75 of the reference) with torch tensors.  ``RnsB200C`` offers the
same six names, argument orders, dtypes, shapes and result ownership on top of the C ABI
(include/rns_b200.h), so a maintainer who keeps the reference's Python backend swaps one
attribute::

    backend = rns_llm.backends.CudaRNSBackend()
    backend._C = rns_llm_b200.compat_c.RnsB200C()

This keeps the reference's plane-materialising pipeline (R bytes per weight value, int32
accumulators in HBM); the fused path of this package is reached through
``rns_llm_b200.backends.CudaRNSBackend`` instead.  Errors become ``RuntimeError`` with the
library's message, as ``TORCH_CHECK`` failures do in the reference.  The constants the
reference passes along (reciprocals, pairwise inverses, byte LUT, modulus product) are
accepted and ignored: the library derives its own from the moduli.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as N

_KIND = {torch.int8: N.INT8, torch.int16: N.INT16, torch.int32: N.INT32}


class RnsB200C:
    """The six functions of ``rns_llm._C``."""

    def __init__(self) -> None:
        self._lib = N.load()
        self._moduli_cache: dict[tuple[int, int], tuple] = {}

    # -- helpers ---------------------------------------------------------------
    def _mods(self, moduli: torch.Tensor):
        """Host copy of the reference's device tensor of moduli, fetched once per tensor
        (the reference caches one such tensor per (device, moduli))."""
        key = (moduli.data_ptr(), int(moduli.numel()))
        hit = self._moduli_cache.get(key)
        if hit is None:
            host = [int(v) for v in moduli.cpu().tolist()]
            hit = (N.moduli_array(host), len(host))
            self._moduli_cache[key] = hit
        return hit

    def _check(self, status: int) -> None:
        if status != N.OK:
            raise RuntimeError(N.last_error() or f"rns status {status}")

    @staticmethod
    def _require(cond: bool, message: str) -> None:
        if not cond:
            raise RuntimeError(message)

    @staticmethod
    def _stream(t: torch.Tensor) -> int:
        return int(torch.cuda.current_stream(t.device).cuda_stream)

    def _planes(self, t: torch.Tensor, name: str, dtype: torch.dtype, channels: int) -> None:
        self._require(t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous CUDA tensor")
        self._require(t.dtype == dtype, f"{name} must be {dtype}")
        self._require(t.ndim == 3 and t.shape[0] == channels, f"{name} must be [channels, rows, cols]")

    # -- bindings.cpp:46-49 ----------------------------------------------------
    def encode_int8(self, values: torch.Tensor, moduli: torch.Tensor) -> torch.Tensor:
        arr, r = self._mods(moduli)
        self._require(values.is_cuda and values.is_contiguous() and values.dtype == torch.int8,
                      "values must be a contiguous CUDA int8 tensor")
        out = torch.empty((r, *values.shape), dtype=torch.uint8, device=values.device)
        with torch.cuda.device(values.device):
            self._check(self._lib.rns_encode_canonical_i8(values.data_ptr(), values.numel(), arr, r,
                                                          out.data_ptr(), self._stream(values)))
        return out

    # -- bindings.cpp:51-54 ----------------------------------------------------
    def encode_centered(self, values: torch.Tensor, moduli: torch.Tensor) -> torch.Tensor:
        arr, r = self._mods(moduli)
        self._require(values.is_cuda and values.is_contiguous() and values.dtype in _KIND,
                      "values must be a contiguous CUDA int8/int16/int32 tensor")
        out = torch.empty((r, *values.shape), dtype=torch.int8, device=values.device)
        with torch.cuda.device(values.device):
            self._check(self._lib.rns_encode_centered(values.data_ptr(), _KIND[values.dtype], values.numel(), arr, r,
                                                      out.data_ptr(), self._stream(values)))
        return out

    # -- bindings.cpp:56-59 ----------------------------------------------------
    def matmul_residues(self, a: torch.Tensor, b: torch.Tensor, moduli: torch.Tensor, reciprocals: torch.Tensor,
                        kernel_id: int) -> torch.Tensor:
        arr, r = self._mods(moduli)
        self._planes(a, "a", torch.uint8, r)
        self._planes(b, "b", torch.uint8, r)
        self._require(a.shape[2] == b.shape[1], "K dimensions do not match")
        m, k, n = int(a.shape[1]), int(a.shape[2]), int(b.shape[2])
        out = torch.empty((r, m, n), dtype=torch.uint8, device=a.device)
        with torch.cuda.device(a.device):
            self._check(self._lib.rns_matmul_canonical_planes(a.data_ptr(), b.data_ptr(), arr, r, m, k, n,
                                                              int(kernel_id), out.data_ptr(), self._stream(a)))
        return out

    # -- bindings.cpp:61-64 ----------------------------------------------------
    def matmul_centered_residues(self, a: torch.Tensor, b: torch.Tensor, moduli: torch.Tensor,
                                 kernel_id: int) -> torch.Tensor:
        arr, r = self._mods(moduli)
        self._planes(a, "a", torch.int8, r)
        self._planes(b, "b", torch.int8, r)
        self._require(a.shape[2] == b.shape[1], "K dimensions do not match")
        m, k, n = int(a.shape[1]), int(a.shape[2]), int(b.shape[2])
        out = torch.empty((r, m, n), dtype=torch.int8, device=a.device)
        with torch.cuda.device(a.device):
            self._check(self._lib.rns_matmul_centered_planes(a.data_ptr(), b.data_ptr(), arr, r, m, k, n,
                                                             int(kernel_id), out.data_ptr(), self._stream(a)))
        return out

    # -- bindings.cpp:66-69 ----------------------------------------------------
    def decode_garner(self, residues: torch.Tensor, moduli: torch.Tensor, reciprocals: torch.Tensor,
                      pairwise_inverses: torch.Tensor, modulus_product: int) -> torch.Tensor:
        arr, r = self._mods(moduli)
        self._require(residues.is_cuda and residues.is_contiguous() and residues.dtype == torch.int8,
                      "residues must be a contiguous CUDA int8 tensor")
        self._require(residues.ndim >= 2 and residues.shape[0] == r, "residues must be [channels, ...]")
        out = torch.empty(tuple(residues.shape[1:]), dtype=torch.int64, device=residues.device)
        with torch.cuda.device(residues.device):
            self._check(self._lib.rns_decode_garner(residues.data_ptr(), out.numel(), arr, r, out.data_ptr(),
                                                    self._stream(residues)))
        return out

    # -- bindings.cpp:71-74 ----------------------------------------------------
    def matmul_centered_fused_out(self, a: torch.Tensor, b: torch.Tensor, moduli: torch.Tensor,
                                  reciprocals: torch.Tensor, pairwise_inverses: torch.Tensor, compact_lut: torch.Tensor,
                                  modulus_product: int, lut_channels: int, accumulators: torch.Tensor,
                                  output: torch.Tensor) -> torch.Tensor:
        """Writes the caller's ``accumulators`` (int32 [R,M,N]) and ``output`` (int64 [M,N])
        and returns ``output`` itself, as csrc/rns_cuda.cu:979 of the reference does."""
        arr, r = self._mods(moduli)
        self._planes(a, "a", torch.int8, r)
        self._planes(b, "b", torch.int8, r)
        self._require(a.shape[2] == b.shape[1], "K dimensions do not match")
        m, k, n = int(a.shape[1]), int(a.shape[2]), int(b.shape[2])
        self._require(accumulators.is_cuda and accumulators.is_contiguous() and accumulators.dtype == torch.int32 and
                      tuple(accumulators.shape) == (r, m, n), "accumulators must be contiguous int32 [channels, M, N]")
        self._require(output.is_cuda and output.is_contiguous() and output.dtype == torch.int64 and
                      tuple(output.shape) == (m, n), "output must be contiguous int64 [M, N]")
        with torch.cuda.device(a.device):
            self._check(self._lib.rns_matmul_centered_fused_out(a.data_ptr(), b.data_ptr(), arr, r, m, k, n,
                                                                int(lut_channels), accumulators.data_ptr(),
                                                                output.data_ptr(), self._stream(a)))
        return output
