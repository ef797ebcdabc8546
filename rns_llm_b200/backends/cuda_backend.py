"""CudaRNSBackend for B200: the reference's backend contract over librns_b200.so.

Same public surface as ``src/rns_llm/backends/cuda_backend.py`` of the reference
(class, dataclasses, method names, argument meaning, exception classes, stats
keys), so code written against the reference backend runs unchanged.  What
differs is underneath:

* a prepared weight is the quantised int8 matrix in the nn.Linear layout
  [N,K], ONE byte per value; residue planes are formed inside the GEMM kernel
  (``PreparedRNSWeight.residues`` materialises [R,K,N] planes only when a
  caller asks for that attribute);
* ``matmul_prepared_fused`` is one kernel launch (encode, R tensor-core GEMMs,
  reduction, Garner, recentring) instead of encode + cuBLAS + Garner, with no
  int32 accumulator round trip through HBM;
* adaptive prefix selection happens on the device: no ``.item()`` on the hot
  path, metadata and per-channel-count statistics are read lazily;
* temporaries come from a per-stream arena.

Every computation goes through the C ABI; there is no PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
from collections import Counter
from collections.abc import Mapping
from dataclasses import dataclass, field
from math import prod
from typing import Iterable, Literal, Sequence

import torch

from .. import _native as N
from ..adaptive import minimal_prefix_channels, safe_l1_dot_bound
from ..arena import StreamArena
from ..moduli import (
    compact_byte_mod_lut,
    crt_constants,
    garner_pairwise_inverses,
    validate_moduli,
)

CanonicalKernelName = Literal["auto", "naive", "tiled", "tiled_safe"]
CenteredKernelName = Literal["auto", "scalar", "dp4a", "dp4a_safe", "cublas", "tcgen05", "planes"]

# Activations with at least this many rows are encoded to planes once by a
# separate kernel; below it every CTA encodes its own A tile inside the GEMM.
PLANES_MIN_ROWS = 512
# Where the two-CTA kernel covers the shape it also wins below that: from 320 rows on, and
# from 33 rows on when the weight is large (K*N >= 2^23; measured on 768 x 2304 and
# 4096 x 4096 / 12288 weights under graph replay).  At most 32 rows go to the one-launch kernel
# where it holds the residues of a token block in shared memory (K up to 1536 at four channels).
PAIR_MIN_ROWS = 320
STREAM_MAX_ROWS = 32         # few tokens beyond the one-launch kernel's K: the weight-streaming kernel
PAIR_LARGE_WEIGHT = 1 << 23
WIDE_MIN_ROWS = 128          # wide sources: fewer rows stay on the plane-level pipeline

_INT_TYPES = {torch.int8: N.INT8, torch.int16: N.INT16, torch.int32: N.INT32}
_FLOAT_TYPES = {torch.float16: N.F16, torch.bfloat16: N.BF16, torch.float32: N.F32}
_OUT_TYPES = {torch.int64: N.OUT_INT64, torch.int32: N.OUT_INT32, torch.float16: N.OUT_F16,
              torch.bfloat16: N.OUT_BF16, torch.float32: N.OUT_F32}


def cuda_extension_available() -> bool:
    """True when librns_b200.so has been built (reference: cuda_backend.py:40-45)."""
    return N.available()


def _load_extension():
    try:
        return N.load()
    except (RuntimeError, OSError, AttributeError) as exc:
        raise RuntimeError(
            "CUDA extension is not built. Run: python -m rns_llm_b200.csrc.build"
        ) from exc


class PreparedRNSWeight:
    """Cached Transformer weight ready for the RNS GEMM.

    Reference: ``PreparedRNSWeight`` (cuda_backend.py:68-76) holds residue
    planes [R,K,N], R bytes per value.  Here (kernel ``"tcgen05"``) the weight
    is kept ONCE, as the quantised int8 matrix in the packed tile layout the
    kernel's bulk copies read (``weight_packed``, one byte per value plus
    padding of N to 384 and K to 64); planes are never stored.  ``weight_nk``
    and ``residues`` rebuild the plain [N,K] matrix / the [R,K,N] planes on
    access for callers that read those attributes.  Sources wider than int8, or
    moduli the packed encoder cannot fold in one step, use the plane-level
    kernels and keep real planes as the reference does; where the two-CTA
    tensor-core kernel covers the shape (4..6 channels, K >= 512, K % 16 == 0)
    ``weight_planes_packed`` also holds those planes in the packed tile layout,
    one [N,K] matrix per channel ``weight_plane_stride`` bytes apart, for
    ``CudaRNSBackend.linear_forward_wide``.
    """

    def __init__(self, *, backend: "CudaRNSBackend", moduli: tuple[int, ...], k: int, n: int,
                 kernel: str, weight_packed: torch.Tensor | None = None,
                 residues: torch.Tensor | None = None,
                 weight_planes_packed: torch.Tensor | None = None, weight_plane_stride: int = 0) -> None:
        self._backend = backend
        self.moduli = moduli
        self.k = int(k)
        self.n = int(n)
        self.kernel = kernel
        self.weight_packed = weight_packed
        self._residues = residues
        self.weight_planes_packed = weight_planes_packed
        self.weight_plane_stride = int(weight_plane_stride)

    @property
    def weight_nk(self) -> torch.Tensor | None:
        """Plain int8 [N,K] copy of the packed weight (rebuilt on every access)."""
        if self.weight_packed is None:
            return None
        return self._backend._unpack_weight(self.weight_packed, self.n, self.k)

    @property
    def residues(self) -> torch.Tensor:
        if self._residues is None:
            kn = self.weight_nk.t().contiguous()
            return self._backend._encode_centered_raw(kn, self.moduli)
        return self._residues

    @property
    def device(self) -> torch.device:
        return (self.weight_packed if self.weight_packed is not None else self._residues).device

    def prefix(self, channels: int, kernel: str) -> "PreparedRNSWeight":
        """The same weight restricted to the first ``channels`` moduli (no copy)."""
        return PreparedRNSWeight(
            backend=self._backend, moduli=self.moduli[:channels], k=self.k, n=self.n, kernel=kernel,
            weight_packed=self.weight_packed,
            residues=None if self._residues is None else self._residues[:channels],
            weight_planes_packed=self.weight_planes_packed, weight_plane_stride=self.weight_plane_stride,
        )


@dataclass
class RNSWorkspace:
    """Reusable output memory for one shape/stream/request (cuda_backend.py:79-88).

    ``accumulators`` ([R,M,N] int32) exists only for the plane-level pipeline; the
    fused kernel keeps its accumulators in tensor memory and needs ``output`` only.
    """

    accumulators: torch.Tensor | None
    output: torch.Tensor
    channels: int
    m: int
    n: int


@dataclass(frozen=True)
class PreparedAdaptiveRNSWeight:
    """One prepared weight with its safe prefix variants (cuda_backend.py:90-97)."""

    variants: dict[int, PreparedRNSWeight]
    full_moduli: tuple[int, ...]
    max_abs_weight: int
    min_channels: int


@dataclass
class RNSRequestBatchWorkspace:
    """Preallocated merged-activation buffer plus output (cuda_backend.py:100-107)."""

    activations: torch.Tensor
    fused: RNSWorkspace
    rows_per_request: tuple[int, ...]
    k: int
    _offsets: tuple[int, ...] = field(default=(), repr=False)


class AdaptiveMetadata(Mapping):
    """``{"channels", "bound", "capacity"}`` of one adaptive call.

    The reference returns Python ints, which costs a device-to-host sync per
    call (cuda_backend.py:591, 617-621).  Here the three numbers stay in a
    device tensor and are fetched the first time a key is read.
    """

    _KEYS = ("channels", "bound", "capacity")

    def __init__(self, device_values: torch.Tensor) -> None:
        self._device_values = device_values
        self._host: dict[str, int] | None = None

    def _fetch(self) -> dict[str, int]:
        if self._host is None:
            values = self._device_values.cpu().tolist()
            self._host = dict(zip(self._KEYS, (int(v) for v in values)))
            self._device_values = None
        return self._host

    def __getitem__(self, key: str) -> int:
        return self._fetch()[key]

    def __iter__(self):
        return iter(self._KEYS)

    def __len__(self) -> int:
        return 3

    def __repr__(self) -> str:
        return f"AdaptiveMetadata({self._fetch()!r})"


@dataclass
class _DeviceState:
    status: torch.Tensor          # int32 [1]: device-side error word
    wait_info: torch.Tensor       # int32 [4]: which bounded wait expired (see rns_linear_args.d_wait_info)
    histogram: torch.Tensor       # int64 [MAX_CHANNELS+1]: adaptive selections per channel count


class CudaRNSBackend:
    """RNS backend over hand-written sm_100a kernels (one process per GPU)."""

    name = "cuda-rns-b200"

    def __init__(self) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is not available in this PyTorch installation")
        self._lib = _load_extension()
        self._stats: Counter[str] = Counter()
        self._device_state: dict[int, _DeviceState] = {}
        self._moduli_arrays: dict[tuple[int, ...], C.Array] = {}
        self.arena = StreamArena()

    # ------------------------------------------------------------------
    # plumbing
    # ------------------------------------------------------------------
    def _mods(self, moduli: Iterable[int]) -> tuple[tuple[int, ...], C.Array]:
        # a tuple that has been validated once is looked up, not validated again
        if isinstance(moduli, tuple):
            arr = self._moduli_arrays.get(moduli)
            if arr is not None:
                return moduli, arr
        mods = validate_moduli(moduli)
        arr = self._moduli_arrays.get(mods)
        if arr is None:
            arr = N.moduli_array(mods)
            self._moduli_arrays[mods] = arr
        return mods, arr

    @staticmethod
    def _stream(device: torch.device) -> int:
        return int(torch.cuda.current_stream(device).cuda_stream)

    def _state(self, device: torch.device) -> _DeviceState:
        index = device.index if device.index is not None else torch.cuda.current_device()
        state = self._device_state.get(index)
        if state is None:
            dev = torch.device("cuda", index)
            state = _DeviceState(
                status=torch.zeros(1, dtype=torch.int32, device=dev),
                wait_info=torch.zeros(4, dtype=torch.int32, device=dev),
                histogram=torch.zeros(N.MAX_CHANNELS + 1, dtype=torch.int64, device=dev),
            )
            self._device_state[index] = state
        return state

    def reset_stats(self) -> None:
        self._stats.clear()
        for state in self._device_state.values():
            state.histogram.zero_()

    def stats_snapshot(self) -> dict[str, int]:
        """Counters with the reference's keys (cuda_backend.py:129-135).  The
        ``adaptive_channels_{c}`` entries live on the device and are read here."""
        snapshot = dict(self._stats)
        for state in self._device_state.values():
            for channels, count in enumerate(state.histogram.cpu().tolist()):
                if count:
                    key = f"adaptive_channels_{channels}"
                    snapshot[key] = snapshot.get(key, 0) + int(count)
        return snapshot

    def check_status(self) -> None:
        """Raises if a kernel recorded a device-side failure (bounded wait expired,
        or an adaptive bound beyond the full set's capacity).  Synchronises."""
        for state in self._device_state.values():
            code = int(state.status.item())
            if code == N.ERR_OVERFLOW:
                state.status.zero_()
                raise OverflowError("full moduli set cannot represent the activation bound")
            if code != N.OK:
                where = [int(v) for v in state.wait_info.cpu().tolist()]
                state.status.zero_()
                state.wait_info.zero_()
                detail = ""
                if code == N.ERR_DEVICE_TIMEOUT and where[0]:
                    detail = (f": bounded wait expired (role {where[0] >> 20}, stage {where[0] & 0xfffff}, "
                              f"CTA ({where[1]}, {where[2]}), kernel form {where[3]})")
                raise RuntimeError(f"RNS kernel reported device status {code}{detail}")

    @staticmethod
    def _validate_matrix(matrix: torch.Tensor, name: str, ndim: int) -> None:
        if not matrix.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor")
        if matrix.ndim != ndim:
            raise ValueError(f"{name} must have rank {ndim}")
        if not matrix.is_contiguous():
            raise ValueError(f"{name} must be contiguous")

    # ------------------------------------------------------------------
    # Encoding
    # ------------------------------------------------------------------
    def encode(self, values: torch.Tensor, moduli: Iterable[int]) -> torch.Tensor:
        """Canonical [0,m) uint8 planes (cuda_backend.py:177-184)."""
        self._validate_matrix(values, "values", values.ndim)
        if values.dtype != torch.int8:
            raise ValueError("canonical CUDA encoder currently expects torch.int8")
        mods, arr = self._mods(moduli)
        out = torch.empty((len(mods), *values.shape), dtype=torch.uint8, device=values.device)
        with torch.cuda.device(values.device):
            N.check(self._lib.rns_encode_canonical_i8(values.data_ptr(), values.numel(), arr, len(mods),
                                                      out.data_ptr(), self._stream(values.device)))
        return out

    def _encode_centered_raw(self, values: torch.Tensor, moduli: Iterable[int]) -> torch.Tensor:
        mods, arr = self._mods(moduli)
        out = torch.empty((len(mods), *values.shape), dtype=torch.int8, device=values.device)
        with torch.cuda.device(values.device):
            N.check(self._lib.rns_encode_centered(values.data_ptr(), _INT_TYPES[values.dtype],
                                                  values.numel(), arr, len(mods), out.data_ptr(),
                                                  self._stream(values.device)))
        return out

    def encode_centered(self, values: torch.Tensor, moduli: Iterable[int]) -> torch.Tensor:
        """int8/int16/int32 -> centred int8 planes [R,*shape] (cuda_backend.py:186-200)."""
        self._validate_matrix(values, "values", values.ndim)
        if values.dtype not in _INT_TYPES:
            raise ValueError("centered encoder supports int8, int16 and int32")
        self._stats["encode_centered_calls"] += 1
        self._stats["encode_centered_values"] += int(values.numel())
        return self._encode_centered_raw(values, moduli)

    # ------------------------------------------------------------------
    # Bounds and selection (cuda_backend.py:205-261)
    # ------------------------------------------------------------------
    @staticmethod
    def accumulator_bound(k: int, moduli: Iterable[int]) -> int:
        return int(k) * (max(validate_moduli(moduli)) - 1) ** 2

    @staticmethod
    def centered_accumulator_bound(k: int, moduli: Iterable[int]) -> int:
        return int(k) * max(m // 2 for m in validate_moduli(moduli)) ** 2

    def select_kernel(self, k: int, moduli: Iterable[int], requested: CanonicalKernelName) -> str:
        if requested != "auto":
            return requested
        return "tiled" if self.accumulator_bound(k, moduli) <= 0xFFFFFFFF else "tiled_safe"

    def cublas_compatible(self, *, k: int, n: int, moduli: Iterable[int], device: torch.device) -> bool:
        """Shape test of the reference's fused path (cuda_backend.py:224-239):
        K and N multiples of 4, 2..10 channels, int32-safe accumulators.  Kept
        because plane-level callers rely on it; see ``tensor_core_compatible``
        for the kernel this backend prefers."""
        return (
            k % 4 == 0
            and n % 4 == 0
            and 2 <= len(validate_moduli(moduli)) <= 10
            and self.centered_accumulator_bound(k, moduli) <= 0x7FFFFFFF
        )

    def tensor_core_compatible(self, *, k: int, moduli: Iterable[int]) -> bool:
        """True when int8 sources with this K and these moduli run on the
        tcgen05 kernel: K % 16 == 0, 2..8 channels, int32-safe channel sums."""
        mods, arr = self._mods(moduli)
        return bool(self._lib.rns_linear_fused_supported(arr, len(mods), int(k), int(k), int(k))) and (
            int(k) * 128 * 128 <= 0x7FFFFFFF
        )

    def select_centered_kernel(self, *, k: int, n: int, moduli: Iterable[int],
                               requested: CenteredKernelName, device: torch.device) -> str:
        if requested != "auto":
            return requested
        if self.cublas_compatible(k=k, n=n, moduli=moduli, device=device):
            return "cublas"
        if self.centered_accumulator_bound(k, moduli) <= 0x7FFFFFFF:
            return "dp4a"
        return "dp4a_safe"

    # ------------------------------------------------------------------
    # Plane-level GEMMs (cuda_backend.py:266-459)
    # ------------------------------------------------------------------
    def matmul_residues(self, a_residues: torch.Tensor, b_residues: torch.Tensor,
                        moduli: Iterable[int], *, kernel: CanonicalKernelName = "auto") -> torch.Tensor:
        self._validate_matrix(a_residues, "a_residues", 3)
        self._validate_matrix(b_residues, "b_residues", 3)
        if a_residues.dtype != torch.uint8 or b_residues.dtype != torch.uint8:
            raise ValueError("canonical residue matrices must use torch.uint8")
        if a_residues.device != b_residues.device:
            raise ValueError("a_residues and b_residues must be on the same device")
        if a_residues.shape[0] != b_residues.shape[0]:
            raise ValueError("residue channel counts do not match")
        if a_residues.shape[2] != b_residues.shape[1]:
            raise ValueError("K dimensions do not match")
        mods, arr = self._mods(moduli)
        if a_residues.shape[0] != len(mods):
            raise ValueError("tensor channel count does not match moduli")
        selected = self.select_kernel(a_residues.shape[2], mods, kernel)
        kernel_id = {"naive": 0, "tiled": 1, "tiled_safe": 2}[selected]
        r, m, k = map(int, a_residues.shape)
        n = int(b_residues.shape[2])
        out = torch.empty((r, m, n), dtype=torch.uint8, device=a_residues.device)
        with torch.cuda.device(a_residues.device):
            N.check(self._lib.rns_matmul_canonical_planes(
                a_residues.data_ptr(), b_residues.data_ptr(), arr, r, m, k, n, kernel_id,
                out.data_ptr(), self._stream(a_residues.device)))
        return out

    def _check_centered_planes(self, a_residues, b_residues, moduli):
        self._validate_matrix(a_residues, "a_residues", 3)
        self._validate_matrix(b_residues, "b_residues", 3)
        if a_residues.dtype != torch.int8 or b_residues.dtype != torch.int8:
            raise ValueError("centered residue matrices must use torch.int8")
        if a_residues.device != b_residues.device:
            raise ValueError("a_residues and b_residues must share a device")
        if a_residues.shape[0] != b_residues.shape[0]:
            raise ValueError("channel counts do not match")
        if a_residues.shape[2] != b_residues.shape[1]:
            raise ValueError("K dimensions do not match")
        mods, arr = self._mods(moduli)
        if len(mods) != a_residues.shape[0]:
            raise ValueError("moduli count does not match residue channels")
        return mods, arr

    def matmul_centered_residues(self, a_residues: torch.Tensor, b_residues: torch.Tensor,
                                 moduli: Iterable[int], *, kernel: CenteredKernelName = "auto") -> torch.Tensor:
        mods, arr = self._check_centered_planes(a_residues, b_residues, moduli)
        r, m, k = map(int, a_residues.shape)
        n = int(b_residues.shape[2])
        selected = self.select_centered_kernel(k=k, n=n, moduli=mods, requested=kernel,
                                               device=a_residues.device)
        if selected == "cublas" and not self.cublas_compatible(k=k, n=n, moduli=mods,
                                                               device=a_residues.device):
            raise ValueError("cuBLAS path constraints are not satisfied")
        kernel_id = {"scalar": 0, "dp4a": 1, "dp4a_safe": 2, "cublas": 3}.get(selected)
        if kernel_id is None:
            raise ValueError(f"unknown centered kernel: {selected}")
        out = torch.empty((r, m, n), dtype=torch.int8, device=a_residues.device)
        with torch.cuda.device(a_residues.device):
            N.check(self._lib.rns_matmul_centered_planes(
                a_residues.data_ptr(), b_residues.data_ptr(), arr, r, m, k, n, kernel_id,
                out.data_ptr(), self._stream(a_residues.device)))
        return out

    def decode_garner(self, residues: torch.Tensor, moduli: Iterable[int]) -> torch.Tensor:
        self._validate_matrix(residues, "residues", residues.ndim)
        if residues.dtype != torch.int8:
            raise ValueError("Garner decoder expects centered int8 residues")
        if residues.ndim < 2:
            raise ValueError("residues must have shape [R,...]")
        mods, arr = self._mods(moduli)
        if residues.shape[0] != len(mods):
            raise ValueError("moduli count mismatch")
        out = torch.empty(residues.shape[1:], dtype=torch.int64, device=residues.device)
        with torch.cuda.device(residues.device):
            N.check(self._lib.rns_decode_garner(residues.data_ptr(), out.numel(), arr, len(mods),
                                                out.data_ptr(), self._stream(residues.device)))
        return out

    def create_workspace(self, *, device: torch.device, channels: int, m: int, n: int,
                         with_accumulators: bool = False) -> RNSWorkspace:
        """Output memory for one shape (cuda_backend.py:366-380).  The int32
        accumulator planes of the reference are allocated only on request or
        when a plane-level call first needs them."""
        return RNSWorkspace(
            accumulators=torch.empty((channels, m, n), dtype=torch.int32, device=device)
            if with_accumulators else None,
            output=torch.empty((m, n), dtype=torch.int64, device=device),
            channels=int(channels), m=int(m), n=int(n),
        )

    @staticmethod
    def _check_workspace(workspace: RNSWorkspace, *, channels: int, m: int, n: int,
                         device: torch.device) -> None:
        if (workspace.channels, workspace.m, workspace.n) != (channels, m, n):
            raise ValueError("workspace shape does not match operation")
        if workspace.output.device != device:
            raise ValueError("workspace device does not match operation")

    def matmul_centered_fused(self, a_residues: torch.Tensor, b_residues: torch.Tensor,
                              moduli: Iterable[int], *, lut_channels: int = 0,
                              workspace: RNSWorkspace | None = None) -> torch.Tensor:
        """Plane-level fused call: planes [R,M,K] x [R,K,N] -> int64 [M,N]
        (cuda_backend.py:398-459).  For callers that already hold planes; the
        hot path is ``matmul_prepared_fused``."""
        if a_residues.dtype != torch.int8 or b_residues.dtype != torch.int8:
            raise ValueError("fused path expects centered int8 residue planes")
        if a_residues.ndim == 3 and b_residues.ndim == 3 and (
            a_residues.shape[0] != b_residues.shape[0] or a_residues.shape[2] != b_residues.shape[1]
        ):
            raise ValueError("R/K dimensions do not match")
        if lut_channels not in (0, 1, 2):
            raise ValueError("lut_channels must be 0, 1 or 2")
        mods, arr = self._check_centered_planes(a_residues, b_residues, moduli)
        r, m, k = map(int, a_residues.shape)
        n = int(b_residues.shape[2])
        if not self.cublas_compatible(k=k, n=n, moduli=mods, device=a_residues.device):
            raise ValueError("fused path requires a cuBLAS-compatible shape/device")
        if workspace is None:
            workspace = self.create_workspace(device=a_residues.device, channels=r, m=m, n=n,
                                              with_accumulators=True)
        self._check_workspace(workspace, channels=r, m=m, n=n, device=a_residues.device)
        if workspace.accumulators is None:
            workspace.accumulators = torch.empty((r, m, n), dtype=torch.int32, device=a_residues.device)
        self._stats["fused_gemm_calls"] += 1
        self._stats[f"fused_gemm_channels_{r}"] += 1
        with torch.cuda.device(a_residues.device):
            N.check(self._lib.rns_matmul_centered_fused_out(
                a_residues.data_ptr(), b_residues.data_ptr(), arr, r, m, k, n, min(lut_channels, r),
                workspace.accumulators.data_ptr(), workspace.output.data_ptr(),
                self._stream(a_residues.device)))
        return workspace.output

    # ------------------------------------------------------------------
    # Prepared weights
    # ------------------------------------------------------------------
    def prepare_weight(self, b: torch.Tensor, moduli: Iterable[int]) -> PreparedRNSWeight:
        """``b`` is [K,N] as in the reference (cuda_backend.py:464-487)."""
        self._validate_matrix(b, "b", 2)
        if b.dtype not in _INT_TYPES:
            raise ValueError("prepared weights support int8/int16/int32")
        mods, _ = self._mods(moduli)
        k, n = int(b.shape[0]), int(b.shape[1])
        if b.dtype == torch.int8 and self.tensor_core_compatible(k=k, moduli=mods):
            return self.prepare_weight_nk(b.t(), mods)
        residues = self.encode_centered(b.contiguous(), mods)
        kernel = self.select_centered_kernel(k=k, n=n, moduli=mods, requested="auto", device=b.device)
        planes_packed, stride = None, 0
        if (b.dtype != torch.int8 and int(self._lib.rns_pair_tile_rows(len(mods), k)) > 0
                and self.tensor_core_compatible(k=k, moduli=mods)):
            # Wide sources on the tensor cores: the same centred planes once more, each as a
            # packed [N,K] matrix (R bytes per value; the reference caches 4 R bytes per value).
            nbytes = int(self._lib.rns_packed_weight_bytes(n, k))
            stride = (nbytes + 255) & ~255
            planes_packed = torch.zeros(len(mods) * stride, dtype=torch.int8, device=b.device)
            for channel in range(len(mods)):
                planes_packed[channel * stride: channel * stride + nbytes].copy_(
                    self._pack_weight(residues[channel].t()))
        return PreparedRNSWeight(backend=self, moduli=mods, k=k, n=n, kernel=kernel, residues=residues,
                                 weight_planes_packed=planes_packed, weight_plane_stride=stride)

    def _pack_weight(self, w: torch.Tensor) -> torch.Tensor:
        n, k = int(w.shape[0]), int(w.shape[1])
        if w.stride(1) != 1 or (w.stride(0) % 16) or (w.data_ptr() % 16):
            w = w.contiguous()
        packed = torch.empty(int(self._lib.rns_packed_weight_bytes(n, k)), dtype=torch.int8, device=w.device)
        with torch.cuda.device(w.device):
            N.check(self._lib.rns_pack_weight(w.data_ptr(), n, k, w.stride(0), packed.data_ptr(),
                                              self._stream(w.device)))
        return packed

    def _unpack_weight(self, packed: torch.Tensor, n: int, k: int) -> torch.Tensor:
        w = torch.empty((n, k), dtype=torch.int8, device=packed.device)
        with torch.cuda.device(packed.device):
            N.check(self._lib.rns_unpack_weight(packed.data_ptr(), n, k, w.data_ptr(), k,
                                                self._stream(packed.device)))
        return w

    def prepare_weight_nk(self, w: torch.Tensor, moduli: Iterable[int]) -> PreparedRNSWeight:
        """``w`` is int8 [N,K] (the nn.Linear layout; any row stride).  The
        prepared weight is its packed copy; ``w`` itself is not kept."""
        if not w.is_cuda:
            raise ValueError("w must be a CUDA tensor")
        if w.ndim != 2:
            raise ValueError("w must have rank 2")
        if w.dtype != torch.int8:
            raise ValueError("prepare_weight_nk expects int8")
        mods, _ = self._mods(moduli)
        n, k = int(w.shape[0]), int(w.shape[1])
        if not self.tensor_core_compatible(k=k, moduli=mods):
            return self.prepare_weight(w.t().contiguous(), mods)
        return PreparedRNSWeight(backend=self, moduli=mods, k=k, n=n, kernel="tcgen05",
                                 weight_packed=self._pack_weight(w))

    def _check_activation(self, a: torch.Tensor, prepared: PreparedRNSWeight) -> None:
        self._validate_matrix(a, "a", 2)
        if a.dtype not in _INT_TYPES:
            raise ValueError("a must be int8/int16/int32")
        if int(a.shape[1]) != prepared.k:
            raise ValueError("K dimension does not match prepared weight")
        if a.device != prepared.device:
            raise ValueError("activation and prepared weight must share device")

    def matmul_prepared(self, a: torch.Tensor, prepared_weight: PreparedRNSWeight, *,
                        decode: bool = True, kernel: CenteredKernelName = "auto") -> torch.Tensor:
        """Unfused path of the reference (cuda_backend.py:489-512): encode, plane
        GEMM to centred residues, CRT decode."""
        self._check_activation(a, prepared_weight)
        a_residues = self.encode_centered(a.contiguous(), prepared_weight.moduli)
        if kernel in ("tcgen05", "planes"):
            kernel = "auto"
        result = self.matmul_centered_residues(a_residues, prepared_weight.residues,
                                               prepared_weight.moduli, kernel=kernel)
        return self.decode(result, prepared_weight.moduli) if decode else result

    def _launch_fused(self, *, prepared: PreparedRNSWeight, m: int, a: torch.Tensor | None,
                      a_planes: torch.Tensor | None, out: torch.Tensor, a_packed: bool = False,
                      active: torch.Tensor | None = None, row_scale: torch.Tensor | None = None,
                      row_scale_stride: int = 0, col_scale: torch.Tensor | None = None,
                      bias: torch.Tensor | None = None, tile_n: int = 0, tile_k: int = 0,
                      plain_weight: torch.Tensor | None = None, pair_mode: int = 2,
                      enc_groups: int = 0, exact_residues: bool = False,
                      enc_stages: int = 0, sub_blocks: int = 0, variant: int = 0,
                      stream: int | None = None, a_tile_rows: int = 0,
                      absmax_out: torch.Tensor | int | None = None,
                      out_copies: Sequence[int] = (), absmax_copies: Sequence[int] = (),
                      weight_planes: bool = False, copies_multicast: bool = False, groups: int = 0,
                      packed_weight: torch.Tensor | None = None) -> None:
        """Fills ``rns_linear_args`` and launches.  ``a`` / ``a_planes`` are plain
        ([M,K] / [R,M,K]) unless ``a_packed``; the weight is the prepared packed
        copy unless ``plain_weight`` ([N,K] int8) is given.  Device buffers may be
        given as tensors or as raw addresses (ints)."""
        def ptr(t):
            return t if isinstance(t, int) else t.data_ptr()
        mods = prepared.moduli
        args = N.LinearArgs()
        args.m, args.n, args.k = m, prepared.n, prepared.k
        args.channels = len(mods)
        for i, mod in enumerate(mods):
            args.moduli[i] = mod
        if a_planes is not None:
            args.d_a_planes = ptr(a_planes)
            args.lda = prepared.k
            args.a_plane_stride = m * prepared.k
        else:
            args.d_a = ptr(a)
            args.lda = prepared.k if a_packed else a.stride(0)
        args.a_packed = 1 if a_packed else 0
        args.groups = int(groups)
        if packed_weight is not None:
            args.d_w = packed_weight.data_ptr()
            args.ldw = prepared.k
            args.w_packed = 1
            device = packed_weight.device
        elif weight_planes:
            args.d_w = prepared.weight_planes_packed.data_ptr()
            args.ldw = prepared.k
            args.w_packed = 1
            args.w_channel_stride = prepared.weight_plane_stride
            device = prepared.weight_planes_packed.device
        elif plain_weight is not None:
            args.d_w = plain_weight.data_ptr()
            args.ldw = plain_weight.stride(0)
            device = plain_weight.device
        else:
            args.d_w = prepared.weight_packed.data_ptr()
            args.ldw = prepared.k
            args.w_packed = 1
            device = prepared.weight_packed.device
        args.d_active_channels = None if active is None else ptr(active)
        args.d_out = out.data_ptr()
        args.ldo = out.stride(0)
        args.out_type = _OUT_TYPES[out.dtype]
        if row_scale is not None:
            args.d_row_scale = ptr(row_scale)
            args.row_scale_stride = row_scale_stride
            args.d_col_scale = col_scale.data_ptr()
            args.d_bias = None if bias is None else bias.data_ptr()
        state = self._state(device)
        args.d_status = state.status.data_ptr()
        args.d_wait_info = state.wait_info.data_ptr()
        args.tile_n, args.tile_k = tile_n, tile_k
        args.pair_mode = pair_mode
        args.enc_groups = enc_groups
        args.exact_residues = 1 if exact_residues else 0
        args.enc_stages = enc_stages
        args.sub_blocks = sub_blocks
        args.variant = variant
        args.a_tile_rows = a_tile_rows
        args.d_absmax_out = None if absmax_out is None else ptr(absmax_out)
        args.n_out_copies = len(out_copies)
        args.out_copies_multicast = 1 if copies_multicast else 0
        for index, address in enumerate(out_copies):
            args.d_out_copies[index] = address
        for index, address in enumerate(absmax_copies):
            args.d_absmax_copies[index] = address
        N.check(self._lib.rns_linear_fused(C.byref(args), self._stream(device) if stream is None else stream))

    def matmul_prepared_fused(self, a: torch.Tensor, prepared_weight: PreparedRNSWeight, *,
                              lut_channels: int = 0, workspace: RNSWorkspace | None = None,
                              _active: torch.Tensor | None = None) -> torch.Tensor:
        """Quantised activations [M,K] x prepared weight -> exact int64 [M,N]
        (cuda_backend.py:514-539).  The result aliases ``workspace.output``."""
        self._check_activation(a, prepared_weight)
        if lut_channels not in (0, 1, 2):
            raise ValueError("lut_channels must be 0, 1 or 2")
        mods = prepared_weight.moduli
        channels = len(mods)
        m = int(a.shape[0])
        if prepared_weight.kernel != "tcgen05" or a.dtype != torch.int8:
            if prepared_weight.kernel not in ("tcgen05", "cublas"):
                raise ValueError("fused prepared path currently requires cuBLAS-compatible weight")
            a_residues = self.encode_centered(a.contiguous(), mods)
            return self.matmul_centered_fused(a_residues, prepared_weight.residues, mods,
                                              lut_channels=lut_channels, workspace=workspace)
        if workspace is None:
            workspace = self.create_workspace(device=a.device, channels=channels, m=m,
                                              n=prepared_weight.n)
        self._check_workspace(workspace, channels=channels, m=m, n=prepared_weight.n, device=a.device)
        self._stats["encode_centered_calls"] += 1
        self._stats["encode_centered_values"] += int(a.numel())
        self._stats["fused_gemm_calls"] += 1
        self._stats[f"fused_gemm_channels_{channels}"] += 1
        with torch.cuda.device(a.device):
            if (_active is None and a.stride(1) == 1 and
                    self._lib.rns_linear_small_supported(m, prepared_weight.k, channels)):
                # Few tokens (merged single-token requests): one launch, no scratch.
                _, arr = self._mods(mods)
                N.check(self._lib.rns_linear_small(
                    a.data_ptr(), -1, m, prepared_weight.k, a.stride(0), 0, prepared_weight.weight_packed.data_ptr(),
                    prepared_weight.n, arr, channels, None, None, workspace.output.data_ptr(),
                    workspace.output.stride(0), N.OUT_INT64, self._stream(a.device)))
            elif m >= PLANES_MIN_ROWS or self._pair_tile_rows(m, prepared_weight.k, prepared_weight.n, channels):
                frame = self.arena.frame(a.device)
                _, arr = self._mods(mods)
                # tiles of 64 / 48 / 32 rows for the two-CTA kernel where it covers the call
                # (an adaptive prefix: 4 or 5 channels), else the 128-row layout
                tile_rows = self._pair_tile_rows(m, prepared_weight.k, prepared_weight.n, channels)
                if _active is not None and channels > 5:
                    tile_rows = 0
                if tile_rows:
                    planes = frame.alloc(int(self._lib.rns_packed_planes_bytes(m, prepared_weight.k, channels,
                                                                               tile_rows)), torch.int8)
                    N.check(self._lib.rns_encode_planes_tiled(a.data_ptr(), m, prepared_weight.k, a.stride(0),
                                                              arr, channels, tile_rows, planes.data_ptr(),
                                                              self._stream(a.device)))
                else:
                    planes = frame.alloc(int(self._lib.rns_packed_activation_bytes(m, prepared_weight.k,
                                                                                   channels)), torch.int8)
                    N.check(self._lib.rns_encode_planes_packed(a.data_ptr(), m, prepared_weight.k, a.stride(0),
                                                               arr, channels, planes.data_ptr(),
                                                               self._stream(a.device)))
                self._launch_fused(prepared=prepared_weight, m=m, a=None, a_planes=planes, a_packed=True,
                                   out=workspace.output, active=_active, a_tile_rows=tile_rows)
            else:
                self._launch_fused(prepared=prepared_weight, m=m, a=a, a_planes=None,
                                   out=workspace.output, active=_active)
        return workspace.output

    # ------------------------------------------------------------------
    # Adaptive channel prefix (cuda_backend.py:541-622)
    # ------------------------------------------------------------------
    def prepare_weight_adaptive(self, b: torch.Tensor, moduli: Iterable[int], *,
                                min_channels: int = 3) -> PreparedAdaptiveRNSWeight:
        full = self.prepare_weight(b, moduli)
        return self._adaptive_from_full(full, int(b.to(torch.int32).abs().max().item()), min_channels)

    def _adaptive_from_full(self, full: PreparedRNSWeight, max_abs_weight: int,
                            min_channels: int) -> PreparedAdaptiveRNSWeight:
        if not 2 <= min_channels <= len(full.moduli):
            raise ValueError("min_channels must be between 2 and full channel count")
        variants: dict[int, PreparedRNSWeight] = {}
        for channels in range(min_channels, len(full.moduli) + 1):
            if full.kernel == "tcgen05":
                kernel = "tcgen05"
            else:
                kernel = self.select_centered_kernel(k=full.k, n=full.n, moduli=full.moduli[:channels],
                                                     requested="auto", device=full.device)
            variants[channels] = full if channels == len(full.moduli) else full.prefix(channels, kernel)
        return PreparedAdaptiveRNSWeight(variants=variants, full_moduli=full.moduli,
                                         max_abs_weight=int(max_abs_weight), min_channels=int(min_channels))

    def select_adaptive_variant(self, a: torch.Tensor, prepared: PreparedAdaptiveRNSWeight
                                ) -> tuple[PreparedRNSWeight, int]:
        """Host-side selection with the reference's signature and its
        device-to-host synchronisation (cuda_backend.py:573-601).  The hot path
        (``matmul_prepared_adaptive_fused``) does not call this."""
        self._validate_matrix(a, "a", 2)
        if a.dtype not in _INT_TYPES:
            raise ValueError("a must be int8/int16/int32")
        max_row_l1 = int(a.to(torch.int32).abs().sum(dim=1).max().item())
        bound = safe_l1_dot_bound(max_row_l1, prepared.max_abs_weight)
        channels = minimal_prefix_channels(prepared.full_moduli, bound, min_channels=prepared.min_channels)
        self._stats["adaptive_selections"] += 1
        self._stats[f"adaptive_channels_{channels}"] += 1
        return prepared.variants[channels], bound

    def matmul_prepared_adaptive_fused(self, a: torch.Tensor, prepared: PreparedAdaptiveRNSWeight, *,
                                       lut_channels: int = 2,
                                       workspace_by_channels: dict[int, RNSWorkspace] | None = None,
                                       return_metadata: bool = False):
        """Adaptive prefix, decided on the device: row-L1 maximum, safe bound,
        smallest sufficient prefix and the GEMM that uses it are all queued
        without a host round trip.  An activation bound beyond the full set's
        capacity (``OverflowError`` in the reference, adaptive.py:38-41) sets
        the device status word; ``check_status()`` raises it."""
        full = prepared.variants[len(prepared.full_moduli)]
        self._check_activation(a, full)
        if full.kernel != "tcgen05" or a.dtype != torch.int8:
            variant, bound = self.select_adaptive_variant(a, prepared)
            workspace = None if workspace_by_channels is None else workspace_by_channels.get(len(variant.moduli))
            output = self.matmul_prepared_fused(a, variant, lut_channels=lut_channels, workspace=workspace)
            if return_metadata:
                return output, {"channels": len(variant.moduli), "bound": bound,
                                "capacity": (prod(variant.moduli) - 1) // 2}
            return output
        mods, arr = self._mods(prepared.full_moduli)
        channels = len(mods)
        m = int(a.shape[0])
        device = a.device
        state = self._state(device)
        workspace = None
        if workspace_by_channels is not None:
            # Any workspace of the right [M,N] serves: the kernel keeps no per-channel memory.
            workspace = workspace_by_channels.get(channels) or next(iter(workspace_by_channels.values()), None)
            if workspace is not None and (workspace.m, workspace.n) != (m, full.n):
                raise ValueError("workspace shape does not match operation")
        out = workspace.output if workspace is not None else torch.empty(
            (m, full.n), dtype=torch.int64, device=device)
        with torch.cuda.device(device):
            frame = self.arena.frame(device)
            scratch = frame.alloc(8, torch.int32)          # [0] row-L1 max, [1] active channels
            meta = torch.empty(3, dtype=torch.int64, device=device) if return_metadata else None
            stream = self._stream(device)
            N.check(self._lib.rns_row_l1_max_i8(a.data_ptr(), m, full.k, a.stride(0),
                                                scratch.data_ptr(), stream))
            N.check(self._lib.rns_select_channels(
                scratch.data_ptr(), prepared.max_abs_weight, arr, channels, prepared.min_channels,
                scratch.data_ptr() + 4, None if meta is None else meta.data_ptr(),
                state.histogram.data_ptr(), state.status.data_ptr(), stream))
            active = scratch[1:2]
            self._stats["adaptive_selections"] += 1
            self._stats["encode_centered_calls"] += 1
            self._stats["encode_centered_values"] += int(a.numel())
            self._stats["fused_gemm_calls"] += 1
            tile_rows = 0
            if channels <= 5 and a.stride(1) == 1:
                tile_rows = self._pair_tile_rows(m, full.k, full.n, channels)
            if tile_rows:
                # many tokens: tiled planes, and the two-CTA kernel computes the chosen prefix
                planes = frame.alloc(int(self._lib.rns_packed_planes_bytes(m, full.k, channels, tile_rows)),
                                     torch.int8)
                N.check(self._lib.rns_encode_planes_tiled(a.data_ptr(), m, full.k, a.stride(0), arr, channels,
                                                          tile_rows, planes.data_ptr(), stream))
                self._launch_fused(prepared=full, m=m, a=None, a_planes=planes, a_packed=True, out=out,
                                   active=active, a_tile_rows=tile_rows)
            else:
                self._launch_fused(prepared=full, m=m, a=a, a_planes=None, out=out, active=active)
        if return_metadata:
            return out, AdaptiveMetadata(meta)
        return out

    # ------------------------------------------------------------------
    # Continuous batching (cuda_backend.py:624-703)
    # ------------------------------------------------------------------
    def create_request_batch_workspace(self, *, device: torch.device, dtype: torch.dtype,
                                       rows_per_request: Sequence[int], k: int, channels: int,
                                       n: int) -> RNSRequestBatchWorkspace:
        rows = tuple(int(x) for x in rows_per_request)
        if not rows or any(x <= 0 for x in rows):
            raise ValueError("rows_per_request must contain positive sizes")
        total = sum(rows)
        offsets = [0]
        for r in rows:
            offsets.append(offsets[-1] + r)
        return RNSRequestBatchWorkspace(
            activations=torch.empty((total, k), dtype=dtype, device=device),
            fused=self.create_workspace(device=device, channels=channels, m=total, n=n),
            rows_per_request=rows, k=int(k), _offsets=tuple(offsets),
        )

    def matmul_prepared_fused_requests(self, requests: Sequence[torch.Tensor],
                                       prepared_weight: PreparedRNSWeight, *, lut_channels: int = 2,
                                       workspace: RNSRequestBatchWorkspace | None = None,
                                       clone_outputs: bool = False) -> tuple[torch.Tensor, ...]:
        """Concatenate requests along M, one RNS GEMM, split the rows again.
        The merge is a single gather launch (``torch.cat(..., out=)``) rather
        than one copy per request (cuda_backend.py:684-688)."""
        if not requests:
            raise ValueError("requests must not be empty")
        first = requests[0]
        rows = tuple(int(x.shape[0]) for x in requests)
        for index, tensor in enumerate(requests):
            self._validate_matrix(tensor, f"requests[{index}]", 2)
            if tensor.dtype != first.dtype or tensor.device != first.device:
                raise ValueError("all requests must share dtype/device")
            if int(tensor.shape[1]) != prepared_weight.k:
                raise ValueError("request K does not match prepared weight")
        if workspace is None:
            workspace = self.create_request_batch_workspace(
                device=first.device, dtype=first.dtype, rows_per_request=rows, k=prepared_weight.k,
                channels=len(prepared_weight.moduli), n=prepared_weight.n)
        if workspace.rows_per_request != rows or workspace.k != prepared_weight.k:
            raise ValueError("request batch workspace does not match request shapes")
        if len(requests) == 1:
            workspace.activations.copy_(first)
        else:
            torch.cat(tuple(requests), dim=0, out=workspace.activations)
        merged = self.matmul_prepared_fused(workspace.activations, prepared_weight,
                                            lut_channels=lut_channels, workspace=workspace.fused)
        outputs = []
        offset = 0
        for row_count in rows:
            view = merged[offset:offset + row_count]
            outputs.append(view.clone() if clone_outputs else view)
            offset += row_count
        self._stats["continuous_batch_calls"] += 1
        self._stats["continuous_batch_requests"] += len(requests)
        return tuple(outputs)

    # ------------------------------------------------------------------
    # Floating-point linear: quantise -> fused GEMM with dequantising epilogue
    # ------------------------------------------------------------------
    def linear_forward(self, x: torch.Tensor, prepared: PreparedRNSWeight, weight_scale: torch.Tensor,
                       bias: torch.Tensor | None, *, per_row: bool = False,
                       adaptive: PreparedAdaptiveRNSWeight | None = None,
                       return_metadata: bool = False, out: torch.Tensor | None = None,
                       absmax_in: tuple[int, int, int] | None = None,
                       absmax_out: torch.Tensor | int | None = None,
                       out_copies: Sequence[int] = (), absmax_copies: Sequence[int] = (),
                       copies_multicast: bool = False):
        """y[M,N] = dequant( quant(x)[M,K] @ Wq[N,K]^T ) in the dtype of ``x``.

        The whole of ``RNSLinear.forward`` after weight preparation
        (layers/rns_linear.py:237-275): activation scale and quantisation
        (per tensor as in the reference, or per row), residue encoding, the
        per-channel GEMMs, reconstruction and ``x*s_a*s_w + bias`` in fp32, in
        two or three launches.  ``x`` is [M,K] float16/bfloat16/float32 with
        unit inner stride, or the [G,M,K/G] result of an all-gather of column
        shards; ``weight_scale`` float32 [N]; ``bias`` float32 [N].
        ``out`` may be a [M,N] view with unit inner stride (e.g. a column block
        of a wider matrix).

        Layer stacks can take the absmax pass out of the quantiser (per-tensor scale
        only): ``absmax_out`` (a device uint32 word) receives the bit pattern of
        max |y| of this call's outputs, written by the GEMM epilogue; ``absmax_in`` =
        (address, parts, stride in words) hands the next call the words whose maximum
        is its input's absmax (one word, or one per rank of a column-sharded layer).
        ``absmax_out`` needs the many-token kernel (M >= 512, 4 to 6 channels,
        K >= 512); otherwise it raises.  ``out_copies`` (device addresses, e.g. the
        same output slot in other ranks' memory) receive the same stores as ``out``
        from that kernel's epilogue, ``absmax_copies`` the finished absmax word.  With
        ``copies_multicast`` the single address in each list is an NVLink multicast address
        that maps the slot on every rank: one ``multimem.st`` per 16 bytes, replicated by the
        switch (two-byte outputs, N % 128 == 0, row stride % 8 == 0)."""
        if prepared.kernel != "tcgen05":
            raise ValueError("linear_forward needs a tensor-core prepared weight")
        if x.dtype not in _FLOAT_TYPES:
            raise ValueError("x must be float16, bfloat16 or float32")
        if x.ndim == 3:
            # [G, M, K/G]: what an all-gather of G column shards produces (or a
            # column-block view of it); only the innermost stride must be 1.
            if x.stride(2) != 1:
                raise ValueError("a gathered activation [G,M,K/G] needs unit inner stride")
            blocks, m, col_block = (int(v) for v in x.shape)
            k, ldx, col_block_stride = blocks * col_block, int(x.stride(1)), int(x.stride(0))
        elif x.ndim == 2 and x.stride(1) == 1:
            m, k = int(x.shape[0]), int(x.shape[1])
            ldx, col_block, col_block_stride = int(x.stride(0)), 0, 0
        else:
            raise ValueError("x must be [M,K] with unit inner stride, or a gathered [G,M,K/G]")
        if k != prepared.k:
            raise ValueError("K dimension does not match prepared weight")
        device = x.device
        mods, arr = self._mods(prepared.moduli if adaptive is None else adaptive.full_moduli)
        channels = len(mods)
        if out is None:
            out = torch.empty((m, prepared.n), dtype=x.dtype, device=device)
        elif out.shape != (m, prepared.n) or out.stride(1) != 1 or out.dtype != x.dtype:
            raise ValueError("out must be [M,N] of x's dtype with unit inner stride")
        if (adaptive is None and absmax_in is None and absmax_out is None and not out_copies and x.ndim == 2 and
                self._lib.rns_linear_small_supported(m, k, channels)):
            # Few tokens: the whole layer in one launch, no scratch.
            with torch.cuda.device(device):
                N.check(self._lib.rns_linear_small(
                    x.data_ptr(), _FLOAT_TYPES[x.dtype], m, k, ldx, 1 if per_row else 0,
                    prepared.weight_packed.data_ptr(), prepared.n, arr, channels, weight_scale.data_ptr(),
                    None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0),
                    _OUT_TYPES[out.dtype], self._stream(device)))
            self._stats["encode_centered_calls"] += 1
            self._stats["encode_centered_values"] += m * k
            self._stats["fused_gemm_calls"] += 1
            self._stats[f"fused_gemm_channels_{channels}"] += 1
            return (out, None) if return_metadata else out
        if (adaptive is None and absmax_out is None and not out_copies and m <= STREAM_MAX_ROWS and k % 8 == 0 and
                k * prepared.n < PAIR_LARGE_WEIGHT and self._lib.rns_linear_stream_supported(m, k, channels)):
            # Few tokens on a weight whose K the one-launch kernel cannot hold (and which is not
            # large: from K*N = 2^23 the two-CTA kernel measured faster): quantise to plain int8
            # (one or two small launches), then ONE launch that streams the weight once.
            with torch.cuda.device(device):
                scale_bytes = ((m if per_row else 1) * 4 + 255) & ~255
                base, stream = self.arena.block(device, scale_bytes + 256 + m * k)
                scale, scratch, act = base, base + scale_bytes, base + scale_bytes + 256
                parts_ptr, parts, parts_stride = absmax_in if absmax_in is not None else (None, 0, 0)
                N.check(self._lib.rns_quantize_activations_tiled(
                    x.data_ptr(), _FLOAT_TYPES[x.dtype], m, k, ldx, col_block, col_block_stride,
                    1 if per_row else 0, 127, arr, channels, act, None, 0, 0, scale, None, scratch,
                    parts_ptr, parts, parts_stride, stream))
                N.check(self._lib.rns_linear_stream(
                    act, m, k, k, scale, 1 if per_row else 0, prepared.weight_packed.data_ptr(), prepared.n, arr,
                    channels, weight_scale.data_ptr(), None if bias is None else bias.data_ptr(), out.data_ptr(),
                    out.stride(0), _OUT_TYPES[out.dtype], stream))
            self._stats["encode_centered_calls"] += 1
            self._stats["encode_centered_values"] += m * k
            self._stats["fused_gemm_calls"] += 1
            self._stats[f"fused_gemm_channels_{channels}"] += 1
            return (out, None) if return_metadata else out
        # Planes in tiles of 64 / 48 / 32 token rows for the two-CTA kernel where it is the
        # faster one; otherwise 128-row planes from 512 rows on, int8 activations below.
        tile_rows = self._pair_tile_rows(m, k, prepared.n, channels)
        use_planes = tile_rows != 0 or m >= PLANES_MIN_ROWS
        # Adaptive calls: the two-CTA kernel reads the prefix chosen on the device and skips
        # the other channels' planes, MMAs and residues (4 or 5 channels in the full set);
        # where it does not cover the shape the general kernel does the same from int8
        # activations.
        if adaptive is not None and (tile_rows == 0 or channels > 5):
            use_planes, tile_rows = False, 0
        if absmax_in is not None and per_row:
            raise ValueError("absmax_in serves the per-tensor scale")
        if absmax_out is not None and (tile_rows == 0 or per_row):
            raise ValueError("absmax_out needs the many-token kernel and a per-tensor scale")
        if out_copies and tile_rows == 0:
            raise ValueError("out_copies need the many-token kernel")
        meta = None
        with torch.cuda.device(device):
            # One block of the stream's arena, addressed by offsets (256-byte aligned):
            # scale [M or 1] f32 | scratch 8 x i32 ([0..3] absmax, [4] row-L1 max,
            # [5] active channels) | packed activations (int8, or R planes).
            scale_bytes = ((m if per_row else 1) * 4 + 255) & ~255
            if tile_rows:
                act_bytes = int(self._lib.rns_packed_planes_bytes(m, k, channels, tile_rows))
            else:
                act_bytes = int(self._lib.rns_packed_activation_bytes(m, k, channels if use_planes else 1))
            base, stream = self.arena.block(device, scale_bytes + 256 + act_bytes)
            scale, scratch, act = base, base + scale_bytes, base + scale_bytes + 256
            parts_ptr, parts, parts_stride = absmax_in if absmax_in is not None else (None, 0, 0)
            N.check(self._lib.rns_quantize_activations_tiled(
                x.data_ptr(), _FLOAT_TYPES[x.dtype], m, k, ldx, col_block, col_block_stride,
                1 if per_row else 0, 127,
                arr, channels, None if use_planes else act, act if use_planes else None, 1, tile_rows, scale,
                scratch + 16 if adaptive is not None else None, scratch, parts_ptr, parts, parts_stride, stream))
            active = None
            if adaptive is not None:
                state = self._state(device)
                if return_metadata:
                    meta = torch.empty(3, dtype=torch.int64, device=device)
                N.check(self._lib.rns_select_channels(
                    scratch + 16, adaptive.max_abs_weight, arr, channels,
                    adaptive.min_channels, scratch + 20,
                    None if meta is None else meta.data_ptr(), state.histogram.data_ptr(),
                    state.status.data_ptr(), stream))
                active = scratch + 20
                self._stats["adaptive_selections"] += 1
            self._stats["encode_centered_calls"] += 1
            self._stats["encode_centered_values"] += m * k
            self._stats["fused_gemm_calls"] += 1
            if adaptive is None:
                self._stats[f"fused_gemm_channels_{channels}"] += 1
            self._launch_fused(prepared=prepared if adaptive is None else adaptive.variants[channels],
                               m=m, a=None if use_planes else act, a_planes=act if use_planes else None,
                               a_packed=True, out=out, active=active,
                               row_scale=scale, row_scale_stride=1 if per_row else 0,
                               col_scale=weight_scale, bias=bias, stream=stream,
                               a_tile_rows=tile_rows, absmax_out=absmax_out,
                               out_copies=out_copies, absmax_copies=absmax_copies,
                               copies_multicast=copies_multicast)
        if return_metadata:
            return out, (AdaptiveMetadata(meta) if meta is not None else None)
        return out

    def matmul_grouped(self, a: torch.Tensor, b_nk: torch.Tensor, moduli: Iterable[int], *,
                       out_dtype: torch.dtype = torch.int64, scale: float | None = None) -> torch.Tensor:
        """Exact integer products of ``G`` independent problems in ONE launch:
        ``out[g] = a[g] @ b_nk[g].T`` for int8 ``a`` [G,M,K] and ``b_nk`` [G,N,K] (both
        operands are activations: nothing is cached).  The grouped multi-head products of
        attention - scores ``Q K^T`` (``a`` = Q [B*H,T,d], ``b_nk`` = K [B*H,T,d]) and
        ``P V`` (``a`` = P [B*H,T,T], ``b_nk`` = V^T [B*H,d,T]) - which the reference lists as
        open work (docs/OPTIMIZATIONS_V04.md:49) and times for one head through the plane
        pipeline (benchmarks/benchmark_attention.py:107-113).  One launch encodes the tiled
        residue planes of all G*M rows, one packs all G*N weight rows, one runs the two-CTA
        kernel over every (problem, tile).  4 to 6 moduli, K % 16 == 0, N % 8 == 0.
        ``out_dtype`` int64 / int32 returns the integers; float16 / bfloat16 / float32 with
        ``scale`` returns ``type(f32(x) * f32(scale))`` from the epilogue (a quarter of the
        output bytes of int64: e.g. scores scaled by s_q * s_k / sqrt(d))."""
        if a.ndim != 3 or b_nk.ndim != 3 or a.dtype != torch.int8 or b_nk.dtype != torch.int8:
            raise ValueError("matmul_grouped takes int8 a [G,M,K] and b_nk [G,N,K]")
        if not a.is_cuda or a.device != b_nk.device:
            raise ValueError("a and b_nk must be CUDA tensors on one device")
        groups, m, k = (int(v) for v in a.shape)
        if int(b_nk.shape[0]) != groups or int(b_nk.shape[2]) != k:
            raise ValueError("group counts or K dimensions do not match")
        n = int(b_nk.shape[1])
        mods, arr = self._mods(moduli)
        channels = len(mods)
        if channels not in (4, 5, 6) or k % 16 != 0 or k < 64 or n % 8 != 0:
            raise ValueError("matmul_grouped needs 4 to 6 moduli, K % 16 == 0, K >= 64 and N % 8 == 0")
        if not self.tensor_core_compatible(k=k, moduli=mods):
            raise ValueError("moduli / K are outside the tensor-core kernel's range")
        floating = out_dtype in _FLOAT_TYPES
        if floating != (scale is not None) or (not floating and out_dtype not in (torch.int64, torch.int32)):
            raise ValueError("out_dtype int64 / int32 without scale, or float16 / bfloat16 / float32 with scale")
        token_tile = {4: 128, 5: 96, 6: 64}[channels]
        m_pad = -(-m // token_tile) * token_tile
        a = a.contiguous()
        if m_pad != m:
            a = torch.nn.functional.pad(a, (0, 0, 0, m_pad - m))            # whole token tiles per problem
        b_nk = b_nk.contiguous()
        device = a.device
        out = torch.empty((groups, m_pad, n), dtype=out_dtype, device=device)
        prepared = PreparedRNSWeight(backend=self, moduli=mods, k=k, n=n, kernel="tcgen05")
        with torch.cuda.device(device):
            stream = self._stream(device)
            frame = self.arena.frame(device)
            tile_rows = token_tile // 2
            planes = frame.alloc(int(self._lib.rns_packed_planes_bytes(groups * m_pad, k, channels, tile_rows)),
                                 torch.int8)
            N.check(self._lib.rns_encode_planes_tiled(a.data_ptr(), groups * m_pad, k, k, arr, channels,
                                                      tile_rows, planes.data_ptr(), stream))
            packed = frame.alloc(int(self._lib.rns_packed_weight_bytes(groups * n, k)), torch.int8)
            N.check(self._lib.rns_pack_weight(b_nk.data_ptr(), groups * n, k, k, packed.data_ptr(), stream))
            self._stats["encode_centered_calls"] += 1
            self._stats["encode_centered_values"] += int(a.numel())
            self._stats["fused_gemm_calls"] += 1
            self._stats[f"fused_gemm_channels_{channels}"] += 1
            scales = {}
            if floating:
                scales = dict(row_scale=torch.full((1,), float(scale), dtype=torch.float32, device=device),
                              row_scale_stride=0, col_scale=torch.ones(n, dtype=torch.float32, device=device))
            self._launch_fused(prepared=prepared, m=m_pad, a=None, a_planes=planes, a_packed=True, out=out[0],
                               a_tile_rows=tile_rows, groups=groups, packed_weight=packed, stream=stream, **scales)
        return out[:, :m] if m_pad != m else out

    def supports_wide_forward(self, prepared: PreparedRNSWeight, m: int) -> bool:
        """True when ``linear_forward_wide`` serves this call: the prepared weight carries
        packed residue planes and there are enough rows to fill tensor-core tiles."""
        return prepared.weight_planes_packed is not None and int(m) >= WIDE_MIN_ROWS

    def linear_forward_wide(self, x: torch.Tensor, prepared: PreparedRNSWeight, weight_scale: torch.Tensor,
                            bias: torch.Tensor | None, *, quant_max: int, per_row: bool = False,
                            out: torch.Tensor | None = None) -> torch.Tensor:
        """``RNSLinear.forward`` for sources wider than 8 bits (quant_bits 12 / 16,
        layers/rns_linear.py:45-46, 96-98, 237-275 of the reference) on the tensor cores:
        the quantiser writes the centred residues of the 12/16-bit integers as tiled planes
        (the integers themselves are never stored), the two-CTA kernel multiplies them
        with the cached residue planes of the weight, one int8 MMA per channel, and its
        epilogue reconstructs the (up to 48-bit) integer, converts it to fp32 as
        ``integer_result.float()`` does and applies ``* s_a * s_w + bias``."""
        if prepared.weight_planes_packed is None:
            raise ValueError("linear_forward_wide needs a prepared weight with packed residue planes")
        if x.dtype not in _FLOAT_TYPES or x.ndim != 2 or x.stride(1) != 1:
            raise ValueError("x must be [M,K] float16, bfloat16 or float32 with unit inner stride")
        if not 127 < int(quant_max) <= 32767:
            raise ValueError("quant_max of a wide source lies in (127, 32767]")
        m, k = int(x.shape[0]), int(x.shape[1])
        if k != prepared.k:
            raise ValueError("K dimension does not match prepared weight")
        device = x.device
        mods, arr = self._mods(prepared.moduli)
        channels = len(mods)
        tile_rows = int(self._lib.rns_pair_tile_rows(channels, k))
        if tile_rows == 0:
            raise ValueError("the two-CTA kernel does not cover this channel count / K")
        if out is None:
            out = torch.empty((m, prepared.n), dtype=x.dtype, device=device)
        elif out.shape != (m, prepared.n) or out.stride(1) != 1 or out.dtype != x.dtype:
            raise ValueError("out must be [M,N] of x's dtype with unit inner stride")
        with torch.cuda.device(device):
            scale_bytes = ((m if per_row else 1) * 4 + 255) & ~255
            act_bytes = int(self._lib.rns_packed_planes_bytes(m, k, channels, tile_rows))
            base, stream = self.arena.block(device, scale_bytes + 256 + act_bytes)
            scale, scratch, act = base, base + scale_bytes, base + scale_bytes + 256
            N.check(self._lib.rns_quantize_activations_tiled(
                x.data_ptr(), _FLOAT_TYPES[x.dtype], m, k, int(x.stride(0)), 0, 0, 1 if per_row else 0,
                int(quant_max), arr, channels, None, act, 1, tile_rows, scale, None, scratch, None, 0, 0, stream))
            self._stats["encode_centered_calls"] += 1
            self._stats["encode_centered_values"] += m * k
            self._stats["fused_gemm_calls"] += 1
            self._stats[f"fused_gemm_channels_{channels}"] += 1
            self._launch_fused(prepared=prepared, m=m, a=None, a_planes=act, a_packed=True, out=out,
                               row_scale=scale, row_scale_stride=1 if per_row else 0, col_scale=weight_scale,
                               bias=bias, stream=stream, a_tile_rows=tile_rows, weight_planes=True)
        return out

    def _pair_tile_rows(self, m: int, k: int, n: int, channels: int) -> int:
        """Token rows per packed tile when this call should take the two-CTA kernel, else 0."""
        rows = int(self._lib.rns_pair_tile_rows(int(channels), int(k)))
        if rows == 0 or self._lib.rns_linear_small_supported(int(m), int(k), int(channels)):
            return 0          # not covered, or few tokens that the one-launch kernel takes
        if m >= PAIR_MIN_ROWS or int(k) * int(n) >= PAIR_LARGE_WEIGHT:
            return rows
        return 0

    def supports_absmax_out(self, *, m: int, k: int, channels: int) -> bool:
        """True when ``linear_forward`` runs the many-token kernel for this problem, the one
        whose epilogue can report max |y| (``absmax_out``)."""
        return m >= PAIR_MIN_ROWS and int(self._lib.rns_pair_tile_rows(int(channels), int(k))) > 0

    def quantize_weight(self, weight: torch.Tensor, quant_max: int = 127
                        ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Per-output-channel symmetric int8 of an nn.Linear weight [N,K]
        (layers/rns_linear.py:183-184), kept in that layout.  Returns
        (int8 [N,K], float32 scale [N], int32 [1] max |q| on the device)."""
        if weight.ndim != 2 or weight.stride(1) != 1 or weight.dtype not in _FLOAT_TYPES:
            raise ValueError("weight must be a [N,K] floating matrix with unit inner stride")
        n, k = int(weight.shape[0]), int(weight.shape[1])
        wq = torch.empty((n, k), dtype=torch.int8, device=weight.device)
        scale = torch.empty(n, dtype=torch.float32, device=weight.device)
        max_abs = torch.empty(1, dtype=torch.int32, device=weight.device)
        with torch.cuda.device(weight.device):
            N.check(self._lib.rns_quantize_weight(
                weight.data_ptr(), _FLOAT_TYPES[weight.dtype], n, k, weight.stride(0), int(quant_max),
                wq.data_ptr(), scale.data_ptr(), max_abs.data_ptr(), self._stream(weight.device)))
        return wq, scale, max_abs

    # ------------------------------------------------------------------
    # CRT decode and wide helpers (cuda_backend.py:705-799)
    # ------------------------------------------------------------------
    def decode(self, residues: torch.Tensor, moduli: Iterable[int], *, signed: bool = True) -> torch.Tensor:
        """Chinese-remainder decode kept as the reference's cross-check of the
        Garner kernel (cuda_backend.py:706-731); a handful of int64 tensor ops,
        not on the hot path."""
        self._validate_matrix(residues, "residues", residues.ndim)
        if residues.dtype not in (torch.uint8, torch.int8):
            raise ValueError("decoder expects uint8 canonical or int8 centered residues")
        product, coefficients = crt_constants(moduli)
        result = torch.zeros(residues.shape[1:], dtype=torch.int64, device=residues.device)
        for channel, coefficient in enumerate(coefficients):
            result = torch.remainder(result + residues[channel].to(torch.int64) * coefficient, product)
        if signed:
            result = torch.where(result > product // 2, result - product, result)
        return result

    def matmul_wide(self, a: torch.Tensor, b: torch.Tensor, moduli: Iterable[int], *,
                    decode: bool = True, kernel: CenteredKernelName = "auto") -> torch.Tensor:
        self._validate_matrix(a, "a", 2)
        self._validate_matrix(b, "b", 2)
        if a.dtype not in _INT_TYPES:
            raise ValueError("a must be int8/int16/int32")
        if b.dtype != a.dtype:
            raise ValueError("a and b must use the same integer dtype")
        if a.shape[1] != b.shape[0]:
            raise ValueError("K dimensions do not match")
        mods, _ = self._mods(moduli)
        a_residues = self.encode_centered(a.contiguous(), mods)
        b_residues = self.encode_centered(b.contiguous(), mods)
        output = self.matmul_centered_residues(a_residues, b_residues, mods, kernel=kernel)
        return self.decode(output, mods) if decode else output

    def matmul_wide_fused(self, a: torch.Tensor, b: torch.Tensor, moduli: Iterable[int], *,
                          lut_channels: int = 0, workspace: RNSWorkspace | None = None) -> torch.Tensor:
        self._validate_matrix(a, "a", 2)
        self._validate_matrix(b, "b", 2)
        if a.dtype not in _INT_TYPES:
            raise ValueError("a must be int8/int16/int32")
        if b.dtype != a.dtype or a.shape[1] != b.shape[0]:
            raise ValueError("dtype/K mismatch")
        mods, _ = self._mods(moduli)
        if a.dtype == torch.int8 and self.tensor_core_compatible(k=int(a.shape[1]), moduli=mods):
            return self.matmul_prepared_fused(a, self.prepare_weight(b, mods), lut_channels=lut_channels,
                                              workspace=workspace)
        a_residues = self.encode_centered(a.contiguous(), mods)
        b_residues = self.encode_centered(b.contiguous(), mods)
        return self.matmul_centered_fused(a_residues, b_residues, mods, lut_channels=lut_channels,
                                          workspace=workspace)

    def matmul_int8(self, a: torch.Tensor, b: torch.Tensor, moduli: Iterable[int], *,
                    decode: bool = True, kernel: CenteredKernelName = "auto") -> torch.Tensor:
        if a.dtype != torch.int8 or b.dtype != torch.int8:
            raise ValueError("matmul_int8 expects int8 inputs")
        return self.matmul_wide(a, b, moduli, decode=decode, kernel=kernel)

    # Host-side constants in the reference's shapes, for callers that want them
    # (cuda_backend.py:48-66): reciprocals, P, CRT coefficients, pairwise inverses, LUT.
    @staticmethod
    def host_constants(moduli: Iterable[int]):
        mods = validate_moduli(moduli)
        product, coefficients = crt_constants(mods)
        return (tuple((1 << 32) // m for m in mods), product, coefficients,
                garner_pairwise_inverses(mods), compact_byte_mod_lut(mods))
