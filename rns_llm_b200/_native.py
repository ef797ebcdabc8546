"""ctypes binding of librns_b200.so (the C ABI declared in include/rns_b200.h).

The library is the only implementation of the RNS path: when it is missing
this module raises, and nothing in the package computes the path another way.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path
from typing import Sequence

# RNS_B200_LIBRARY points at another build of the same library (e.g. one with
# extra instrumentation); by default the in-tree build is loaded.
_LIB_PATH = Path(os.environ.get("RNS_B200_LIBRARY") or
                 Path(__file__).resolve().parent / "csrc" / "librns_b200.so")
_lock = threading.Lock()
_lib: C.CDLL | None = None

MAX_CHANNELS = 10
TC_MAX_CHANNELS = 8
MAX_PEERS = 7

# rns_status
OK, ERR_INVALID_ARGUMENT, ERR_BAD_MODULI, ERR_UNSUPPORTED, ERR_OVERFLOW, ERR_CUDA, ERR_DEVICE_TIMEOUT = range(7)
# rns_int_type / rns_out_type / rns_float_type
INT8, INT16, INT32 = 0, 1, 2
OUT_INT64, OUT_INT32, OUT_F16, OUT_BF16, OUT_F32 = 0, 1, 2, 3, 4
F16, BF16, F32 = 0, 1, 2


class LinearArgs(C.Structure):
    """struct rns_linear_args."""

    _fields_ = [
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("channels", C.c_int32),
        ("moduli", C.c_int32 * MAX_CHANNELS),
        ("d_a", C.c_void_p),
        ("d_a_planes", C.c_void_p),
        ("lda", C.c_int64),
        ("a_plane_stride", C.c_int64),
        ("d_w", C.c_void_p),
        ("ldw", C.c_int64),
        ("d_active_channels", C.c_void_p),
        ("d_out", C.c_void_p),
        ("ldo", C.c_int64),
        ("out_type", C.c_int32),
        ("d_row_scale", C.c_void_p),
        ("row_scale_stride", C.c_int32),
        ("d_col_scale", C.c_void_p),
        ("d_bias", C.c_void_p),
        ("d_status", C.c_void_p),
        ("tile_n", C.c_int32),
        ("tile_k", C.c_int32),
        ("a_packed", C.c_int32),
        ("w_packed", C.c_int32),
        ("pair_mode", C.c_int32),
        ("enc_groups", C.c_int32),
        ("enc_stages", C.c_int32),
        ("sub_blocks", C.c_int32),
        ("variant", C.c_int32),
        ("exact_residues", C.c_int32),
        ("a_tile_rows", C.c_int32),
        ("d_absmax_out", C.c_void_p),
        ("n_out_copies", C.c_int32),
        ("d_out_copies", C.c_void_p * MAX_PEERS),
        ("d_absmax_copies", C.c_void_p * MAX_PEERS),
        ("d_wait_info", C.c_void_p),
        ("w_channel_stride", C.c_int64),
        ("out_copies_multicast", C.c_int32),
        ("groups", C.c_int32),
    ]


_I32P = C.POINTER(C.c_int32)
_I64P = C.POINTER(C.c_int64)
_VP = C.c_void_p

# name -> (restype, argtypes); every symbol include/rns_b200.h declares.
SIGNATURES: dict[str, tuple] = {
    "rns_last_error": (C.c_char_p, []),
    "rns_version": (C.c_int, []),
    "rns_host_constants": (C.c_int, [_I32P, C.c_int, _I64P, _I32P, _I64P]),
    "rns_minimal_prefix_channels": (C.c_int, [_I32P, C.c_int, C.c_int64, C.c_int]),
    "rns_host_reconstruct": (C.c_int, [_VP, C.c_int64, _I32P, C.c_int, C.c_int, _VP]),
    "rns_host_encode_centered_i8": (C.c_int, [_VP, C.c_int64, _I32P, C.c_int, _VP]),
    "rns_host_encode_reduced_i8": (C.c_int, [_VP, C.c_int64, _I32P, C.c_int, _VP]),
    "rns_encode_canonical_i8": (C.c_int, [_VP, C.c_int64, _I32P, C.c_int, _VP, _VP]),
    "rns_encode_centered": (C.c_int, [_VP, C.c_int, C.c_int64, _I32P, C.c_int, _VP, _VP]),
    "rns_matmul_canonical_planes": (C.c_int, [_VP, _VP, _I32P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP]),
    "rns_matmul_centered_planes": (C.c_int, [_VP, _VP, _I32P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP]),
    "rns_decode_garner": (C.c_int, [_VP, C.c_int64, _I32P, C.c_int, _VP, _VP]),
    "rns_matmul_centered_fused_out": (C.c_int, [_VP, _VP, _I32P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, _VP]),
    "rns_linear_fused": (C.c_int, [C.POINTER(LinearArgs), _VP]),
    "rns_linear_fused_supported": (C.c_int, [_I32P, C.c_int, C.c_int, C.c_int64, C.c_int64]),
    "rns_quantize_activations": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int64, C.c_int, C.c_int, _I32P, C.c_int, _VP, _VP, C.c_int, _VP, _VP, _VP, _VP]),
    "rns_packed_weight_bytes": (C.c_int64, [C.c_int, C.c_int]),
    "rns_packed_activation_bytes": (C.c_int64, [C.c_int, C.c_int, C.c_int]),
    "rns_packed_planes_bytes": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "rns_pair_tile_rows": (C.c_int, [C.c_int, C.c_int]),
    "rns_quantize_activations_tiled": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int64, C.c_int,
                                                 C.c_int, _I32P, C.c_int, _VP, _VP, C.c_int, C.c_int, _VP, _VP, _VP,
                                                 _VP, C.c_int, C.c_int64, _VP]),
    "rns_pack_weight": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int64, _VP, _VP]),
    "rns_unpack_weight": (C.c_int, [_VP, C.c_int, C.c_int, _VP, C.c_int64, _VP]),
    "rns_encode_planes_packed": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int64, _I32P, C.c_int, _VP, _VP]),
    "rns_encode_planes_tiled": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int64, _I32P, C.c_int, C.c_int, _VP, _VP]),
    "rns_row_l1_max_i8": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int64, _VP, _VP]),
    "rns_select_channels": (C.c_int, [_VP, C.c_int32, _I32P, C.c_int, C.c_int, _VP, _VP, _VP, _VP, _VP]),
    "rns_linear_small_supported": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "rns_linear_stream_supported": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "rns_linear_stream": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int64, _VP, C.c_int, _VP, C.c_int, _I32P, C.c_int,
                                    _VP, _VP, _VP, C.c_int64, C.c_int32, _VP]),
    "rns_linear_small": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, _VP, C.c_int, _I32P, C.c_int,
                                   _VP, _VP, _VP, C.c_int64, C.c_int32, _VP]),
    "rns_static_scratch_bytes": (C.c_int64, []),
    "rns_linear_static": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.c_int64, _VP, C.c_int, _I32P, C.c_int, _VP, _VP,
                                    _VP, C.c_int64, C.c_int32, _VP, _VP]),
    "rns_quantize_weight": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, _VP, _VP, _VP, _VP]),
}


def library_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load() -> C.CDLL:
    """Loads the library once; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                raise RuntimeError(
                    f"{_LIB_PATH} is not built. Run: python -m rns_llm_b200.csrc.build"
                )
            lib = C.CDLL(str(_LIB_PATH))
            for name, (restype, argtypes) in SIGNATURES.items():
                fn = getattr(lib, name)  # AttributeError if the symbol is missing
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = lib
    return _lib


def last_error() -> str:
    return load().rns_last_error().decode("utf-8", "replace")


_EXCEPTIONS = {
    ERR_INVALID_ARGUMENT: ValueError,
    ERR_BAD_MODULI: ValueError,
    ERR_UNSUPPORTED: ValueError,
    ERR_OVERFLOW: OverflowError,
    ERR_CUDA: RuntimeError,
    ERR_DEVICE_TIMEOUT: RuntimeError,
}


def check(status: int) -> None:
    """Maps an rns_status to the exception class the reference raises for the
    same condition (ValueError for shapes/dtypes/moduli, OverflowError for
    range, RuntimeError for CUDA failures)."""
    if status != OK:
        raise _EXCEPTIONS.get(status, RuntimeError)(last_error() or f"rns status {status}")


def moduli_array(moduli: Sequence[int]):
    arr = (C.c_int32 * len(moduli))(*[int(m) for m in moduli])
    return arr
