"""ctypes access to oracle/librns_oracle.so (the C restatement).  Test infrastructure."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "librns_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "rns_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "librns_oracle.so"], check=True, capture_output=True)
    return LIB


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB))
        _lib.rns_oracle_linear.restype = C.c_int
        _lib.rns_oracle_garner.restype = C.c_int
        _lib.rns_oracle_threads.restype = C.c_int
    return _lib


def threads() -> int:
    return int(load().rns_oracle_threads())


def _ptr(arr):
    return None if arr is None else arr.ctypes.data_as(C.c_void_p)


def linear(a_q: np.ndarray, w_q: np.ndarray, moduli, row_scale=None, col_scale=None, bias=None,
           want_float: bool = False):
    """a_q int8 [M,K], w_q int8 [N,K] -> (int64 [M,N], float32 [M,N] or None)."""
    a_q = np.ascontiguousarray(a_q, dtype=np.int8)
    w_q = np.ascontiguousarray(w_q, dtype=np.int8)
    m, k = a_q.shape
    n = w_q.shape[0]
    mods = np.asarray(moduli, dtype=np.int32)
    out_i = np.empty((m, n), dtype=np.int64)
    out_f = np.empty((m, n), dtype=np.float32) if want_float else None
    rs = cs = bs = None
    stride = 0
    if want_float:
        rs = np.ascontiguousarray(row_scale, dtype=np.float32).reshape(-1)
        stride = 0 if rs.size == 1 else 1
        cs = np.ascontiguousarray(col_scale, dtype=np.float32)
        bs = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    rc = load().rns_oracle_linear(_ptr(a_q), _ptr(w_q), C.c_int(m), C.c_int(n), C.c_int(k),
                                  _ptr(mods), C.c_int(len(mods)), _ptr(out_i), _ptr(out_f),
                                  _ptr(rs), C.c_int(stride), _ptr(cs), _ptr(bs))
    if rc != 0:
        raise ValueError("rns_oracle_linear: bad argument")
    return out_i, out_f


def garner(sums: np.ndarray, moduli) -> np.ndarray:
    sums = np.ascontiguousarray(sums, dtype=np.int32)
    mods = np.asarray(moduli, dtype=np.int32)
    out = np.empty(sums.shape[1:], dtype=np.int64)
    rc = load().rns_oracle_garner(_ptr(sums), C.c_int64(out.size), _ptr(mods), C.c_int(len(mods)), _ptr(out))
    if rc != 0:
        raise ValueError("rns_oracle_garner: bad argument")
    return out
