"""CPU oracle for CSR SpMV / SpMM: ctypes wrapper around oracle/csr_oracle.c.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the CPU-baseline /
reference arms of bench.py.  The shipped package (flagsparse_b200/) never imports it.

The C file restates FlagSparse's Triton kernels with the dtype promotion of their launchers
(see the header of csr_oracle.c for the file:line map).  Parity is pinned: tests/golden/ holds
outputs of FlagSparse's own kernels (run on CPU through Triton's interpreter by
tests/golden/make_golden.py) and tests/test_oracle.py checks this oracle against them.

All functions take and return numpy arrays.  alpha / beta are applied in the promoted
precision (float64 / complex128), then the result is cast to the input dtype: the reference has
no alpha / beta, so this is `alpha * ref + beta * y0` evaluated the way its own tests evaluate
their dense references (tests/pytest/test_spmv_csr_accuracy.py:39-46, :113-115).
"""

from __future__ import annotations

import ctypes
import subprocess
from ctypes import c_int, c_int64, c_void_p
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
LIB_PATH = _DIR / "_ref" / "libcsr_oracle.so"
_lib = None

OPS = ("non", "trans", "conj")


def build(force=False):
    """Compile csr_oracle.c with the Makefile next to it."""
    src = _DIR / "csr_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B", "_ref/libcsr_oracle.so"], check=True,
                       capture_output=True)
    return LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        lib = ctypes.CDLL(str(LIB_PATH))
        lib.orc_spmv_real.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int64, c_int]
        lib.orc_spmv_cplx.argtypes = lib.orc_spmv_real.argtypes
        lib.orc_spmm_real.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_int64, c_void_p, c_int64]
        lib.orc_spmm_cplx.argtypes = lib.orc_spmm_real.argtypes
        lib.orc_transpose.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64,
                                      c_int64, c_void_p, c_void_p, c_void_p]
        lib.orc_set_threads.argtypes = [c_int]
        lib.orc_set_threads.restype = c_int
        for f in (lib.orc_spmv_real, lib.orc_spmv_cplx, lib.orc_spmm_real, lib.orc_spmm_cplx,
                  lib.orc_transpose):
            f.restype = None
        _lib = lib
    return _lib


def set_threads(n=0):
    """Ask for n OpenMP threads in the row loops (0: leave as is); returns the number in use."""
    return int(_load().orc_set_threads(int(n)))


def _p(a):
    return a.ctypes.data_as(c_void_p)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


_PROMOTED = {np.dtype(np.float32): np.float64, np.dtype(np.float64): np.float64,
             np.dtype(np.complex64): np.complex128, np.dtype(np.complex128): np.complex128}


def transpose_csr(data, indices, indptr, shape, conj=False):
    """CSR(A) -> CSR(A^T) (A^H with conj=True); entries of an output row keep ascending source
    position.  Index arrays come back as int64."""
    lib = _load()
    n_rows, n_cols = int(shape[0]), int(shape[1])
    data = np.ascontiguousarray(data)
    idx, ptr = _i64(indices), _i64(indptr)
    t_data = np.empty_like(data)
    t_idx = np.empty(data.shape[0], dtype=np.int64)
    t_ptr = np.empty(n_cols + 1, dtype=np.int64)
    kind = 0
    if conj and data.dtype == np.complex64:
        kind = 1
    elif conj and data.dtype == np.complex128:
        kind = 2
    lib.orc_transpose(_p(data), data.dtype.itemsize, kind, _p(idx), _p(ptr), n_rows, n_cols,
                      _p(t_data), _p(t_idx), _p(t_ptr))
    return t_data, t_idx, t_ptr, (n_cols, n_rows)


def _materialize(data, indices, indptr, shape, op):
    if op not in OPS:
        raise ValueError(f"op must be one of {OPS}")
    if op == "non":
        return np.ascontiguousarray(data), _i64(indices), _i64(indptr), (int(shape[0]),
                                                                         int(shape[1]))
    return transpose_csr(data, indices, indptr, shape, conj=(op == "conj"))


def spmv_acc(data, indices, indptr, x, shape, op="non", block_nnz=256):
    """op(A) @ x in the reference's accumulation dtype (float64, or the complex dtype itself)."""
    lib = _load()
    data, idx, ptr, (n_rows, _) = _materialize(data, indices, indptr, shape, op)
    x = np.ascontiguousarray(x, dtype=data.dtype)
    if data.dtype in (np.float32, np.float64):
        y = np.empty(n_rows, dtype=np.float64)
        lib.orc_spmv_real(_p(data), int(data.dtype == np.float32), _p(idx), _p(ptr), _p(x),
                          _p(y), n_rows, int(block_nnz))
    else:
        y = np.empty(n_rows, dtype=data.dtype)
        lib.orc_spmv_cplx(_p(data), int(data.dtype == np.complex64), _p(idx), _p(ptr), _p(x),
                          _p(y), n_rows, int(block_nnz))
    return y


def spmv(data, indices, indptr, x, shape, op="non", alpha=1.0, beta=0.0, y0=None,
         block_nnz=256):
    """alpha * op(A) @ x + beta * y0, cast to data.dtype."""
    data = np.asarray(data)
    acc = spmv_acc(data, indices, indptr, x, shape, op=op, block_nnz=block_nnz)
    wide = _PROMOTED[data.dtype]
    if alpha == 1.0 and beta == 0.0:
        return acc.astype(data.dtype)
    out = np.asarray(alpha, dtype=wide) * acc.astype(wide)
    if beta != 0.0:
        out = out + np.asarray(beta, dtype=wide) * np.asarray(y0).astype(wide)
    return out.astype(data.dtype)


def spmm_acc(data, indices, indptr, B, shape, op="non"):
    lib = _load()
    data, idx, ptr, (n_rows, _) = _materialize(data, indices, indptr, shape, op)
    B = np.ascontiguousarray(B, dtype=data.dtype)
    n_dense = int(B.shape[1])
    if data.dtype in (np.float32, np.float64):
        C = np.empty((n_rows, n_dense), dtype=np.float64)
        lib.orc_spmm_real(_p(data), int(data.dtype == np.float32), _p(idx), _p(ptr), _p(B),
                          n_dense, n_dense, _p(C), n_rows)
    else:
        C = np.empty((n_rows, n_dense), dtype=data.dtype)
        lib.orc_spmm_cplx(_p(data), int(data.dtype == np.complex64), _p(idx), _p(ptr), _p(B),
                          n_dense, n_dense, _p(C), n_rows)
    return C


def spmm(data, indices, indptr, B, shape, op="non", alpha=1.0, beta=0.0, C0=None):
    """alpha * op(A) @ B + beta * C0, cast to data.dtype."""
    data = np.asarray(data)
    acc = spmm_acc(data, indices, indptr, B, shape, op=op)
    wide = _PROMOTED[data.dtype]
    if alpha == 1.0 and beta == 0.0:
        return acc.astype(data.dtype)
    out = np.asarray(alpha, dtype=wide) * acc.astype(wide)
    if beta != 0.0:
        out = out + np.asarray(beta, dtype=wide) * np.asarray(C0).astype(wide)
    return out.astype(data.dtype)


def rel_l2(actual, expected):
    """||actual - expected||_2 / ||expected||_2 in float64 (0 when both are zero)."""
    a = np.asarray(actual).astype(np.complex128).ravel()
    e = np.asarray(expected).astype(np.complex128).ravel()
    den = np.linalg.norm(e)
    num = np.linalg.norm(a - e)
    if den == 0.0:
        return 0.0 if num == 0.0 else float("inf")
    return float(num / den)
