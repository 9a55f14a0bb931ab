"""Prepared CSR SpMM ("route" API) with row- or column-major dense operands.

Mirrors ``prepare_spmm_csr_route`` / ``flagsparse_spmm_csr_run`` of
``flagsparse.sparse_operations.spmm_csr`` (spmm_csr.py:2040-2174) with the handle class
``PreparedCsrSpmmRoute`` (:527-569), the algorithm names of its registry (:571-583, :1973-2037)
and the dense-layout helpers (:586-639).

What differs underneath: the reference registers several Triton schedules of the same product
("csr_base", "spmm_csr_alg1", ...); here every name runs the one sm_100a tile kernel, and a name
is only checked against the dtypes / layouts the reference allows for it, so that code written
against the reference raises the same exceptions.  ``op = trans / conj`` uses the transpose cached
with the matrix (the reference materialises it on every run, :683-710).  ``dense_layout="col"``
transposes B into the row-major operand the kernel gathers 16-byte row pieces from and transposes
the result into a column-major C (``b2s_dense_transpose``); gathering single elements of a
column-major B, as the reference's strided kernel does, would cost one divergent load per
(non-zero, dense column) instead of one row read per non-zero.
"""

from __future__ import annotations

import torch

from . import _lib
from ._contract import HALF_VALUE_DTYPES
from ._contract import OP_CONJ_TRANS, is_complex, normalize_op, op_name, op_transposes
from .spmm import (SUPPORTED_SPMM_VALUE_DTYPES, _checked_spmm_plan, _launch_spmm,
                   _launch_spmm_colmajor_c, _row_major_ok)


class SpmmCsrAlgorithmUnavailable(RuntimeError):
    """Raised when a registered SpMM CSR route is unavailable in this runtime."""


# name -> (display name, value dtypes the reference registers the route for)
_REAL = (torch.float32, torch.float64)
SPMM_CSR_ALGORITHMS = {
    "csr_base": ("Base", HALF_VALUE_DTYPES + SUPPORTED_SPMM_VALUE_DTYPES),
    "alpha_alg1_tle_opt": ("TLEOpt", _REAL),
    "alpha_alg1_tle_opt2": ("TLEOpt2", _REAL),
    "spmm_csr_alg1": ("Alg1", _REAL),
    "spmm_csr_alg2": ("Alg2", _REAL),
}


_ALG_ALIASES = {
    "base": "csr_base", "csr": "csr_base", "csr_base": "csr_base",
    "alg1": "spmm_csr_alg1", "csr_alg1": "spmm_csr_alg1", "spmm_csr_alg1": "spmm_csr_alg1",
    "alg2": "spmm_csr_alg2", "csr_alg2": "spmm_csr_alg2", "spmm_csr_alg2": "spmm_csr_alg2",
}


def _normalize_spmm_csr_alg(alg):
    """Alias table of the reference (spmm_csr.py:571-583); unknown tokens pass through so that
    the registry lookup reports them."""
    if alg is None:
        return "auto"
    token = str(alg).strip().lower()
    return _ALG_ALIASES.get(token, token)


def resolve_spmm_csr_algorithm(alg, op, dtype):
    """Name of the route `alg` resolves to ("auto" -> "csr_base"); ValueError for an unknown
    name, TypeError when the reference does not register that route for `dtype`."""
    token = _normalize_spmm_csr_alg(alg)
    if token == "auto":
        token = "csr_base"
    if token not in SPMM_CSR_ALGORITHMS:
        supported = ", ".join(sorted(SPMM_CSR_ALGORITHMS))
        raise ValueError(f"unsupported CSR SpMM algorithm {alg!r}; supported: auto, {supported}")
    op_name(normalize_op(op))  # every route takes all three ops; this validates the token
    if dtype not in SPMM_CSR_ALGORITHMS[token][1]:
        raise TypeError(f"algorithm {token!r} does not support dtype {dtype}")
    return token


def list_spmm_csr_algorithms(op=None, dtype=None):
    if op is not None:
        normalize_op(op)
    return tuple(name for name, (_, dtypes) in SPMM_CSR_ALGORITHMS.items()
                 if dtype is None or dtype in dtypes)


_ROW_LAYOUT_NAMES = frozenset(("auto", "default", "row", "row_major", "row-major", "c", "c_order"))
_COL_LAYOUT_NAMES = frozenset(("col", "column", "col_major", "column_major", "col-major",
                               "column-major", "f", "fortran"))


def _normalize_dense_layout(layout):
    """'row' or 'col' from the spellings the reference accepts (spmm_csr.py:586-594)."""
    token = "row" if layout is None else str(layout).strip().lower()
    if token in _ROW_LAYOUT_NAMES:
        return "row"
    if token in _COL_LAYOUT_NAMES:
        return "col"
    raise ValueError("dense_layout must be one of: auto, row, col")


def _is_col_major_2d(t):
    return (torch.is_tensor(t) and t.ndim == 2 and t.stride(0) == 1
            and t.stride(1) >= max(1, int(t.shape[0])))


def _dense_layout_name(t):
    if not torch.is_tensor(t) or t.ndim != 2:
        return "unknown"
    if t.is_contiguous():
        return "row"
    if _is_col_major_2d(t):
        return "col"
    return "strided"


def _empty_col_major(rows, cols, dtype, device):
    return torch.empty_strided((rows, cols), (1, max(1, rows)), dtype=dtype, device=device)


class PreparedCsrSpmmRoute:
    """A validated CSR matrix ready for repeated ``flagsparse_spmm_csr_run`` calls.

    Attribute names follow the reference's handle (spmm_csr.py:527-569).  The tile plan, the
    scratch buffers and -- once an ``op = trans / conj`` run has asked for it -- the transposed
    matrix live in the plan object kept here."""

    def __init__(self, plan, shape, op, alg, value_dtype=None):
        self._plan = plan
        # dtype of the caller's values, of B and of C; float16 / bfloat16 matrices are kept and
        # multiplied in float32 (plan.data)
        self.value_dtype = plan.data.dtype if value_dtype is None else value_dtype
        self.data = plan.data
        self.kernel_indices = plan.indices
        self.kernel_indptr = plan.indptr
        self.shape = (int(shape[0]), int(shape[1]))
        self.n_rows = plan.n_rows
        self.n_cols = plan.n_cols
        self.max_row_nnz = int(plan.max_row_nnz)
        self.nnz = plan.nnz
        self.avg_nnz_per_row = float(self.nnz) / float(max(1, self.n_rows))
        self.op = str(op)
        self.alg = str(alg)
        self._row_lengths = None

    @property
    def row_lengths(self):
        if self._row_lengths is None:
            p = self.kernel_indptr.to(torch.int64)
            self._row_lengths = p[1:] - p[:-1] if self.n_rows > 0 else p.new_empty((0,))
        return self._row_lengths


def prepare_spmm_csr_route(data, indices, indptr, shape, *, op="non", alg="auto"):
    """Validate the matrix once (same contract and exceptions as ``flagsparse_spmm_csr``) and
    return the handle for ``flagsparse_spmm_csr_run``."""
    name = op_name(normalize_op(op))
    value_dtype = data.dtype if torch.is_tensor(data) else None
    plan = _checked_spmm_plan(data, indices, indptr, shape)
    resolved = _normalize_spmm_csr_alg(alg)
    if resolved != "auto":
        resolve_spmm_csr_algorithm(resolved, name, value_dtype)
    return PreparedCsrSpmmRoute(plan, shape, name, resolved, value_dtype)


def _transpose_dense(src, rows, cols, ld_src, dst, ld_dst):
    """dst (cols x rows, leading dimension ld_dst) = transpose of src (rows x cols, ld_src)."""
    st = _lib.load().b2s_dense_transpose(src.element_size(), _lib.ptr(src), rows, cols, ld_src,
                                         _lib.ptr(dst), ld_dst, _lib.stream_handle(src.device))
    _lib.check(st, "b2s_dense_transpose")


def flagsparse_spmm_csr_run(prepared, B, *, alg=None, op=None, dense_layout="auto",
                            return_time=False, return_meta=False, timing=False,
                            diagnostics=False):
    """C = op(A) @ B for a prepared matrix.

    dense_layout "row" (default): B is read row-major, C is a new row-major tensor.  "col":
    B is read column-major (a B in another layout is used as it is, the values are the same)
    and C comes back column-major, strides (1, n_rows); real dtypes and the "csr_base" route
    only, as in the reference.  Returns C, or C with ``operator_ms`` and / or the reference's
    meta dict when ``return_time`` / ``return_meta`` ask for them."""
    if not isinstance(prepared, PreparedCsrSpmmRoute):
        raise TypeError("prepared must be a PreparedCsrSpmmRoute instance")
    op_code = normalize_op(prepared.op if op is None else op)
    name = op_name(op_code)
    alg_name = prepared.alg if alg is None else _normalize_spmm_csr_alg(alg)
    dtype = prepared.data.dtype
    value_dtype = prepared.value_dtype
    algorithm = resolve_spmm_csr_algorithm(alg_name, name, value_dtype)
    layout = _normalize_dense_layout(dense_layout)
    if layout == "col" and algorithm != "csr_base":
        raise SpmmCsrAlgorithmUnavailable(
            "col-major layout is currently supported only by csr_base")
    if B is None or not torch.is_tensor(B):
        raise TypeError("B must be a torch.Tensor")
    if B.ndim != 2:
        raise ValueError("B must be a 2D dense tensor")
    if not B.is_cuda:
        raise ValueError("B must be a CUDA tensor")
    if B.device != prepared.data.device:
        raise ValueError("B must be on the same CUDA device as sparse matrix data")
    if B.dtype != value_dtype:
        raise TypeError("B dtype must match sparse matrix dtype")

    want_ms = bool(return_time or return_meta)
    if want_ms:
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    plan = prepared._plan
    op_process_gpu_ms = 0.0 if timing else None
    if op_transposes(op_code):
        if timing:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        plan = plan.transposed(conj=(op_code == OP_CONJ_TRANS))
        if timing:
            e1.record()
            torch.cuda.synchronize()
            op_process_gpu_ms = e0.elapsed_time(e1)
    if B.shape[0] != plan.n_cols:
        raise ValueError(f"B.shape[0] must be n_cols={plan.n_cols}, got {B.shape[0]}")
    if layout == "col" and is_complex(dtype):
        raise SpmmCsrAlgorithmUnavailable(
            "csr_base col-major layout does not support complex dtypes yet")

    n_rows, n_inner, n_dense = plan.n_rows, plan.n_cols, int(B.shape[1])
    device = plan.device
    if timing:
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
    empty = n_rows == 0 or n_dense == 0 or n_inner == 0
    if layout == "row":
        B_run = B if _row_major_ok(B) else B.contiguous()
        C = torch.empty((n_rows, n_dense), dtype=dtype, device=device)
        if empty:
            C.zero_()
        else:
            _launch_spmm(plan, B_run, C, None, 1.0, 0.0)
        b_stride = tuple(int(v) for v in B_run.stride())
    else:
        C = _empty_col_major(n_rows, n_dense, dtype, device)
        if _is_col_major_2d(B) and B.data_ptr() % B.element_size() == 0:
            b_stride = tuple(int(v) for v in B.stride())
        else:
            b_stride = (1, max(1, n_inner))  # what a column-major copy of B would have
        if empty:
            C.zero_()
        else:
            if _row_major_ok(B):
                B_run = B  # same values, already the layout the kernel reads
            elif _is_col_major_2d(B) and B.data_ptr() % B.element_size() == 0:
                B_run = torch.empty((n_inner, n_dense), dtype=dtype, device=device)
                with torch.cuda.device(device):
                    # column-major n_inner x n_dense = row-major n_dense x n_inner, ld = stride(1)
                    _transpose_dense(B, n_dense, n_inner, int(B.stride(1)), B_run, n_dense)
            else:
                B_run = B.contiguous()
            if not _launch_spmm_colmajor_c(plan, B_run, C):
                C_row = torch.empty((n_rows, n_dense), dtype=dtype, device=device)
                _launch_spmm(plan, B_run, C_row, None, 1.0, 0.0)
                with torch.cuda.device(device):
                    _transpose_dense(C_row, n_rows, n_dense, n_dense, C, int(C.stride(1)))
    compute_ms = None
    if timing:
        c1.record()
        torch.cuda.synchronize()
        compute_ms = c0.elapsed_time(c1)

    gpu_ms = None
    process_cpu_ms = 0.0
    if want_ms:
        end.record()
        torch.cuda.synchronize()
        gpu_ms = start.elapsed_time(end)
    operator_ms = (process_cpu_ms + float(gpu_ms)) if gpu_ms is not None else None
    meta = None
    if return_meta:
        meta = {
            "alg": algorithm,
            "display_name": SPMM_CSR_ALGORITHMS[algorithm][0],
            "op": name,
            "operator_ms": operator_ms,
            "gpu_ms": gpu_ms,
            "process_cpu_ms": process_cpu_ms,
            "dense_layout": layout,
            "b_stride": b_stride,
            "c_stride": tuple(int(v) for v in C.stride()),
            "output_layout": _dense_layout_name(C),
        }
        if timing:
            meta["process_gpu_ms"] = float(op_process_gpu_ms or 0.0)
            meta["compute_ms"] = compute_ms
        if diagnostics:
            meta["diagnostics"] = {
                "launch_config_scope": "matrix",
                "launch_config_count": 1,
                "bucket_count": 0,
                "long_row_count": 0,
                "launch_version": "b200_tile_v1",
                "dense_layout": layout,
                "b_stride": b_stride,
                "c_stride": tuple(int(v) for v in C.stride()),
                "output_layout": _dense_layout_name(C),
            }
    if return_time and return_meta:
        return C, operator_ms, meta
    if return_time:
        return C, operator_ms
    if return_meta:
        return C, meta
    return C
