"""CSR SpMM with FlagSparse's call signature, computed by libb200sparse.so.

Mirrors ``flagsparse.sparse_operations.spmm_csr``: ``flagsparse_spmm_csr`` (spmm_csr.py:3292-3448),
its input contract (:239-297, :3339-3364), the dense-column tile heuristic (:384-419 with
_alpha_spmm_alg1_common.py:6-23) and the op materialisation (:341-349).  ``alpha=1.0, beta=0.0``
are appended to the signature: C = alpha * op(A) @ B + beta * out.

The transpose needed by op = trans / conj is built once per matrix by the CSR -> CSC kernel and
kept with the matrix's plan; the reference rebuilds it with an argsort on every call
(spmm_csr.py:3374-3390).
"""

from __future__ import annotations

import time

import torch

from . import _lib
from ._contract import (
    ALL_VALUE_DTYPES,
    INDEX_LIMIT_INT32,
    OP_CONJ_TRANS,
    SUPPORTED_INDEX_DTYPES,
    SUPPORTED_VALUE_DTYPES,
    check_scalar,
    normalize_op,
    op_name,
    op_transposes,
)
from . import _plan as _plan_mod
from ._plan import (
    ST_DECREASING,
    ST_MAXCOL,
    ST_MAXLEN,
    ST_MINCOL,
    ST_PTR0,
    ST_PTRN,
    CsrPlan,
    cache_get,
    cache_put,
    inspect_csr,
    plan_key,
)

SUPPORTED_SPMM_VALUE_DTYPES = SUPPORTED_VALUE_DTYPES
SPMM_OP_NON, SPMM_OP_TRANS, SPMM_OP_CONJ_TRANS = 0, 1, 2
SPMM_OP_NAMES = {0: "non", 1: "trans", 2: "conj"}
_normalize_spmm_op = normalize_op
_spmm_op_to_name = op_name
_spmm_op_transposes = op_transposes


def _select_spmm_alg1_warp_and_factor(n_dense_cols):
    """Dense-column tile of the reference's base kernel (_alpha_spmm_alg1_common.py:6-23):
    (lanes, factor) with BLOCK_N = lanes * factor."""
    n = int(n_dense_cols)
    if n > 64:
        return 32, 4
    if n > 32:
        return 32, 2
    if n > 16:
        return 32, 1
    if n > 8:
        return 16, 1
    if n > 4:
        return 8, 1
    return 4, 1


def _resolve_spmm_alg1_launch_config(n_dense_cols, max_row_nnz, block_n=None, block_nnz=None,
                                     max_segments=None):
    """Validate the tuning overrides the way spmm_csr.py:384-419 does.  The values are reported
    back but the B200 kernel picks its own tile (16 bytes per lane, see b2s_spmm.cu)."""
    warp_size, factor = _select_spmm_alg1_warp_and_factor(n_dense_cols)
    if block_n is None:
        block_n = warp_size * factor
    if block_nnz is None:
        block_nnz = warp_size
    if block_n <= 0 or block_nnz <= 0:
        raise ValueError("block_n and block_nnz must be positive when provided")
    if max_segments is not None and max_segments <= 0:
        raise ValueError("max_segments must be positive when provided")
    required = -(-int(max_row_nnz) // int(block_nnz)) if max_row_nnz > 0 else 0
    if max_segments is not None and required > int(max_segments):
        raise ValueError(
            "row nnz requires more CSR segments than the explicit max_segments override allows: "
            f"required {required}, provided {int(max_segments)}")
    return {
        "block_n": int(block_n), "block_nnz": int(block_nnz),
        "max_segments": None if max_segments is None else int(max_segments),
        "required_segments": int(required), "warp_size": int(warp_size), "factor": int(factor),
        "max_row_nnz": int(max_row_nnz), "auto_max_segments": max_segments is None,
    }


# -------------------------------------------------------------------------------------------------
# input contract  (spmm_csr.py:239-297)
# -------------------------------------------------------------------------------------------------
def _checked_spmm_plan(data, indices, indptr, shape):
    if len(shape) != 2:
        raise ValueError("shape must be a 2-tuple: (n_rows, n_cols)")
    if data.ndim != 1 or indices.ndim != 1 or indptr.ndim != 1:
        raise ValueError("data, indices, and indptr must be 1D tensors")
    n_rows, n_cols = int(shape[0]), int(shape[1])
    if n_rows < 0 or n_cols < 0:
        raise ValueError("shape dimensions must be non-negative")
    if indptr.numel() != n_rows + 1:
        raise ValueError(f"indptr length must be n_rows+1={n_rows + 1}, got {indptr.numel()}")
    if data.numel() != indices.numel():
        raise ValueError("data and indices must have the same length (nnz)")
    if not all(t.is_cuda for t in (data, indices, indptr)):
        raise ValueError("data, indices, and indptr must be CUDA tensors")
    if not all(t.device == data.device for t in (indices, indptr)):
        raise ValueError("data, indices, and indptr must be on the same CUDA device")
    if data.dtype not in ALL_VALUE_DTYPES:
        raise TypeError(
            "data dtype must be one of: float16, bfloat16, float32, float64, complex64, "
            "complex128")
    if indices.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError("indices dtype must be torch.int32 or torch.int64")
    if indptr.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError("indptr dtype must be torch.int32 or torch.int64")

    key = plan_key("spmm", data, indices, indptr, (n_rows, n_cols))
    plan = cache_get(key)
    if plan is not None:
        return plan

    d, i, p = data.contiguous(), indices.contiguous(), indptr.contiguous()
    if d.data_ptr() % d.element_size():
        d = d.clone()
    nnz = d.numel()
    stats = inspect_csr(i, p, n_rows, nnz)
    if stats[ST_PTR0] != 0:
        raise ValueError("indptr[0] must be 0")
    if stats[ST_PTRN] != nnz:
        raise ValueError(f"indptr[-1] must equal nnz={nnz}, got {stats[ST_PTRN]}")
    if stats[ST_DECREASING] != 0:
        raise ValueError("indptr must be nondecreasing")
    if nnz > 0:
        if stats[ST_MINCOL] < 0 or stats[ST_MAXCOL] >= n_cols:
            raise IndexError("indices out of range for n_cols")
        if stats[ST_MAXCOL] > INDEX_LIMIT_INT32:
            # kept for drop-in behaviour (spmm_csr.py:280-283); the kernels themselves take int64
            raise ValueError(
                "column indices exceed the int32 range supported by the Triton kernel")
    if i.dtype == torch.int64:
        # the columns fit int32 (checked above); like the reference (spmm_csr.py:289) the kernels
        # read a narrowed copy: half the index stream, smaller staging buffers, more CTAs per SM
        i = i.to(torch.int32)
    plan = CsrPlan(d, i, p, (n_rows, n_cols), stats[ST_MAXLEN],
                   keepalive=(data, indices, indptr))
    cache_put(key, plan)
    return plan


def _launch_spmm(plan: CsrPlan, B, C, C_in, alpha, beta):
    """Enqueue C = alpha * A B + beta * C_in on the current stream (no synchronisation).

    When B is too large for L2 and the matrix has long rows that hold a good share of the
    non-zeros, the product runs in three launches: the matrix without its long rows (which also
    puts beta * C_in into the long rows of C), the long rows as a stack of column panels into
    one partial row per (panel, long row), and the sum of those partials into C."""
    n_dense = int(B.shape[1])
    split = plan.long_row_split(n_dense * B.element_size())
    if split is None:
        _launch_spmm_plain(plan, B, C, C_in, alpha, beta)
        return
    lib = _lib.load()
    _launch_spmm_plain(split.short, B, C, C_in, alpha, beta)
    stack = split.stack
    part = stack.scratch("spmm_long_part", stack.n_rows * n_dense).view(stack.n_rows, n_dense)
    _launch_spmm_plain(stack, B, part, None, 1.0, 0.0)
    a = _lib.scalar_buffer(alpha, plan.data.dtype)
    with torch.cuda.device(plan.device):
        st = lib.b2s_spmm_rows_combine(
            plan.vcode, _lib.ptr(part), _lib.ptr(split.subpos), _lib.ptr(split.rows),
            split.n_long, split.n_panels, n_dense, _lib.ptr(C), int(C.stride(0)), a,
            _lib.stream_handle(plan.device))
    _lib.check(st, "b2s_spmm_rows_combine")


def _launch_spmm_colmajor_c(plan: CsrPlan, B, C):
    """Enqueue C = A B with C column-major (strides (1, ldc_col)): the kernel stores column-major
    itself (b2s_spmm_csr_colmajor_c).  Returns False, having done nothing, when the matrix runs
    with its long rows split off (that route combines row-major partials); the caller then
    takes the row-major product and transposes it."""
    n_dense = int(B.shape[1])
    if plan.long_row_split(n_dense * B.element_size()) is not None:
        return False
    lib = _lib.load()
    items = lib.b2s_spmm_tile_items(plan.vcode, plan.icode)
    n_tiles, tile_row = plan.tiles(items)
    carry = plan.carry_on("spmm_carry", n_tiles * n_dense,
                          torch.cuda.current_stream(plan.device).cuda_stream)
    dtype = plan.data.dtype
    a, b = _lib.scalar_buffer(1.0, dtype), _lib.scalar_buffer(0.0, dtype)
    with torch.cuda.device(plan.device):
        st = lib.b2s_spmm_csr_colmajor_c(
            plan.vcode, plan.icode, plan.pcode,
            _lib.ptr(plan.data), _lib.ptr(plan.indices), _lib.ptr(plan.indptr),
            plan.n_rows, plan.n_cols, plan.nnz, _lib.ptr(B), int(B.stride(0)), n_dense,
            None, _lib.ptr(C), int(C.stride(1)), a, b, _lib.ptr(tile_row), _lib.ptr(carry),
            _lib.ptr(plan.status), _lib.stream_handle(plan.device))
    _lib.check(st, "b2s_spmm_csr_colmajor_c")
    plan.note_launch()
    return True


def _launch_spmm_plain(plan: CsrPlan, B, C, C_in, alpha, beta):
    """One b2s_spmm_csr launch for the matrix of `plan` as it is."""
    lib = _lib.load()
    n_dense = int(B.shape[1])
    dtype = plan.data.dtype
    # banded / local matrices: when the B rows of every tile fit a shared-memory window the
    # kernel copies them there once per tile and gathers from shared memory; that kernel has its
    # own tile length, so the window is settled before the tile plan is picked
    window, table = 0, None
    items = lib.b2s_spmm_tile_items(plan.vcode, plan.icode)
    pitch = int(B.stride(0)) * B.element_size()
    if (_plan_mod.WINDOW_POLICY == "auto" and 0 < pitch <= _plan_mod.WINDOW_MAX_BYTES
            and dtype in SUPPORTED_VALUE_DTYPES):
        w_items = lib.b2s_spmm_window_tile_items(plan.vcode, plan.icode)
        rows, w_table = plan.window(w_items)
        if w_table is not None and rows > 0 and lib.b2s_spmm_window_usable(
                plan.vcode, _lib.ptr(B), int(B.stride(0)), n_dense, _lib.ptr(C_in), _lib.ptr(C),
                int(C.stride(0)), plan.n_cols, rows):
            window, table, items = rows, w_table, w_items
    n_tiles, tile_row = plan.tiles(items)
    carry = plan.carry_on("spmm_carry", n_tiles * n_dense,
                          torch.cuda.current_stream(plan.device).cuda_stream)
    a = _lib.scalar_buffer(alpha, dtype)
    b = _lib.scalar_buffer(beta, dtype)
    with torch.cuda.device(plan.device):
        st = lib.b2s_spmm_csr_windowed(
            plan.vcode, plan.icode, plan.pcode,
            _lib.ptr(plan.data), _lib.ptr(plan.indices), _lib.ptr(plan.indptr),
            plan.n_rows, plan.n_cols, plan.nnz,
            _lib.ptr(B), int(B.stride(0)), n_dense,
            _lib.ptr(C_in), _lib.ptr(C), int(C.stride(0)), a, b,
            _lib.ptr(tile_row), _lib.ptr(carry), _lib.ptr(plan.status), window,
            _lib.ptr(table) if window else None, _lib.stream_handle(plan.device))
    _lib.check(st, "b2s_spmm_csr")
    plan.note_launch()


def _row_major_ok(t):
    return (t.ndim == 2 and (t.shape[1] <= 1 or t.stride(1) == 1)
            and (t.shape[0] <= 1 or t.stride(0) >= max(int(t.shape[1]), 1))
            and t.data_ptr() % t.element_size() == 0)


def flagsparse_spmm_csr(data, indices, indptr, B, shape, block_n=None, block_nnz=None,
                        max_segments=None, out=None, return_time=False, transpose=None, op=None,
                        return_meta=False, alpha=1.0, beta=0.0):
    """CSR SpMM on B200: C = alpha * op(A) @ B + beta * out.

    op: 0/'non' for A @ B, 1/'trans' for A.T @ B, 2/'conj' for A.conj().T @ B.
    B is read row-major (a non-contiguous B is copied once); C is row-major.
    alpha, beta default to 1, 0 (the reference's behaviour); beta != 0 needs ``out``.
    """
    op_explicit = op is not None
    op_code = normalize_op(op, transpose=False if transpose is None else bool(transpose))
    if op_explicit and transpose is not None and bool(transpose) != op_transposes(op_code):
        raise ValueError("transpose conflicts with op")
    if block_n is not None and block_n <= 0:
        raise ValueError("block_n must be positive when provided")
    if block_nnz is not None and block_nnz <= 0:
        raise ValueError("block_nnz must be positive when provided")
    if max_segments is not None and max_segments <= 0:
        raise ValueError("max_segments must be positive when provided")

    plan = _checked_spmm_plan(data, indices, indptr, shape)
    if B.ndim != 2:
        raise ValueError("B must be a 2D dense tensor")
    transposes = op_transposes(op_code)
    eff_rows, eff_cols = (plan.n_cols, plan.n_rows) if transposes else (plan.n_rows, plan.n_cols)
    if B.shape[0] != eff_cols:
        raise ValueError(f"B.shape[0] must be n_cols={eff_cols}, got {B.shape[0]}")
    if not B.is_cuda:
        raise ValueError("B must be a CUDA tensor")
    if B.device != plan.device:
        raise ValueError("B must be on the same CUDA device as the sparse matrix")
    if B.dtype != plan.data.dtype:
        raise TypeError("B dtype must match data dtype")
    if not _row_major_ok(B):
        B = B.contiguous()
    n_dense = int(B.shape[1])
    dtype = plan.data.dtype
    alpha = check_scalar(alpha, dtype, "alpha")
    beta = check_scalar(beta, dtype, "beta")

    if out is not None:
        if not out.is_cuda:
            raise ValueError("out must be a CUDA tensor")
        if out.device != plan.device:
            raise ValueError("out must be on the same CUDA device as the inputs")
        if out.shape != (eff_rows, n_dense) or out.dtype != dtype:
            raise ValueError("out shape/dtype must match result")
    elif beta != 0:
        raise ValueError("beta != 0 requires out= holding the matrix to scale")

    do_timing = bool(return_time or return_meta)
    symbolic_ms = 0.0 if do_timing else None
    compute_ms = None
    op_total_ms = None
    if do_timing:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
    run_plan = plan
    if transposes:
        run_plan = plan.transposed(conj=(op_code == OP_CONJ_TRANS))
    if do_timing:
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        symbolic_ms = (t1 - t0) * 1000.0 if transposes else 0.0

    if max_segments is not None or block_n is not None or block_nnz is not None:
        if run_plan.max_row_nnz < 0:
            run_plan.max_row_nnz = inspect_csr(run_plan.indices, run_plan.indptr,
                                               run_plan.n_rows, run_plan.nnz)[ST_MAXLEN]
        _resolve_spmm_alg1_launch_config(n_dense, run_plan.max_row_nnz, block_n=block_n,
                                         block_nnz=block_nnz, max_segments=max_segments)
    if do_timing:
        torch.cuda.synchronize()
        t1 = time.perf_counter()

    direct = out is not None and _row_major_ok(out)
    C = out if direct else torch.empty((eff_rows, n_dense), dtype=dtype, device=plan.device)
    if eff_rows == 0 or n_dense == 0 or eff_cols == 0:
        # spmm_csr.py:2706-2710: empty problem -> zeros (scaled prior contents with beta)
        if out is not None and beta != 0:
            out.mul_(beta)
            C = out
        else:
            C.zero_()
    else:
        C_in = None
        if beta != 0:
            C_in = out if direct else out.contiguous()
        _launch_spmm(run_plan, B, C, C_in, alpha, beta)
    if out is not None and not direct:
        out.copy_(C)
    if out is not None:
        C = out
    if do_timing:
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        compute_ms = (t2 - t1) * 1000.0
        op_total_ms = symbolic_ms + compute_ms

    if return_meta:
        meta = {
            "symbolic_ms": symbolic_ms,
            "compute_ms": compute_ms,
            "op_total_ms": op_total_ms,
            "op": op_name(op_code),
        }
        if return_time:
            return C, op_total_ms, meta
        return C, meta
    if return_time:
        return C, op_total_ms
    return C


spmm_csr = flagsparse_spmm_csr
