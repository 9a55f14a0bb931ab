"""Every measured configuration at its full benchmark size, with the code paths that only switch
on at that size asserted active: the column-panel stack and the shared-memory long-row kernel of
SpMV, the long-row split of SpMM, int64 columns narrowed for SpMM, the cached transpose with
conjugation.

The independent product is torch's own CSR multiplication (cuSPARSE) in float64 / complex128:
rows are independent, so rel-L2 over the whole result is the same measure the reference's
accuracy checks use (tests/pytest/test_spmv_csr_accuracy.py:98-125, tolerances
tests/pytest/accuracy_utils.py:17-30).  Where the unmodified reference is installed beside the
repository (baseline/_ref) it is also run on a row slice that contains the longest rows: its
kernel walks ceil(longest row / 256) segments for EVERY row of the matrix it is given
(spmv_csr.py:183), so the slice keeps that affordable.

Tolerances: rel-L2 <= 1e-5 for float32 / complex64, <= 1e-12 for float64.
"""

from __future__ import annotations

import gc
import importlib
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

_REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                        "baseline", "_ref")


def _rel_l2(got, want):
    wide = torch.complex128 if want.is_complex() else torch.float64
    diff = got.to(wide) - want
    denom = float(torch.linalg.vector_norm(want))
    return float(torch.linalg.vector_norm(diff)) / (denom if denom > 0 else 1.0)


def _torch_csr(p, conj=False):
    wide = torch.complex128 if p.data.is_complex() else torch.float64
    vals = p.data.to(wide)
    if conj:
        vals = vals.conj().resolve_conj()
    return torch.sparse_csr_tensor(p.indptr.long(), p.indices.long(), vals, size=p.shape)


def _free():
    from flagsparse_b200 import clear_plan_cache
    clear_plan_cache()
    gc.collect()
    torch.cuda.empty_cache()


def _plan_of(kind, p):
    from flagsparse_b200 import _plan
    plan = _plan.cache_get(_plan.plan_key(kind, p.data, p.indices, p.indptr, p.shape))
    assert plan is not None
    return plan


def _reference_or_none():
    if not os.path.isdir(os.path.join(_REF_DIR, "flagsparse")):
        return None
    sys.path.insert(0, _REF_DIR)
    try:
        return importlib.import_module("flagsparse")
    except Exception:  # noqa: BLE001 - a reference that does not import is not a failure here
        return None
    finally:
        sys.path.remove(_REF_DIR)


def _slice_with_longest_rows(p, n_rows_slice=4096):
    """Rows [r0, r0 + n) around the longest row, as a CSR triple with indptr re-based to 0."""
    lens = (p.indptr[1:] - p.indptr[:-1]).long()
    longest = int(torch.argmax(lens))
    r0 = max(0, min(longest - n_rows_slice // 2, p.shape[0] - n_rows_slice))
    r1 = r0 + n_rows_slice
    j0, j1 = int(p.indptr[r0]), int(p.indptr[r1])
    return (r0, r1, p.data[j0:j1].clone(), p.indices[j0:j1].clone(),
            (p.indptr[r0:r1 + 1] - p.indptr[r0]).clone())


def test_cfg2_spmv_full_size_runs_on_the_panel_stack_and_the_long_row_kernel():
    from flagsparse_b200 import flagsparse_spmv_csr, workloads
    _free()
    p = workloads.cfg2_powerlaw_spmv(device="cuda")
    out = p.y0.clone()
    y = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, out=out, alpha=p.alpha,
                            beta=p.beta)
    lay = _plan_of("spmv", p).panels()
    assert lay is not None and lay.n_panels == 4
    assert lay.long_rows is not None and lay.long_rows.n_long > 1000
    want = p.alpha * (_torch_csr(p) @ p.x) + p.beta * p.y0
    assert _rel_l2(y, want) <= 1e-12
    ref = _reference_or_none()
    if ref is not None:
        r0, r1, d, i, ptr = _slice_with_longest_rows(p)
        want_slice = ref.flagsparse_spmv_csr(d, i, ptr, p.x, (r1 - r0, p.shape[1]))
        plain = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape)
        assert _rel_l2(plain[r0:r1], want_slice.double()) <= 1e-12
    _free()


def test_cfg5_spmv_full_size_float32_int64():
    """2^26 x 2^26, 1.07 G non-zeros: eight column panels of 2^23 columns; more than 2^31 / 16
    stacked rows, a position table of 2^29 entries."""
    from flagsparse_b200 import flagsparse_spmv_csr, workloads
    _free()
    p = workloads.cfg5_scaling(device="cuda", with_B=False)
    assert p.nnz > 1_000_000_000 and p.indices.dtype == torch.int64
    y = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape)
    lay = _plan_of("spmv", p).panels()
    assert lay is not None and lay.n_panels == 8
    again = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape)
    assert torch.equal(y, again)
    ref = _reference_or_none()
    if ref is not None:
        r0, r1, d, i, ptr = _slice_with_longest_rows(p)
        want_slice = ref.flagsparse_spmv_csr(d, i, ptr, p.x, (r1 - r0, p.shape[1]))
        assert _rel_l2(y[r0:r1], want_slice.double()) <= 1e-5
    _free()                                   # room for the float64 copy torch multiplies
    want = _torch_csr(p) @ p.x.double()
    assert _rel_l2(y, want) <= 1e-5
    del want
    _free()


def test_cfg5_spmm_full_size_n16_narrowed_columns_and_long_row_split():
    from flagsparse_b200 import flagsparse_spmm_csr, workloads
    _free()
    p = workloads.cfg5_scaling(device="cuda")
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    plan = _plan_of("spmm", p)
    assert plan.indices.dtype == torch.int32          # int64 columns narrowed once (1.07 G)
    assert plan.long_row_split(16 * 4) is not None
    _free()
    A = _torch_csr(p)
    err2, ref2 = 0.0, 0.0
    for c0 in range(0, 16, 4):                        # four columns of B at a time: memory
        want = A @ p.B[:, c0:c0 + 4].double()
        err2 += float(torch.linalg.matrix_norm(C[:, c0:c0 + 4].double() - want)) ** 2
        ref2 += float(torch.linalg.matrix_norm(want)) ** 2
        del want
    assert (err2 / ref2) ** 0.5 <= 1e-5
    _free()


def test_cfg2_matrix_spmm_n32_full_size_with_the_long_rows_split_off():
    from flagsparse_b200 import flagsparse_spmm_csr, workloads
    _free()
    p = workloads.cfg2_powerlaw_spmv(device="cuda", n_dense=32)
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    split = _plan_of("spmm", p).long_row_split(32 * 8)
    assert split is not None and split.n_long > 1000 and split.n_panels >= 64
    want = _torch_csr(p) @ p.B
    assert _rel_l2(C, want) <= 1e-12
    del want
    assert torch.equal(C, flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape))
    _free()


def test_cfg4_conj_complex64_full_size():
    from flagsparse_b200 import flagsparse_spmm_csr, workloads
    _free()
    p = workloads.cfg4_poisson_spmm(device="cuda", dtype=torch.complex64)
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape, op="conj")
    assert C.shape == (p.shape[1], p.B.shape[1])
    A_h = _torch_csr(p, conj=True).to_sparse_coo().t().coalesce()
    want = A_h @ p.B.to(torch.complex128)
    assert _rel_l2(C, want) <= 1e-5
    _free()
