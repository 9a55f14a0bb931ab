"""The CPU oracle against (a) outputs of FlagSparse's own kernels (tests/golden/*.npz, made by
tests/golden/make_golden.py) and (b) scipy.sparse in float64 / complex128."""

import numpy as np
import pytest
import scipy.sparse as sp

import oracle
from conftest import ALLCLOSE_TOL, REL_L2_TOL, load_golden

SPMV_CASES = sorted(load_golden("spmv_reference.npz"))
SPMM_CASES = sorted(load_golden("spmm_reference.npz"))


def _op_of(case):
    return case.rsplit("_", 1)[1]


def _shape_of(case, c):
    n_rows = c["indptr"].shape[0] - 1
    if case.startswith("spmv_longrows"):
        return n_rows, 3000
    if case.startswith("spmm_longrow"):
        return n_rows, 2048
    dims = case.split("_")[1].split("x")
    return n_rows, int(dims[1])


@pytest.mark.parametrize("case", SPMV_CASES)
def test_oracle_spmv_matches_reference_kernels(case, spmv_golden):
    c = spmv_golden[case]
    op = _op_of(case)
    shape = _shape_of(case, c)
    y = oracle.spmv(c["data"], c["indices"], c["indptr"], c["x"], shape, op=op)
    assert y.dtype == c["y"].dtype
    tol = ALLCLOSE_TOL[y.dtype]
    assert np.allclose(y, c["y"], rtol=tol, atol=tol)
    assert oracle.rel_l2(y, c["y"]) <= REL_L2_TOL[y.dtype] * 0.1
    if y.dtype in (np.float32, np.float64):
        # same promotion, same segment structure: at most the last bit may differ
        assert np.max(np.abs(y - c["y"])) <= 4 * np.finfo(y.dtype).eps * max(
            1.0, float(np.max(np.abs(c["y"]))))


@pytest.mark.parametrize("case", [c for c in SPMV_CASES if not c.endswith("_non")])
def test_oracle_transpose_is_bit_identical_to_reference(case, spmv_golden):
    c = spmv_golden[case]
    shape = _shape_of(case, c)
    t_data, t_idx, t_ptr, t_shape = oracle.transpose_csr(
        c["data"], c["indices"], c["indptr"], shape, conj=_op_of(case) == "conj")
    assert t_shape == (shape[1], shape[0])
    assert np.array_equal(t_ptr, c["t_indptr"])
    assert np.array_equal(t_idx, c["t_indices"])
    assert np.array_equal(t_data.view(np.uint8), c["t_data"].view(np.uint8))


@pytest.mark.parametrize("case", SPMM_CASES)
def test_oracle_spmm_matches_reference_kernels(case, spmm_golden):
    c = spmm_golden[case]
    op = _op_of(case)
    shape = _shape_of(case, c)
    if case.startswith("spmm_") and not case.startswith("spmm_longrow"):
        M, K, _ = (int(v) for v in case.split("_")[1].split("x"))
        shape = (M, K)
    C = oracle.spmm(c["data"], c["indices"], c["indptr"], c["B"], shape, op=op)
    tol = ALLCLOSE_TOL[C.dtype]
    assert np.allclose(C, c["C"], rtol=tol, atol=tol)
    assert oracle.rel_l2(C, c["C"]) <= REL_L2_TOL[C.dtype] * 0.1


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.complex64, np.complex128])
@pytest.mark.parametrize("op", ["non", "trans", "conj"])
def test_oracle_matches_scipy(dtype, op):
    rng = np.random.default_rng(7)
    A = sp.random(257, 193, density=0.04, format="csr", random_state=3, dtype=np.float64)
    data = A.data.astype(dtype)
    if np.issubdtype(dtype, np.complexfloating):
        data = (data + 1j * rng.standard_normal(A.nnz)).astype(dtype)
    M = sp.csr_matrix((data, A.indices, A.indptr), shape=A.shape)
    Mop = {"non": M, "trans": M.T, "conj": M.conj().T}[op].astype(np.complex128)
    k = Mop.shape[1]
    x = rng.standard_normal(k).astype(dtype)
    B = rng.standard_normal((k, 7)).astype(dtype)
    y0 = rng.standard_normal(Mop.shape[0]).astype(dtype)
    y = oracle.spmv(data, A.indices, A.indptr, x, A.shape, op=op, alpha=1.5, beta=0.5, y0=y0)
    ref = 1.5 * (Mop @ x.astype(np.complex128)) + 0.5 * y0
    assert oracle.rel_l2(y, ref) <= REL_L2_TOL[np.dtype(dtype)] * 0.1
    C = oracle.spmm(data, A.indices, A.indptr, B, A.shape, op=op)
    assert oracle.rel_l2(C, Mop @ B.astype(np.complex128)) <= REL_L2_TOL[np.dtype(dtype)] * 0.1


def test_oracle_edge_cases():
    # empty rows, duplicate and unsorted columns, an empty matrix
    data = np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float64)
    idx = np.array([2, 0, 0, 1])
    ptr = np.array([0, 0, 3, 3, 4])
    x = np.array([1.0, 10.0, 100.0])
    assert np.array_equal(oracle.spmv(data, idx, ptr, x, (4, 3)), [0.0, 105.0, 0.0, 40.0])
    y = oracle.spmv(data[:0], idx[:0], np.zeros(4, dtype=np.int64), x, (3, 3))
    assert np.array_equal(y, np.zeros(3))
    t_data, t_idx, t_ptr, _ = oracle.transpose_csr(data, idx, ptr, (4, 3))
    assert t_ptr.tolist() == [0, 2, 3, 4]
    assert t_idx.tolist() == [1, 1, 3, 1]
    assert t_data.tolist() == [2.0, 3.0, 4.0, 1.0]
