"""GPU parity of the prepared SpMM route API (prepare_spmm_csr_route / flagsparse_spmm_csr_run,
reference spmm_csr.py:2040-2174) against the CPU oracle: row- and column-major dense operands,
the three ops, the meta dict, and the exceptions the reference raises for the same misuse.
Tolerance: rel-L2 <= 1e-5 (float32 / complex64), <= 1e-12 (float64 / complex128)."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import assert_parity, csr_from_lengths, dev, host, random_values

pytestmark = pytest.mark.gpu

REAL = [np.float32, np.float64]
ALL = [np.float32, np.float64, np.complex64, np.complex128]


def _problem(rng, dtype, n_rows=1300, n_cols=900):
    lengths = np.concatenate([[0, 1, 40, 0, 2500], rng.integers(0, 24, n_rows - 5)])
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype, sort=False)
    return data, idx, ptr, (n_rows, n_cols)


def _col_major(t):
    """A column-major device copy of a 2-D tensor (strides (1, rows))."""
    out = torch.empty_strided(t.shape, (1, max(1, t.shape[0])), dtype=t.dtype, device=t.device)
    out.copy_(t)
    return out


@pytest.mark.parametrize("dtype", ALL, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("op", ["non", "trans", "conj"])
def test_route_row_major_matches_oracle_and_the_plain_call(dtype, op):
    from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmm_csr_run, prepare_spmm_csr_route
    rng = np.random.default_rng(5)
    data, idx, ptr, shape = _problem(rng, dtype)
    k = shape[0] if op != "non" else shape[1]
    B = random_values(rng, k * 24, dtype).reshape(k, 24)
    d, i, p = dev(data), dev(idx, torch.int32), dev(ptr, torch.int64)
    prepared = prepare_spmm_csr_route(d, i, p, shape, op=op)
    assert (prepared.n_rows, prepared.n_cols, prepared.nnz) == (*shape, data.size)
    assert prepared.max_row_nnz == 2500 and prepared.op == op and prepared.alg == "auto"
    assert int(prepared.row_lengths.sum()) == data.size
    C = flagsparse_spmm_csr_run(prepared, dev(B))
    assert C.is_contiguous()
    assert_parity(host(C), oracle.spmm(data, idx, ptr, B, shape, op=op), dtype)
    plain = flagsparse_spmm_csr(d, i, p, dev(B), shape, op=op)
    assert torch.equal(C.view(torch.uint8), plain.view(torch.uint8))
    # the op given at run time overrides the prepared one
    k2 = shape[1]
    B2 = random_values(rng, k2 * 5, dtype).reshape(k2, 5)
    C2 = flagsparse_spmm_csr_run(prepared, dev(B2), op="non")
    assert_parity(host(C2), oracle.spmm(data, idx, ptr, B2, shape, op="non"), dtype)


@pytest.mark.parametrize("dtype", REAL, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("n_dense", [1, 7, 32, 33, 70])
@pytest.mark.parametrize("op", ["non", "trans"])
def test_route_column_major_matches_oracle(dtype, n_dense, op):
    from flagsparse_b200 import flagsparse_spmm_csr_run, prepare_spmm_csr_route
    rng = np.random.default_rng(40 + n_dense)
    data, idx, ptr, shape = _problem(rng, dtype, n_rows=1111, n_cols=777)
    k = shape[0] if op != "non" else shape[1]
    B = random_values(rng, k * n_dense, dtype).reshape(k, n_dense)
    expect = oracle.spmm(data, idx, ptr, B, shape, op=op)
    prepared = prepare_spmm_csr_route(dev(data), dev(idx, torch.int64), dev(ptr, torch.int64),
                                      shape, op=op, alg="base")
    n_out = expect.shape[0]
    for B_dev in (_col_major(dev(B)), dev(B)):  # a true column-major B and a row-major one
        C, meta = flagsparse_spmm_csr_run(prepared, B_dev, dense_layout="col", return_meta=True)
        assert C.shape == (n_out, n_dense) and C.stride() == (1, max(1, n_out))
        assert_parity(host(C), expect, dtype)
        assert meta["dense_layout"] == "col" and meta["c_stride"] == (1, n_out)
        assert meta["b_stride"] == (1, k) and meta["alg"] == "csr_base" and meta["op"] == op
        assert meta["output_layout"] == ("col" if n_dense > 1 else "row")
    # a column-major B with padding between its columns (leading dimension > rows)
    wide = torch.empty_strided((k, n_dense), (1, k + 3), dtype=B_dev.dtype, device="cuda")
    wide.copy_(dev(B))
    C = flagsparse_spmm_csr_run(prepared, wide, dense_layout="F")
    assert_parity(host(C), expect, dtype)
    row = flagsparse_spmm_csr_run(prepared, dev(B), dense_layout="row")
    assert torch.equal(C, row)  # same kernel, same order of additions: equal value by value


def test_route_meta_and_timing_keys():
    from flagsparse_b200 import flagsparse_spmm_csr_run, prepare_spmm_csr_route
    rng = np.random.default_rng(2)
    data, idx, ptr, shape = _problem(rng, np.float32)
    prepared = prepare_spmm_csr_route(dev(data), dev(idx, torch.int32), dev(ptr, torch.int32),
                                      shape, alg="alg1")
    B = dev(random_values(rng, shape[1] * 8, np.float32).reshape(shape[1], 8))
    C, ms, meta = flagsparse_spmm_csr_run(prepared, B, return_time=True, return_meta=True,
                                          timing=True, diagnostics=True)
    assert ms == meta["operator_ms"] and ms > 0 and meta["gpu_ms"] > 0
    assert meta["alg"] == "spmm_csr_alg1" and meta["display_name"] == "Alg1"
    for key in ("op", "process_cpu_ms", "dense_layout", "b_stride", "c_stride", "output_layout",
                "process_gpu_ms", "compute_ms", "diagnostics"):
        assert key in meta
    assert meta["b_stride"] == (8, 1) and meta["c_stride"] == (8, 1)
    C2, ms2 = flagsparse_spmm_csr_run(prepared, B, return_time=True)
    assert torch.equal(C, C2) and ms2 > 0


def test_route_rejects_what_the_reference_rejects():
    from flagsparse_b200 import (SpmmCsrAlgorithmUnavailable, flagsparse_spmm_csr_run,
                                 prepare_spmm_csr_route)
    rng = np.random.default_rng(3)
    data, idx, ptr, shape = _problem(rng, np.float32)
    d, i, p = dev(data), dev(idx, torch.int32), dev(ptr, torch.int32)
    prepared = prepare_spmm_csr_route(d, i, p, shape)
    B = dev(random_values(rng, shape[1] * 4, np.float32).reshape(shape[1], 4))
    with pytest.raises(TypeError, match="PreparedCsrSpmmRoute"):
        flagsparse_spmm_csr_run(object(), B)
    with pytest.raises(TypeError, match="torch.Tensor"):
        flagsparse_spmm_csr_run(prepared, None)
    with pytest.raises(ValueError, match="2D"):
        flagsparse_spmm_csr_run(prepared, B[:, 0])
    with pytest.raises(ValueError, match="CUDA"):
        flagsparse_spmm_csr_run(prepared, B.cpu())
    with pytest.raises(TypeError, match="dtype"):
        flagsparse_spmm_csr_run(prepared, B.double())
    with pytest.raises(ValueError, match="n_cols"):
        flagsparse_spmm_csr_run(prepared, B[:-1])
    with pytest.raises(ValueError, match="dense_layout"):
        flagsparse_spmm_csr_run(prepared, B, dense_layout="diagonal")
    with pytest.raises(ValueError, match="unsupported CSR SpMM algorithm"):
        flagsparse_spmm_csr_run(prepared, B, alg="magic")
    with pytest.raises(SpmmCsrAlgorithmUnavailable, match="only by csr_base"):
        flagsparse_spmm_csr_run(prepared, B, alg="alg2", dense_layout="col")
    with pytest.raises(ValueError):
        prepare_spmm_csr_route(d, i, p, shape, op="sideways")
    cd = dev(random_values(rng, data.size, np.complex64))
    with pytest.raises(TypeError, match="does not support dtype"):
        prepare_spmm_csr_route(cd, i, p, shape, alg="alg1")
    cprep = prepare_spmm_csr_route(cd, i, p, shape)
    cB = dev(random_values(rng, shape[1] * 4, np.complex64).reshape(shape[1], 4))
    with pytest.raises(SpmmCsrAlgorithmUnavailable, match="complex"):
        flagsparse_spmm_csr_run(cprep, cB, dense_layout="col")


def test_route_empty_problems_give_zeros():
    from flagsparse_b200 import flagsparse_spmm_csr_run, prepare_spmm_csr_route
    ptr = torch.zeros(5, dtype=torch.int64, device="cuda")
    none = torch.zeros(0, device="cuda")
    prepared = prepare_spmm_csr_route(none, none.to(torch.int64), ptr, (4, 6))
    B = torch.ones(6, 3, device="cuda")
    for layout in ("row", "col"):
        C = flagsparse_spmm_csr_run(prepared, B, dense_layout=layout)
        assert C.shape == (4, 3) and float(C.abs().sum()) == 0.0
    C = flagsparse_spmm_csr_run(prepared, torch.ones(6, 0, device="cuda"), dense_layout="col")
    assert C.shape == (4, 0)


def test_dense_transpose_entry_point():
    """b2s_dense_transpose on ragged tile edges for the three element sizes, with leading
    dimensions larger than the rows, and its argument checks."""
    from flagsparse_b200 import _lib as L
    lib = L.load()
    stream = L.stream_handle(torch.device("cuda", 0))
    for dtype in (torch.float16, torch.float32, torch.float64, torch.complex128):
        for rows, cols in ((1, 1), (31, 33), (64, 32), (100, 7), (5, 1000)):
            src = torch.randn(rows, cols + 2, dtype=torch.float64, device="cuda").to(dtype)
            dst = torch.zeros(cols, rows + 3, dtype=dtype, device="cuda")
            st = lib.b2s_dense_transpose(src.element_size(), L.ptr(src), rows, cols, cols + 2,
                                         L.ptr(dst), rows + 3, stream)
            assert st == 0
            torch.cuda.synchronize()
            assert torch.equal(dst[:, :rows], src[:, :cols].t())
            assert float(dst[:, rows:].abs().sum()) == 0.0
    a = torch.zeros(8, 8, device="cuda")
    assert lib.b2s_dense_transpose(3, L.ptr(a), 8, 8, 8, L.ptr(a), 8, stream) == 1
    assert lib.b2s_dense_transpose(4, L.ptr(a), 8, 8, 7, L.ptr(a), 8, stream) == 2
    assert lib.b2s_dense_transpose(4, None, 8, 8, 8, L.ptr(a), 8, stream) == 2
    assert lib.b2s_dense_transpose(4, L.ptr(a), 0, 8, 8, L.ptr(a), 8, stream) == 0
