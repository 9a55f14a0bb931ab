"""Seeded random sweep of small CSR problems through the public API against the CPU oracle:
shapes from empty to a few hundred rows, every value / index dtype, all ops, alpha / beta,
unsorted and duplicate columns, dense widths that straddle the 16-byte lane tiles."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import assert_parity, dev, host, random_values

pytestmark = pytest.mark.gpu

DTYPES = [np.float32, np.float64, np.complex64, np.complex128]


def _random_problem(rng):
    n_rows = int(rng.choice([0, 1, 2, 7, 33, 100, 257, 600]))
    n_cols = int(rng.choice([1, 2, 5, 31, 64, 300, 1000]))
    kind = rng.integers(0, 4)
    if kind == 0:
        lengths = rng.integers(0, 4, n_rows)
    elif kind == 1:
        lengths = rng.integers(0, 60, n_rows)
    elif kind == 2:
        lengths = np.where(rng.random(n_rows) < 0.05, rng.integers(500, 3000, n_rows), 0)
    else:
        lengths = np.zeros(n_rows, dtype=np.int64)
    ptr = np.zeros(n_rows + 1, dtype=np.int64)
    np.cumsum(lengths, out=ptr[1:])
    idx = rng.integers(0, n_cols, int(ptr[-1]))          # unsorted, duplicates allowed
    return n_rows, n_cols, idx, ptr


@pytest.mark.parametrize("seed", range(12))
def test_random_spmv_and_spmm_against_oracle(seed):
    from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr
    rng = np.random.default_rng(1000 + seed)
    for _ in range(10):
        n_rows, n_cols, idx, ptr = _random_problem(rng)
        dtype = DTYPES[int(rng.integers(0, 4))]
        tdt_i = [torch.int32, torch.int64][int(rng.integers(0, 2))]
        tdt_p = [torch.int32, torch.int64][int(rng.integers(0, 2))]
        op = ["non", "trans", "conj"][int(rng.integers(0, 3))]
        data = random_values(rng, idx.size, dtype)
        n_in, n_out = (n_rows, n_cols) if op != "non" else (n_cols, n_rows)
        cplx = np.dtype(dtype).kind == "c"
        alpha = (0.75 - 0.5j) if cplx else -1.25
        use_beta = bool(rng.integers(0, 2))
        beta = ((0.5 + 0.25j) if cplx else 2.0) if use_beta else 0.0
        d, i, p = dev(data), dev(idx, tdt_i), dev(ptr, tdt_p)

        x = random_values(rng, n_in, dtype)
        y0 = random_values(rng, n_out, dtype)
        expect = oracle.spmv(data, idx, ptr, x, (n_rows, n_cols), op=op, alpha=alpha, beta=beta,
                             y0=y0)
        out = dev(y0) if use_beta else None
        y = flagsparse_spmv_csr(d, i, p, dev(x), (n_rows, n_cols), op=op, alpha=alpha, beta=beta,
                                out=out)
        assert y.shape == (n_out,)
        assert_parity(host(y), expect, dtype, f"spmv seed {seed} {n_rows}x{n_cols} {op}")

        n_dense = int(rng.choice([1, 2, 3, 7, 8, 17, 32, 40]))
        B = random_values(rng, n_in * n_dense, dtype).reshape(n_in, n_dense)
        C0 = random_values(rng, n_out * n_dense, dtype).reshape(n_out, n_dense)
        expect = oracle.spmm(data, idx, ptr, B, (n_rows, n_cols), op=op, alpha=alpha, beta=beta,
                             C0=C0)
        outC = dev(C0) if use_beta else None
        C = flagsparse_spmm_csr(d, i, p, dev(B), (n_rows, n_cols), op=op, alpha=alpha, beta=beta,
                                out=outC)
        assert C.shape == (n_out, n_dense)
        assert_parity(host(C), expect, dtype, f"spmm seed {seed} {n_rows}x{n_cols}x{n_dense} {op}")


def test_full_size_transposed_spmm_against_torch():
    """Config 4 at full size (1,000,000 x 500,000, Poisson(24) rows, N = 64, op = trans) against
    torch's own sparse product of the explicitly transposed matrix."""
    from flagsparse_b200 import flagsparse_spmm_csr, workloads
    p = workloads.cfg4_poisson_spmm(device="cuda")
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape, op="trans")
    A = torch.sparse_csr_tensor(p.indptr.long(), p.indices.long(), p.data.double(), size=p.shape)
    ref = A.to_sparse_coo().t().coalesce() @ p.B.double()
    err = float(torch.linalg.matrix_norm(C.double() - ref) / torch.linalg.matrix_norm(ref))
    assert err <= 1e-5, err
    assert torch.equal(C, flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape,
                                              op="trans"))
