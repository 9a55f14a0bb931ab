"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

import oracle
from conftest import REL_L2_TOL

TORCH_OF = {np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64,
            np.dtype(np.complex64): torch.complex64, np.dtype(np.complex128): torch.complex128}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.detach().cpu().numpy()


def random_values(rng, n, dtype, scale=1.0):
    dtype = np.dtype(dtype)
    if dtype.kind == "c":
        comp = np.float32 if dtype == np.complex64 else np.float64
        return ((rng.standard_normal(n) + 1j * rng.standard_normal(n)) * scale).astype(dtype)
    return (rng.standard_normal(n) * scale).astype(dtype)


def csr_from_lengths(rng, lengths, n_cols, dtype, sort=True):
    lengths = np.asarray(lengths, dtype=np.int64)
    indptr = np.zeros(lengths.size + 1, dtype=np.int64)
    np.cumsum(lengths, out=indptr[1:])
    nnz = int(indptr[-1])
    cols = rng.integers(0, max(n_cols, 1), nnz)
    if sort and nnz:
        rows = np.repeat(np.arange(lengths.size), lengths)
        cols = (np.sort(rows * n_cols + cols) % n_cols)
    return random_values(rng, nnz, dtype), cols.astype(np.int64), indptr


def assert_parity(actual, expected, dtype, what=""):
    """rel-L2 within the north-star tolerance (1e-5 fp32/complex64, 1e-12 fp64/complex128)."""
    err = oracle.rel_l2(actual, expected)
    tol = REL_L2_TOL[np.dtype(dtype)]
    assert err <= tol, f"{what}: rel-L2 {err:.3e} > {tol:.1e}"
    return err
