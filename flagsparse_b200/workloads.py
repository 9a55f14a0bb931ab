"""Seeded synthetic CSR inputs for tests and benchmarks.

FlagSparse ships a random CSR builder for its own benchmarks (_common.py:186-201, used by
benchmarks.py:343-505); this module plays that role for the shapes this build is measured on.
Every generator takes a ``scale`` divisor for the row count so that the same distribution can be
drawn small enough for a CPU check.  Tensors are created on ``device`` with a
``torch.Generator`` seeded explicitly, so a (device type, torch version, seed) triple always
gives the same matrix.
"""

from __future__ import annotations

import math

import torch


class CsrProblem:
    """A CSR matrix plus the dense operands of one benchmark configuration."""

    def __init__(self, name, data, indices, indptr, shape, **extra):
        self.name = name
        self.data = data
        self.indices = indices
        self.indptr = indptr
        self.shape = (int(shape[0]), int(shape[1]))
        self.extra = extra

    @property
    def nnz(self):
        return int(self.data.numel())

    def __getattr__(self, item):
        extra = self.__dict__.get("extra", {})
        if item in extra:
            return extra[item]
        raise AttributeError(item)


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _values(n, dtype, dist, gen, device):
    """n values ~ U(-1,1) ('uniform') or N(0,1) ('normal'); complex: independent re / im."""
    if dtype.is_complex:
        comp = torch.float32 if dtype == torch.complex64 else torch.float64
        return torch.complex(_values(n, comp, dist, gen, device),
                             _values(n, comp, dist, gen, device))
    if dist == "normal":
        return torch.randn(n, dtype=dtype, device=device, generator=gen)
    return torch.rand(n, dtype=dtype, device=device, generator=gen) * 2 - 1


def _csr_from_lengths(lengths, n_cols, index_dtype, gen, device, sort_cols=True):
    """Row lengths -> (indices, indptr): columns uniform over [0, n_cols), sorted inside each row
    when sort_cols (duplicates allowed: the kernels sum them)."""
    n_rows = lengths.numel()
    indptr64 = torch.zeros(n_rows + 1, dtype=torch.int64, device=device)
    torch.cumsum(lengths, 0, out=indptr64[1:])
    nnz = int(indptr64[-1].item())
    cols = torch.randint(0, max(n_cols, 1), (nnz,), dtype=torch.int64, device=device,
                         generator=gen)
    if sort_cols and nnz > 0:
        rows = torch.repeat_interleave(torch.arange(n_rows, dtype=torch.int64, device=device),
                                       lengths)
        key = rows * int(n_cols) + cols
        del rows
        key, _ = torch.sort(key)
        cols = key % int(n_cols)
        del key
    return cols.to(index_dtype), indptr64.to(index_dtype)


def zipf_row_lengths(n_rows, s, max_len, mean, gen, device):
    """Truncated Zipf(s) on {1..max_len} by inverse CDF, then L = clip(ceil(c*z), 1, max_len) with
    c bisected so that mean(L) is `mean` (to within 0.5)."""
    z = torch.arange(1, max_len + 1, dtype=torch.float64, device=device)
    cdf = torch.cumsum(z.pow(-float(s)), 0)
    cdf = cdf / cdf[-1]
    u = torch.rand(n_rows, dtype=torch.float64, device=device, generator=gen)
    zs = (torch.searchsorted(cdf, u) + 1).clamp_(max=max_len).to(torch.float64)

    def lengths_for(c):
        return torch.ceil(zs * c).clamp_(1, max_len).to(torch.int64)

    lo, hi = 1e-3, 64.0
    for _ in range(60):
        mid = math.sqrt(lo * hi)
        m = float(lengths_for(mid).double().mean().item())
        if abs(m - mean) <= 0.05:
            lo = hi = mid
            break
        if m < mean:
            lo = mid
        else:
            hi = mid
    return lengths_for(math.sqrt(lo * hi))


# -------------------------------------------------------------------------------------------------
# the five measured configurations
# -------------------------------------------------------------------------------------------------
def cfg1_uniform_spmv(device="cpu", scale=1, seed=0):
    """SpMV float32/int32, 65,536^2, row length ~ U{1..32}, sorted random columns, values and
    x ~ U(-1,1), alpha=1 beta=0."""
    n = max(65536 // scale, 1)
    g = _gen(device, seed)
    lengths = torch.randint(1, 33, (n,), dtype=torch.int64, device=device, generator=g)
    idx, ptr = _csr_from_lengths(lengths, n, torch.int32, g, device)
    data = _values(idx.numel(), torch.float32, "uniform", g, device)
    x = _values(n, torch.float32, "uniform", g, device)
    return CsrProblem("cfg1", data, idx, ptr, (n, n), x=x, alpha=1.0, beta=0.0)


def cfg2_powerlaw_spmv(device="cpu", scale=1, seed=0, n_dense=0):
    """SpMV float64/int64, 2^24 rows, Zipf(1.8) row lengths (min 1, max 100,000, mean 16),
    sorted random columns, values / x / y0 ~ N(0,1), alpha=1.5 beta=0.5.  n_dense > 0 adds the
    dense B (2^24 x n_dense, N(0,1)) of the SpMM run on the same matrix."""
    n = max((1 << 24) // scale, 1)
    g = _gen(device, seed)
    lengths = zipf_row_lengths(n, 1.8, min(100_000, n), 16.0, g, device)
    idx, ptr = _csr_from_lengths(lengths, n, torch.int64, g, device)
    data = _values(idx.numel(), torch.float64, "normal", g, device)
    x = _values(n, torch.float64, "normal", g, device)
    y0 = _values(n, torch.float64, "normal", g, device)
    extra = dict(x=x, y0=y0, alpha=1.5, beta=0.5)
    if n_dense:
        extra["B"] = _values(n * n_dense, torch.float64, "normal", g, device).view(n, n_dense)
    return CsrProblem("cfg2", data, idx, ptr, (n, n), **extra)


def cfg3_banded_spmm(device="cpu", scale=1, seed=0, n_dense=32):
    """SpMM float32/int32 op=non, 2^22 rows, band [i-32, i+32) kept with p=0.4, values and
    B (2^22 x 32) ~ U(-1,1)."""
    n = max((1 << 22) // scale, 1)
    g = _gen(device, seed)
    half, width = 32, 64
    chunks_idx, counts = [], torch.zeros(n, dtype=torch.int64, device=device)
    step = 1 << 20
    for r0 in range(0, n, step):
        r1 = min(n, r0 + step)
        rows = torch.arange(r0, r1, dtype=torch.int64, device=device).unsqueeze(1)
        cols = rows - half + torch.arange(width, dtype=torch.int64, device=device).unsqueeze(0)
        keep = torch.rand(r1 - r0, width, device=device, generator=g) < 0.4
        keep &= (cols >= 0) & (cols < n)
        counts[r0:r1] = keep.sum(1)
        chunks_idx.append(cols[keep])
    idx = torch.cat(chunks_idx).to(torch.int32)
    ptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=ptr[1:])
    data = _values(idx.numel(), torch.float32, "uniform", g, device)
    B = _values(n * n_dense, torch.float32, "uniform", g, device).view(n, n_dense)
    return CsrProblem("cfg3", data, idx, ptr.to(torch.int32), (n, n), B=B, alpha=1.0, beta=0.0)


def cfg4_poisson_spmm(device="cpu", scale=1, seed=0, dtype=torch.float32, n_dense=64):
    """SpMM op=trans (float32) / op=conj (complex64), A 1,000,000 x 500,000, row length
    ~ Poisson(24), unsorted random columns, values ~ U(-1,1), B 1,000,000 x 64."""
    n_rows = max(1_000_000 // scale, 1)
    n_cols = max(500_000 // scale, 1)
    g = _gen(device, seed)
    lengths = torch.poisson(torch.full((n_rows,), 24.0, device=device), generator=g).to(
        torch.int64)
    idx, ptr = _csr_from_lengths(lengths, n_cols, torch.int32, g, device, sort_cols=False)
    data = _values(idx.numel(), dtype, "uniform", g, device)
    B = _values(n_rows * n_dense, dtype, "uniform", g, device).view(n_rows, n_dense)
    return CsrProblem("cfg4", data, idx, ptr, (n_rows, n_cols), B=B, alpha=1.0, beta=0.0,
                      op="conj" if dtype.is_complex else "trans")


def cfg5_scaling(device="cpu", scale=1, seed=0, n_dense=16, with_B=True):
    """SpMV + SpMM float32/int64, 2^26 rows, Zipf(2.0) row lengths scaled to mean 16
    (max 100,000), sorted random columns, values / x / B ~ U(-1,1)."""
    n = max((1 << 26) // scale, 1)
    g = _gen(device, seed)
    lengths = zipf_row_lengths(n, 2.0, min(100_000, n), 16.0, g, device)
    idx, ptr = _csr_from_lengths(lengths, n, torch.int64, g, device)
    data = _values(idx.numel(), torch.float32, "uniform", g, device)
    x = _values(n, torch.float32, "uniform", g, device)
    extra = dict(x=x, alpha=1.0, beta=0.0)
    if with_B:
        extra["B"] = _values(n * n_dense, torch.float32, "uniform", g, device).view(n, n_dense)
    return CsrProblem("cfg5", data, idx, ptr, (n, n), **extra)


# -------------------------------------------------------------------------------------------------
# algorithmic bytes / flops (compulsory traffic; every array counted once)
# -------------------------------------------------------------------------------------------------
def spmv_bytes(n_out_rows, n_x, nnz, value_bytes, index_bytes, ptr_bytes=None, beta_nonzero=False):
    ptr_bytes = index_bytes if ptr_bytes is None else ptr_bytes
    return ((n_out_rows + 1) * ptr_bytes + nnz * (index_bytes + value_bytes) + n_x * value_bytes
            + n_out_rows * value_bytes * (2 if beta_nonzero else 1))


def spmm_bytes(n_out_rows, n_b_rows, nnz, n_dense, value_bytes, index_bytes, ptr_bytes=None,
               beta_nonzero=False):
    ptr_bytes = index_bytes if ptr_bytes is None else ptr_bytes
    return ((n_out_rows + 1) * ptr_bytes + nnz * (index_bytes + value_bytes)
            + n_b_rows * n_dense * value_bytes
            + n_out_rows * n_dense * value_bytes * (2 if beta_nonzero else 1))


def sp_flops(nnz, n_dense=1, complex_values=False):
    return 2 * nnz * n_dense * (4 if complex_values else 1)
