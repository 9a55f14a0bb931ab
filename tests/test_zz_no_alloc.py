"""b2s_spmv_csr_fixed: the SpMV entry point for callers that are not allowed to allocate device
memory (all memory handed to their own arena at start-up, or a no-allocation rule after
initialisation).  It must give what b2s_spmv_csr gives, on two calls in a row, although it keeps
its tile plan and carries in one fixed array inside the library that every call reuses.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It also passes when run alone in a fresh process."""

import ctypes

import numpy as np
import pytest
import torch

import oracle
from gpu_util import assert_parity, csr_from_lengths, dev, host, random_values

pytestmark = pytest.mark.gpu


def _reference_call(lib, L, d, i, p, x, y_in, n_rows, n_cols, alpha, beta):
    """The existing entry point, with caller-allocated plan and carry."""
    vcode, icode, pcode = L.VALUE_CODE[d.dtype], L.INDEX_CODE[i.dtype], L.INDEX_CODE[p.dtype]
    nnz = d.numel()
    items = lib.b2s_spmv_tile_items(vcode, icode)
    T = lib.b2s_tile_count(n_rows, nnz, items)
    tile_row = torch.empty(T + 1, dtype=torch.int64, device="cuda")
    s = L.stream_handle(d.device)
    assert lib.b2s_tile_plan(L.ptr(p), pcode, n_rows, nnz, items, L.ptr(tile_row), s) == 0
    carry = torch.empty(max(T, 1), dtype=d.dtype, device="cuda")
    y = torch.empty(n_rows, dtype=d.dtype, device="cuda")
    st = lib.b2s_spmv_csr(vcode, icode, pcode, L.ptr(d), L.ptr(i), L.ptr(p), n_rows, n_cols, nnz,
                          L.ptr(x), L.ptr(y_in), L.ptr(y), alpha, beta, L.ptr(tile_row),
                          L.ptr(carry), None, s)
    assert st == 0
    return y


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.complex64, np.complex128],
                         ids=lambda d: np.dtype(d).name)
def test_fixed_scratch_spmv_matches_the_allocating_entry_point_twice(dtype):
    from flagsparse_b200 import _lib as L
    lib = L.load()
    rng = np.random.default_rng(42)
    # two different matrices back to back: the second call finds the first call's plan and
    # carries in the shared array and must not be affected by them
    problems = []
    for lengths in (np.concatenate([rng.integers(0, 20, 5000), [9000, 0, 3]]),
                    np.concatenate([[4000, 1], rng.integers(0, 6, 2000)])):
        n_rows, n_cols = lengths.size, 3000
        data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype)
        problems.append((data, idx, ptr, random_values(rng, n_cols, dtype),
                         random_values(rng, n_rows, dtype), n_rows, n_cols))
    cplx = np.dtype(dtype).kind == "c"
    a_val, b_val = ((1.5 - 0.25j, 0.5 + 2j) if cplx else (1.5, 0.5))
    tdt = dev(problems[0][0]).dtype
    alpha, beta = L.scalar_buffer(a_val, tdt), L.scalar_buffer(b_val, tdt)
    for data, idx, ptr, x, y0, n_rows, n_cols in problems:
        d, i, p, xd, y0d = dev(data), dev(idx, torch.int32), dev(ptr), dev(x), dev(y0)
        want = _reference_call(lib, L, d, i, p, xd, y0d, n_rows, n_cols, alpha, beta)
        got = torch.empty_like(want)
        st = lib.b2s_spmv_csr_fixed(L.VALUE_CODE[d.dtype], L.B2S_I32, L.B2S_I64, L.ptr(d),
                                    L.ptr(i), L.ptr(p), n_rows, n_cols, d.numel(), L.ptr(xd),
                                    L.ptr(y0d), L.ptr(got), alpha, beta,
                                    L.stream_handle(d.device))
        assert st == 0, lib.b2s_status_string(st)
        torch.cuda.synchronize()
        assert_parity(host(got), host(want), dtype, "fixed-scratch vs allocating entry point")
        assert_parity(host(got), oracle.spmv(data, idx, ptr, x, (n_rows, n_cols), alpha=a_val,
                                             beta=b_val, y0=y0), dtype, "fixed-scratch vs oracle")


def test_fixed_scratch_spmv_rejects_problems_beyond_its_limit():
    from flagsparse_b200 import _lib as L
    lib = L.load()
    limit = lib.b2s_spmv_csr_fixed_max_items()
    assert limit == 1 << 26      # rows + non-zeros, the same for every dtype
    one = (ctypes.c_float * 1)(1.0)
    zero = (ctypes.c_float * 1)(0.0)
    dummy = torch.zeros(8, device="cuda")
    # sizes alone decide: nothing is launched, no pointer is read
    st = lib.b2s_spmv_csr_fixed(L.B2S_F32, L.B2S_I32, L.B2S_I32, L.ptr(dummy), L.ptr(dummy),
                                L.ptr(dummy), limit // 2, 10, limit // 2 + 1, L.ptr(dummy), None,
                                L.ptr(dummy), one, zero, L.stream_handle(dummy.device))
    assert st == 8
    assert b"fixed scratch" in lib.b2s_status_string(st)
