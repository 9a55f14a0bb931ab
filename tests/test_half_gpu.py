"""float16 / bfloat16 values (FlagSparse lists both, _common.py:21-29, and computes them in
float32: spmv_csr.py:124-129, spmm_csr.py:2716-2719).  The kernels read the 16-bit arrays
themselves; the result must be the float32 product of the widened operands rounded once to the
16-bit dtype: bit-identical to rounding this package's own float32 result, and within the
reference's tolerance for the dtype (tests/pytest/accuracy_utils.py:24-26: 1e-3 for float16,
0.016 for bfloat16) of the oracle."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import csr_from_lengths, dev, host, random_values

pytestmark = pytest.mark.gpu

HALF = [torch.float16, torch.bfloat16]
TOL = {torch.float16: 1e-3, torch.bfloat16: 0.016}


def _matrix(rng, n_rows=700, n_cols=500):
    lengths = np.concatenate([[0, 1, 300, 0, 1500], rng.integers(0, 20, n_rows - 5)])
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, np.float32, sort=False)
    return data * 0.125, idx, ptr, (n_rows, n_cols)


def _close(got, want32, dtype):
    want = torch.from_numpy(np.ascontiguousarray(want32)).to(dtype).float()
    assert torch.allclose(got.float().cpu(), want, rtol=TOL[dtype], atol=TOL[dtype])


@pytest.mark.parametrize("dtype", HALF, ids=["float16", "bfloat16"])
@pytest.mark.parametrize("op", ["non", "trans"])
def test_spmv_half_values(dtype, op):
    from flagsparse_b200 import flagsparse_spmv_csr, prepare_spmv_csr
    rng = np.random.default_rng(12)
    data, idx, ptr, shape = _matrix(rng)
    k = shape[0] if op != "non" else shape[1]
    d, i, p = dev(data).to(dtype), dev(idx, torch.int32), dev(ptr, torch.int64)
    x = dev(random_values(rng, k, np.float32)).to(dtype)
    y = flagsparse_spmv_csr(d, i, p, x, shape, op=op)
    assert y.dtype == dtype and y.shape == (shape[1] if op != "non" else shape[0],)
    wide = flagsparse_spmv_csr(d.float(), i, p, x.float(), shape, op=op)
    assert torch.equal(y, wide.to(dtype))
    _close(y, oracle.spmv(host(d.float()), idx, ptr, host(x.float()), shape, op=op), dtype)
    # prepared handle, out and beta
    h = prepare_spmv_csr(d, i, p, shape, op=op)
    assert h.value_dtype == dtype and h.data.dtype == dtype      # kept as stored: no float32 copy
    assert torch.equal(flagsparse_spmv_csr(x=x, prepared=h), y)
    y0 = dev(random_values(rng, y.numel(), np.float32)).to(dtype)
    out = y0.clone()
    got = flagsparse_spmv_csr(x=x, prepared=h, out=out, alpha=0.5, beta=2.0)
    assert got is out
    expect = oracle.spmv(host(d.float()), idx, ptr, host(x.float()), shape, op=op, alpha=0.5,
                         beta=2.0, y0=host(y0.float()))
    _close(out, expect, dtype)
    with pytest.raises(TypeError, match="x dtype must match"):
        flagsparse_spmv_csr(d, i, p, x.float(), shape, op=op)
    with pytest.raises(ValueError, match="out shape/dtype must match result"):
        flagsparse_spmv_csr(d, i, p, x, shape, op=op, out=y0.float())


@pytest.mark.parametrize("dtype", HALF, ids=["float16", "bfloat16"])
@pytest.mark.parametrize("op", ["non", "trans"])
def test_spmm_half_values(dtype, op):
    from flagsparse_b200 import (flagsparse_spmm_csr, flagsparse_spmm_csr_run,
                                 prepare_spmm_csr_route)
    rng = np.random.default_rng(13)
    data, idx, ptr, shape = _matrix(rng)
    k = shape[0] if op != "non" else shape[1]
    m = shape[1] if op != "non" else shape[0]
    d, i, p = dev(data).to(dtype), dev(idx, torch.int32), dev(ptr, torch.int64)
    B = dev(random_values(rng, k * 24, np.float32).reshape(k, 24)).to(dtype)
    C = flagsparse_spmm_csr(d, i, p, B, shape, op=op)
    assert C.dtype == dtype and C.shape == (m, 24)
    wide = flagsparse_spmm_csr(d.float(), i, p, B.float(), shape, op=op)
    assert torch.equal(C, wide.to(dtype))
    _close(C, oracle.spmm(host(d.float()), idx, ptr, host(B.float()), shape, op=op), dtype)
    out = torch.zeros_like(C)
    assert flagsparse_spmm_csr(d, i, p, B, shape, op=op, out=out) is out
    assert torch.equal(out, C)
    with pytest.raises(TypeError, match="B dtype must match"):
        flagsparse_spmm_csr(d, i, p, B.float(), shape, op=op)
    # the prepared route, row- and column-major
    r = prepare_spmm_csr_route(d, i, p, shape, op=op)
    assert r.value_dtype == dtype
    assert torch.equal(flagsparse_spmm_csr_run(r, B), C)
    Cc = flagsparse_spmm_csr_run(r, B, dense_layout="col")
    assert Cc.dtype == dtype and Cc.stride() == (1, m) and torch.equal(Cc, C)
    with pytest.raises(TypeError, match="does not support dtype"):
        prepare_spmm_csr_route(d, i, p, shape, alg="alg1")


@pytest.mark.parametrize("dtype", HALF, ids=["float16", "bfloat16"])
def test_spmv_coo_front_door_half_values(dtype):
    from flagsparse_b200 import flagsparse_spmv_coo_tocsr, flagsparse_spmv_csr
    rng = np.random.default_rng(14)
    data, idx, ptr, shape = _matrix(rng, 300, 200)
    rows = np.repeat(np.arange(shape[0]), np.diff(ptr))
    perm = rng.permutation(data.size)
    d = dev(data).to(dtype)
    x = dev(random_values(rng, shape[1], np.float32)).to(dtype)
    y = flagsparse_spmv_coo_tocsr(d[dev(perm)], dev(rows[perm]), dev(idx[perm]), x, shape)
    assert y.dtype == dtype
    ref = flagsparse_spmv_csr(d, dev(idx, torch.int32), dev(ptr, torch.int64), x, shape)
    assert torch.allclose(y.float(), ref.float(), rtol=TOL[dtype], atol=TOL[dtype])
