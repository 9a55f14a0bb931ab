"""Side by side with the unmodified FlagSparse package on the same device tensors.

The reference is pure Python + Triton.  When a copy of it has been installed beside this
repository (``python -m pip install --no-index --no-build-isolation --no-deps --target
baseline/_ref <reference checkout>``; the folder is git-ignored) these tests call its own
``flagsparse_spmv_csr`` / ``flagsparse_spmm_csr`` (src/flagsparse/sparse_operations/spmv_csr.py,
spmm_csr.py) and this package's functions on identical CUDA tensors and compare the results with
the tolerances the reference's accuracy checks use for parity: rel-L2 <= 1e-5 for float32 /
complex64 and <= 1e-12 for float64 / complex128.  Without that folder every test here is skipped;
the committed fixtures under ``tests/golden`` and the C oracle carry the parity claim then.
"""

from __future__ import annotations

import importlib
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

_REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                        "baseline", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not os.path.isdir(os.path.join(_REF_DIR, "flagsparse")):
        pytest.skip("no installed copy of the reference package under baseline/_ref")
    sys.path.insert(0, _REF_DIR)
    try:
        mod = importlib.import_module("flagsparse")
        getattr(mod, "flagsparse_spmv_csr")
        getattr(mod, "flagsparse_spmm_csr")
    except Exception as exc:  # noqa: BLE001 - a reference that does not import is not a failure here
        pytest.skip(f"reference package does not import: {exc}")
    finally:
        sys.path.remove(_REF_DIR)
    yield mod
    for name in [m for m in sys.modules if m == "flagsparse" or m.startswith("flagsparse.")]:
        sys.modules.pop(name, None)


def _rel_l2(got, want):
    wide = torch.complex128 if want.is_complex() else torch.float64
    got, want = got.to(wide), want.to(wide)
    denom = float(torch.linalg.vector_norm(want))
    return float(torch.linalg.vector_norm(got - want)) / (denom if denom > 0 else 1.0)


def _tol(dtype):
    return 1e-5 if dtype in (torch.float32, torch.complex64) else 1e-12


@pytest.mark.parametrize("op", ["non", "trans", "conj"])
def test_spmv_uniform_f32_i32_matches_reference(ref, op):
    import flagsparse_b200 as ours
    from flagsparse_b200 import workloads as W

    p = W.cfg1_uniform_spmv("cuda")
    want = ref.flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, op=op)
    got = ours.flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, op=op)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert _rel_l2(got, want) <= _tol(p.data.dtype)


@pytest.mark.parametrize("op", ["non", "trans"])
def test_spmv_powerlaw_f64_i64_matches_reference(ref, op):
    import flagsparse_b200 as ours
    from flagsparse_b200 import workloads as W

    # 1/256 of the rows: the reference's baseline kernel walks ceil(longest row / 256) masked
    # segments for every row, which is what makes the full-size matrix take seconds there
    p = W.cfg2_powerlaw_spmv("cuda", scale=256)
    want = ref.flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, op=op)
    got = ours.flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, op=op)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert _rel_l2(got, want) <= _tol(p.data.dtype)


def test_spmv_prepared_handle_matches_reference(ref):
    import flagsparse_b200 as ours
    from flagsparse_b200 import workloads as W

    p = W.cfg1_uniform_spmv("cuda", scale=4)
    ref_prep = ref.prepare_spmv_csr(p.data, p.indices, p.indptr, p.shape)
    our_prep = ours.prepare_spmv_csr(p.data, p.indices, p.indptr, p.shape)
    want = ref.flagsparse_spmv_csr(x=p.x, prepared=ref_prep)
    got = ours.flagsparse_spmv_csr(x=p.x, prepared=our_prep)
    assert _rel_l2(got, want) <= 1e-5


def test_spmm_banded_f32_i32_matches_reference(ref):
    import flagsparse_b200 as ours
    from flagsparse_b200 import workloads as W

    p = W.cfg3_banded_spmm("cuda", scale=16)
    want = ref.flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    got = ours.flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert _rel_l2(got, want) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64])
def test_spmm_transposed_matches_reference(ref, dtype):
    import flagsparse_b200 as ours
    from flagsparse_b200 import workloads as W

    p = W.cfg4_poisson_spmm("cuda", scale=8, dtype=dtype)
    want = ref.flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape, op=p.op)
    got = ours.flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape, op=p.op)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert _rel_l2(got, want) <= 1e-5


def test_spmm_powerlaw_f64_i64_matches_reference(ref):
    import flagsparse_b200 as ours
    from flagsparse_b200 import workloads as W

    p = W.cfg2_powerlaw_spmv("cuda", scale=64, n_dense=32)
    want = ref.flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    got = ours.flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    assert _rel_l2(got, want) <= 1e-12
    again = ours.flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    assert torch.equal(got, again)
