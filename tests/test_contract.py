"""Host-side logic that needs no GPU: op codes, scalar handling, the checks that fire before any
device work, and that CPU tensors are refused (there is no CPU path)."""

import pytest
import torch

from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr, prepare_spmv_csr
from flagsparse_b200._contract import (check_scalar, normalize_op, op_name, op_transposes,
                                       resolve_op)
from flagsparse_b200.spmm import (_resolve_spmm_alg1_launch_config,
                                  _select_spmm_alg1_warp_and_factor)


def test_op_codes_follow_reference():
    # spmv_csr.py:29-43 / spmm_csr.py:22-36
    assert [normalize_op(v) for v in (0, 1, 2, "non", " Trans ", "CONJ")] == [0, 1, 2, 0, 1, 2]
    assert normalize_op(None, transpose=True) == 1 and normalize_op(None) == 0
    for bad in ("bad", 3, -1, object()):
        with pytest.raises(ValueError, match="op must be one of: 0=non, 1=trans, 2=conj"):
            normalize_op(bad)
    assert op_name(2) == "conj" and op_transposes("trans") and not op_transposes(0)
    assert resolve_op("trans", True) == 1 and resolve_op(None, None) == 0
    with pytest.raises(ValueError, match="transpose conflicts with op"):
        resolve_op("non", True)
    with pytest.raises(ValueError, match="transpose conflicts with op"):
        resolve_op("conj", False)


def test_scalars():
    assert check_scalar(torch.tensor(2.0), torch.float32, "alpha") == 2.0
    assert check_scalar(1 + 0j, torch.float64, "alpha") == 1.0
    with pytest.raises(TypeError):
        check_scalar(1 + 1j, torch.float64, "alpha")
    assert check_scalar(1 + 1j, torch.complex64, "alpha") == 1 + 1j


def test_dense_tile_heuristic_matches_reference_table():
    # _alpha_spmm_alg1_common.py:6-23
    table = {1: (4, 1), 4: (4, 1), 5: (8, 1), 8: (8, 1), 9: (16, 1), 16: (16, 1), 17: (32, 1),
             32: (32, 1), 33: (32, 2), 64: (32, 2), 65: (32, 4), 128: (32, 4)}
    for n, want in table.items():
        assert _select_spmm_alg1_warp_and_factor(n) == want
    cfg = _resolve_spmm_alg1_launch_config(48, 1536)
    assert (cfg["block_n"], cfg["block_nnz"], cfg["required_segments"]) == (64, 32, 48)
    with pytest.raises(ValueError, match="more CSR segments"):
        _resolve_spmm_alg1_launch_config(48, 1536, block_nnz=128, max_segments=4)
    with pytest.raises(ValueError, match="must be positive"):
        _resolve_spmm_alg1_launch_config(48, 10, block_n=0)


def _cpu_csr():
    data = torch.tensor([1.0, 2.0, 3.0])
    indices = torch.tensor([0, 1, 1], dtype=torch.int32)
    indptr = torch.tensor([0, 2, 3], dtype=torch.int64)
    return data, indices, indptr


def test_spmv_checks_before_device_work():
    data, indices, indptr = _cpu_csr()
    x = torch.ones(2)
    with pytest.raises(ValueError, match="must be CUDA tensors"):  # spmv_csr.py:531-532
        flagsparse_spmv_csr(data, indices, indptr, x, (2, 2))
    with pytest.raises(ValueError, match="are required when prepared is not provided"):
        flagsparse_spmv_csr(data, indices, indptr, x)
    with pytest.raises(TypeError, match="must all be torch.Tensor"):
        flagsparse_spmv_csr([1.0], indices, indptr, x, (2, 2))
    with pytest.raises(ValueError, match="must be 1D tensors"):
        flagsparse_spmv_csr(data.view(1, 3), indices, indptr, x, (2, 2))
    with pytest.raises(ValueError, match=r"indptr length must be n_rows\+1=4, got 3"):
        flagsparse_spmv_csr(data, indices, indptr, x, (3, 2))
    with pytest.raises(ValueError, match="same length"):
        flagsparse_spmv_csr(data[:2], indices, indptr, x, (2, 2))
    with pytest.raises(ValueError, match="index_fallback_policy must be"):
        flagsparse_spmv_csr(data, indices, indptr, x, (2, 2), index_fallback_policy="maybe")
    with pytest.raises(ValueError, match="transpose conflicts with op"):
        flagsparse_spmv_csr(data, indices, indptr, x, (2, 2), op="non", transpose=True)
    with pytest.raises(ValueError, match="transpose=True conflicts with op=non"):
        prepare_spmv_csr(data, indices, indptr, (2, 2), transpose=True, op="non")


def test_spmm_checks_before_device_work():
    data, indices, indptr = _cpu_csr()
    B = torch.ones(2, 4)
    with pytest.raises(ValueError, match="must be CUDA tensors"):  # spmm_csr.py:255-256
        flagsparse_spmm_csr(data, indices, indptr, B, (2, 2))
    with pytest.raises(ValueError, match="shape must be a 2-tuple"):
        flagsparse_spmm_csr(data, indices, indptr, B, (2,))
    with pytest.raises(ValueError, match="non-negative"):
        flagsparse_spmm_csr(data, indices, indptr, B, (-1, 2))
    with pytest.raises(ValueError, match="block_n must be positive"):
        flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), block_n=0)
    with pytest.raises(ValueError, match="op must be one of"):
        flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), op="bad")


def test_install_rebinds_a_flagsparse_like_package():
    """install() on a stand-in module tree with the reference's layout
    (src/flagsparse/__init__.py:247-254, sparse_operations/__init__.py:36-72)."""
    import sys
    import types

    import flagsparse_b200

    root = types.ModuleType("fake_flagsparse")
    ops = types.ModuleType("fake_flagsparse.sparse_operations")
    spmv = types.ModuleType("fake_flagsparse.sparse_operations.spmv_csr")
    spmm = types.ModuleType("fake_flagsparse.sparse_operations.spmm_csr")
    sentinel = object()
    ops.flagsparse_spmv_csr = spmv.flagsparse_spmv_csr = sentinel
    ops.flagsparse_spmm_csr = spmm.flagsparse_spmm_csr = sentinel
    root.sparse_operations, ops.spmv_csr, ops.spmm_csr = ops, spmv, spmm
    for m in (root, ops, spmv, spmm):
        sys.modules[m.__name__] = m
    try:
        replaced = flagsparse_b200.install(root)
        assert root.flagsparse_spmv_csr is flagsparse_b200.flagsparse_spmv_csr
        assert ops.flagsparse_spmm_csr is flagsparse_b200.flagsparse_spmm_csr
        assert spmv.flagsparse_spmv_csr is flagsparse_b200.flagsparse_spmv_csr
        flagsparse_b200.uninstall(replaced)
        assert ops.flagsparse_spmv_csr is sentinel and not hasattr(root, "flagsparse_spmv_csr")
        # replace_modules=True: the two submodules themselves are swapped for this package's,
        # in sys.modules and as attributes, and put back by uninstall()
        replaced = flagsparse_b200.install(root, replace_modules=True)
        import flagsparse_b200.spmm as our_spmm
        import flagsparse_b200.spmv as our_spmv
        assert sys.modules["fake_flagsparse.sparse_operations.spmv_csr"] is our_spmv
        assert sys.modules["fake_flagsparse.sparse_operations.spmm_csr"] is our_spmm
        assert ops.spmv_csr is our_spmv and ops.spmm_csr is our_spmm
        flagsparse_b200.uninstall(replaced)
        assert sys.modules["fake_flagsparse.sparse_operations.spmv_csr"] is spmv
        assert ops.spmv_csr is spmv and ops.spmm_csr is spmm
        assert ops.flagsparse_spmv_csr is sentinel
    finally:
        for m in (root, ops, spmv, spmm):
            sys.modules.pop(m.__name__, None)


def test_install_into_the_real_flagsparse_package_when_its_source_is_at_hand():
    """Only where FlagSparse is reachable (FLAGSPARSE_SRC, or the package installed under
    baseline/_ref):
    install() rebinds the public names on the package and its submodules; uninstall() puts the
    Triton implementations back."""
    import importlib
    import os
    import sys

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.environ.get("FLAGSPARSE_SRC", os.path.join(here, "baseline", "_ref"))
    if not os.path.isdir(os.path.join(src, "flagsparse")):
        pytest.skip("no FlagSparse source tree here")
    sys.path.insert(0, src)
    try:
        flagsparse = importlib.import_module("flagsparse")
        ops = importlib.import_module("flagsparse.sparse_operations")
        ref_spmv, ref_spmm = ops.flagsparse_spmv_csr, ops.flagsparse_spmm_csr
        import flagsparse_b200
        replaced = flagsparse_b200.install(flagsparse)
        assert flagsparse.flagsparse_spmv_csr is flagsparse_b200.flagsparse_spmv_csr
        assert ops.flagsparse_spmm_csr is flagsparse_b200.flagsparse_spmm_csr
        assert ops.spmv_csr.flagsparse_spmv_csr is flagsparse_b200.flagsparse_spmv_csr
        assert ops.spmm_csr.flagsparse_spmm_csr is flagsparse_b200.flagsparse_spmm_csr
        # same signature prefix as the reference: every reference parameter, in order
        import inspect
        for ours, theirs in ((flagsparse_b200.flagsparse_spmv_csr, ref_spmv),
                             (flagsparse_b200.flagsparse_spmm_csr, ref_spmm),
                             (flagsparse_b200.prepare_spmv_csr, ops.prepare_spmv_csr),
                             (flagsparse_b200.prepare_spmm_csr_route, ops.prepare_spmm_csr_route),
                             (flagsparse_b200.flagsparse_spmm_csr_run,
                              ops.flagsparse_spmm_csr_run)):
            a = list(inspect.signature(ours).parameters.items())
            b = list(inspect.signature(theirs).parameters.items())
            assert [k for k, _ in a[:len(b)]] == [k for k, _ in b]
            assert [v.default for _, v in a[:len(b)]] == [v.default for _, v in b]
            assert [v.kind for _, v in a[:len(b)]] == [v.kind for _, v in b]
        # the route registry answers the same questions as the reference's
        import torch
        for dtype in (torch.float32, torch.float64, torch.complex64, torch.complex128):
            assert (flagsparse_b200.list_spmm_csr_algorithms(dtype=dtype)
                    == ops.spmm_csr.list_spmm_csr_algorithms(dtype=dtype))
        for token in ("base", "CSR", " alg1 ", "csr_alg2", "auto", None):
            from flagsparse_b200 import spmm_route
            assert (spmm_route._normalize_spmm_csr_alg(token)
                    == ops.spmm_csr._normalize_spmm_csr_alg(token))
        for token in ("auto", None, "Row-Major", "F", "fortran", "column", "c_order"):
            assert (spmm_route._normalize_dense_layout(token)
                    == ops.spmm_csr._normalize_dense_layout(token))
        assert issubclass(flagsparse_b200.SpmmCsrAlgorithmUnavailable, RuntimeError)
        flagsparse_b200.uninstall(replaced)
        assert ops.flagsparse_spmv_csr is ref_spmv and ops.flagsparse_spmm_csr is ref_spmm
    finally:
        sys.path.remove(src)
        for name in [m for m in sys.modules if m == "flagsparse" or m.startswith("flagsparse.")]:
            sys.modules.pop(name, None)


def test_route_names_layouts_and_registry_without_a_gpu():
    """The route API's name handling (spmm_csr.py:571-639, :2012-2037): aliases, "auto",
    unknown names, the dtypes each route is registered for, dense-layout spellings."""
    import torch

    import flagsparse_b200 as fb
    from flagsparse_b200 import spmm_route as R

    assert R._normalize_spmm_csr_alg(None) == "auto"
    assert R._normalize_spmm_csr_alg(" Base ") == "csr_base"
    assert R._normalize_spmm_csr_alg("ALG1") == "spmm_csr_alg1"
    assert R._normalize_spmm_csr_alg("csr_alg2") == "spmm_csr_alg2"
    assert fb.resolve_spmm_csr_algorithm("auto", "non", torch.complex64) == "csr_base"
    assert fb.resolve_spmm_csr_algorithm("alg2", 1, torch.float64) == "spmm_csr_alg2"
    with pytest.raises(ValueError, match="unsupported CSR SpMM algorithm"):
        fb.resolve_spmm_csr_algorithm("fastest", "non", torch.float32)
    with pytest.raises(TypeError, match="does not support dtype"):
        fb.resolve_spmm_csr_algorithm("alg1", "non", torch.complex128)
    with pytest.raises(ValueError):
        fb.resolve_spmm_csr_algorithm("base", "upside-down", torch.float32)
    assert fb.list_spmm_csr_algorithms() == ("csr_base", "alpha_alg1_tle_opt",
                                             "alpha_alg1_tle_opt2", "spmm_csr_alg1",
                                             "spmm_csr_alg2")
    assert fb.list_spmm_csr_algorithms(op="conj", dtype=torch.complex64) == ("csr_base",)
    for token in (None, "auto", "default", "row", "Row_Major", "C", "c_order"):
        assert R._normalize_dense_layout(token) == "row"
    for token in ("col", "COLUMN", "col-major", "column_major", "f", "Fortran"):
        assert R._normalize_dense_layout(token) == "col"
    with pytest.raises(ValueError, match="dense_layout"):
        R._normalize_dense_layout("tiled")
    with pytest.raises(TypeError, match="PreparedCsrSpmmRoute"):
        fb.flagsparse_spmm_csr_run("not a handle", torch.zeros(2, 2))
    t = torch.zeros(6, 4)
    assert R._dense_layout_name(t) == "row" and R._dense_layout_name(t.t()) == "col"
    assert R._dense_layout_name(t[:, ::2]) == "strided" and R._dense_layout_name(t[0]) == "unknown"
    c = R._empty_col_major(5, 3, torch.float32, "cpu")
    assert c.shape == (5, 3) and c.stride() == (1, 5) and R._is_col_major_2d(c)
