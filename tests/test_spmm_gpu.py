"""GPU parity of flagsparse_spmm_csr (CUDA path) against the CPU oracle and the reference
fixtures.  Tolerance: rel-L2 <= 1e-5 (float32 / complex64), <= 1e-12 (float64 / complex128)."""

import numpy as np
import pytest
import torch

import oracle
from conftest import ALLCLOSE_TOL, load_golden
from gpu_util import TORCH_OF, assert_parity, csr_from_lengths, dev, host, random_values

pytestmark = pytest.mark.gpu

SPMM_CASES = sorted(load_golden("spmm_reference.npz"))
DTYPES = [np.float32, np.float64, np.complex64, np.complex128]


def _shape_of(case, c):
    n_rows = c["indptr"].shape[0] - 1
    if case.startswith("spmm_longrow"):
        return n_rows, 2048
    M, K, _ = (int(v) for v in case.split("_")[1].split("x"))
    return M, K


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64], ids=["int32", "int64"])
@pytest.mark.parametrize("case", SPMM_CASES)
def test_spmm_matches_reference_fixture(case, index_dtype, spmm_golden):
    from flagsparse_b200 import flagsparse_spmm_csr
    c = spmm_golden[case]
    op = case.rsplit("_", 1)[1]
    C = flagsparse_spmm_csr(dev(c["data"]), dev(c["indices"], index_dtype),
                            dev(c["indptr"], index_dtype), dev(c["B"]), _shape_of(case, c), op=op)
    assert_parity(host(C), c["C"], c["C"].dtype, case)
    tol = ALLCLOSE_TOL[c["C"].dtype]
    assert np.allclose(host(C), c["C"], rtol=max(tol, 1e-5 if tol > 1e-7 else tol), atol=tol * 8)


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("n_dense", [1, 3, 4, 5, 16, 31, 32, 33, 64, 130])
@pytest.mark.parametrize("op", ["non", "trans"])
def test_spmm_dense_widths_vs_oracle(dtype, n_dense, op):
    """Every dense-column tile (1 .. 32 lanes per B row, and more than one column tile), widths
    that are not a multiple of 16 bytes, ragged rows including one longer than several tiles."""
    from flagsparse_b200 import flagsparse_spmm_csr
    rng = np.random.default_rng(100 + n_dense)
    lengths = np.concatenate([[0, 1, 31, 32, 33, 0, 3000, 2, 600, 513, 0],
                              rng.integers(0, 5, 700), np.zeros(1200, dtype=np.int64),
                              rng.integers(0, 80, 300), [0]])
    n_rows, n_cols = lengths.size, 1500
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype)
    k = n_rows if op != "non" else n_cols
    B = random_values(rng, k * n_dense, dtype).reshape(k, n_dense)
    expect = oracle.spmm(data, idx, ptr, B, (n_rows, n_cols), op=op)
    args = (dev(data), dev(idx, torch.int32), dev(ptr, torch.int64), dev(B), (n_rows, n_cols))
    C = flagsparse_spmm_csr(*args, op=op)
    assert_parity(host(C), expect, dtype)
    C2 = flagsparse_spmm_csr(*args, op=op)
    assert torch.equal(C.view(torch.uint8), C2.view(torch.uint8)), "not bit-identical run to run"


@pytest.mark.parametrize("dtype", [np.complex64, np.complex128], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64], ids=["i32", "i64"])
def test_spmm_conj_vs_oracle(dtype, idx_dtype):
    from flagsparse_b200 import flagsparse_spmm_csr
    rng = np.random.default_rng(21)
    data, idx, ptr = csr_from_lengths(rng, rng.integers(0, 30, 900), 400, dtype, sort=False)
    B = random_values(rng, 900 * 8, dtype).reshape(900, 8)
    C = flagsparse_spmm_csr(dev(data), dev(idx, idx_dtype), dev(ptr, idx_dtype), dev(B),
                            (900, 400), op="conj")
    assert_parity(host(C), oracle.spmm(data, idx, ptr, B, (900, 400), op="conj"), dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
def test_spmm_alpha_beta_out_and_strides(dtype):
    from flagsparse_b200 import flagsparse_spmm_csr
    rng = np.random.default_rng(8)
    lengths = rng.integers(0, 30, 1000)
    lengths[5] = 5000
    data, idx, ptr = csr_from_lengths(rng, lengths, 800, dtype)
    B = random_values(rng, 800 * 12, dtype).reshape(800, 12)
    C0 = random_values(rng, 1000 * 12, dtype).reshape(1000, 12)
    alpha, beta = (1.5, 0.5) if np.dtype(dtype).kind != "c" else (1.5 - 0.25j, 0.5 + 2j)
    expect = oracle.spmm(data, idx, ptr, B, (1000, 800), alpha=alpha, beta=beta, C0=C0)
    out = dev(C0)
    C = flagsparse_spmm_csr(dev(data), dev(idx), dev(ptr), dev(B), (1000, 800), out=out,
                            alpha=alpha, beta=beta)
    assert C is out
    assert_parity(host(C), expect, dtype)
    # B as a column slice of a wider matrix (row-major, leading dimension 20) and a transposed B
    wide = torch.zeros((800, 20), dtype=TORCH_OF[np.dtype(dtype)], device="cuda")
    wide[:, 3:15] = dev(B)
    C = flagsparse_spmm_csr(dev(data), dev(idx), dev(ptr), wide[:, 3:15], (1000, 800))
    assert_parity(host(C), oracle.spmm(data, idx, ptr, B, (1000, 800)), dtype)
    Bt = dev(np.ascontiguousarray(B.T)).t()
    assert not Bt.is_contiguous()
    C = flagsparse_spmm_csr(dev(data), dev(idx), dev(ptr), Bt, (1000, 800))
    assert_parity(host(C), oracle.spmm(data, idx, ptr, B, (1000, 800)), dtype)


def test_spmm_cfg3_and_cfg4_scaled_vs_oracle():
    """Banded float32/int32 N=32 and Poisson(24) op=trans float32 / op=conj complex64 N=64, at
    1/16 and 1/32 of the benchmark's row counts."""
    from flagsparse_b200 import flagsparse_spmm_csr, workloads
    p = workloads.cfg3_banded_spmm(device="cuda", scale=16)
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    expect = oracle.spmm(host(p.data), host(p.indices), host(p.indptr), host(p.B), p.shape)
    assert_parity(host(C), expect, np.float32, "cfg3")
    for dtype in (torch.float32, torch.complex64):
        p = workloads.cfg4_poisson_spmm(device="cuda", scale=32, dtype=dtype)
        C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape, op=p.op)
        assert C.shape == (p.shape[1], 64)
        expect = oracle.spmm(host(p.data), host(p.indices), host(p.indptr), host(p.B), p.shape,
                             op=p.op)
        assert_parity(host(C), expect, host(p.data).dtype, f"cfg4 {p.op}")


def test_spmm_powerlaw_scaled_vs_oracle():
    """float64/int64 power-law matrix (1/256 of 2^24 rows) with N=32, and float32/int64 N=16."""
    from flagsparse_b200 import flagsparse_spmm_csr, workloads
    p = workloads.cfg2_powerlaw_spmv(device="cuda", scale=256, n_dense=32)
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    expect = oracle.spmm(host(p.data), host(p.indices), host(p.indptr), host(p.B), p.shape)
    assert_parity(host(C), expect, np.float64, "cfg2-MM")
    p = workloads.cfg5_scaling(device="cuda", scale=1024)
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    expect = oracle.spmm(host(p.data), host(p.indices), host(p.indptr), host(p.B), p.shape)
    assert_parity(host(C), expect, np.float32, "cfg5 SpMM")


def test_spmm_full_size_banded_properties():
    """Full-size banded config (2^22 rows, N=32): compared with torch's CSR product, and repeats
    bit for bit."""
    from flagsparse_b200 import flagsparse_spmm_csr, workloads
    p = workloads.cfg3_banded_spmm(device="cuda")
    C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
    A = torch.sparse_csr_tensor(p.indptr.long(), p.indices.long(), p.data.double(), size=p.shape)
    ref = A @ p.B.double()
    err = float(torch.linalg.matrix_norm(C.double() - ref) / torch.linalg.matrix_norm(ref))
    assert err <= 1e-5, err
    assert torch.equal(C, flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape))


def test_spmm_api_contract():
    """The negative / positive cases of the reference's CLI checks (tests/test_spmm.py:766-898)
    and of tests/pytest/test_spmm_csr_accuracy.py:135-215."""
    from flagsparse_b200 import flagsparse_spmm_csr as f
    cuda = "cuda"
    data = torch.tensor([1.0, 2.0, 3.0], device=cuda)
    indices = torch.tensor([0, 1, 1], dtype=torch.int32, device=cuda)
    indptr = torch.tensor([0, 2, 3], dtype=torch.int64, device=cuda)
    B = torch.randn((2, 4), device=cuda)
    t64 = lambda v: torch.tensor(v, dtype=torch.int64, device=cuda)  # noqa: E731
    negative = [
        (lambda: f(data, indices, indptr, B, (2,)), ValueError),
        (lambda: f(data, indices, indptr, B[0], (2, 2)), ValueError),
        (lambda: f(data, indices, indptr, B.double(), (2, 2)), TypeError),
        (lambda: f(data, indices, indptr, torch.randn((3, 4), device=cuda), (2, 2)), ValueError),
        (lambda: f(data, indices, indptr[:-1], B, (2, 2)), ValueError),
        (lambda: f(data, indices, t64([1, 2, 3]), B, (2, 2)), ValueError),
        (lambda: f(data, indices, t64([0, 2, 2]), B, (2, 2)), ValueError),
        (lambda: f(data, indices, t64([0, 3, 2]), B, (2, 2)), ValueError),
        (lambda: f(data, torch.tensor([0, 3, 1], dtype=torch.int32, device=cuda), indptr, B,
                   (2, 2)), IndexError),
        (lambda: f(data, indices, indptr, B, (2, 2), block_n=0), ValueError),
        (lambda: f(data, indices, indptr, B, (2, 2), block_nnz=0), ValueError),
        (lambda: f(data, indices, indptr, B, (2, 2), max_segments=0), ValueError),
        (lambda: f(data, indices, indptr, B, (2, 2), out=torch.empty((3, 4), device=cuda)),
         ValueError),
        (lambda: f(data, indices, indptr, B, (2, 2), out=torch.empty((2, 4))), ValueError),
        (lambda: f(data, indices, indptr, B, (2, 2), op="bad"), ValueError),
        (lambda: f(data, indices, indptr, B, (2, 2), op="non", transpose=True), ValueError),
        (lambda: f(data, indices, indptr, torch.randn((3, 4), device=cuda), (2, 2), op="trans"),
         ValueError),
        (lambda: f(data, indices, indptr, B, (2, 2), op="trans",
                   out=torch.empty((2, 3), device=cuda)), ValueError),
    ]
    for fn, exc in negative:
        with pytest.raises(exc):
            fn()
    # the explicit max_segments override that is too small for a 1536-entry row
    idx = torch.cat([torch.arange(1536), torch.tensor([7, 129, 511, 1024])]).to(torch.int32).cuda()
    ptr = t64([0, 1536, 1540])
    vals = torch.randn(1540, device=cuda)
    Bl = torch.randn((2048, 48), device=cuda)
    with pytest.raises(ValueError, match="more CSR segments"):
        f(vals, idx, ptr, Bl, (2, 2048), block_nnz=128, max_segments=4)
    # messages pinned by the reference's pytest file
    with pytest.raises(ValueError, match="B.shape\\[0\\] must be n_cols=2"):
        f(data, indices, indptr, torch.randn((3, 4), device=cuda), (2, 2), op="trans")
    with pytest.raises(ValueError, match="out shape/dtype must match result"):
        f(data, indices, indptr, B, (2, 2), op="trans", out=torch.empty((2, 3), device=cuda))

    dense = torch.tensor([[1.0, 2.0], [0.0, 3.0]], device=cuda)
    out = torch.empty((2, 4), device=cuda)
    C = f(data, indices, indptr, B, (2, 2), out=out)
    assert C.data_ptr() == out.data_ptr()
    assert torch.allclose(C, dense @ B, atol=1e-6)
    assert torch.allclose(f(data, indices, indptr, B, (2, 2), op="trans"), dense.t() @ B, atol=1e-6)
    empty = f(data[:0], indices[:0], torch.zeros(3, dtype=torch.int64, device=cuda), B, (2, 2))
    assert empty.shape == (2, 4) and float(empty.abs().sum()) == 0.0
    assert f(data, indices, indptr, torch.empty((2, 0), device=cuda), (2, 2)).shape == (2, 0)
    # meta / timing
    C, ms, meta = f(data, indices.long(), indptr, B, (2, 2), op="trans", return_time=True,
                    return_meta=True)
    assert meta["op"] == "trans" and meta["symbolic_ms"] >= 0.0 and meta["compute_ms"] >= 0.0
    assert ms == pytest.approx(meta["op_total_ms"])
    assert meta["op_total_ms"] == pytest.approx(meta["symbolic_ms"] + meta["compute_ms"])
    C, meta = f(data, indices, indptr, B, (2, 2), op="non", return_meta=True)
    assert meta["op"] == "non" and meta["symbolic_ms"] == 0.0


def test_spmm_does_not_touch_rows_of_B_it_does_not_reference():
    """Non-finite values in a row of B that no entry of A points at must not reach C (guards the
    masked lanes of the vectorised inner loop, which read row 0 of B without adding it)."""
    from flagsparse_b200 import flagsparse_spmm_csr
    rng = np.random.default_rng(31)
    lengths = rng.integers(0, 40, 700)
    data, idx, ptr = csr_from_lengths(rng, lengths, 399, np.float32)
    idx = idx + 1                                  # nothing references column 0
    B = random_values(rng, 400 * 32, np.float32).reshape(400, 32)
    expect = oracle.spmm(data, idx, ptr, B, (700, 400))
    B[0, :] = np.inf
    B[0, ::2] = np.nan
    C = flagsparse_spmm_csr(dev(data), dev(idx, torch.int32), dev(ptr, torch.int32), dev(B),
                            (700, 400))
    assert np.isfinite(host(C)).all()
    assert_parity(host(C), expect, np.float32)


@pytest.fixture
def forced_long_row_split():
    """Thresholds low enough that small matrices take the long-row / column-panel route."""
    from flagsparse_b200 import _plan, clear_plan_cache, set_long_row_policy
    saved = (_plan.LONG_ROW_POLICY, _plan.LONG_ROW_MIN, _plan.LONG_ROW_TRIGGER_BYTES,
             _plan.LONG_ROW_TARGET_BYTES, _plan.LONG_ROW_MIN_SHARE, _plan.LONG_ROW_MIN_NNZ)
    clear_plan_cache()
    set_long_row_policy("auto", min_len=48, trigger_bytes=0, target_bytes=16 << 10,
                        min_share=0.0, min_nnz=0)
    yield
    set_long_row_policy(saved[0], *saved[1:])
    clear_plan_cache()


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("n_dense", [4, 32, 70])
@pytest.mark.parametrize("op", ["non", "trans"])
def test_spmm_long_rows_by_column_panel(dtype, n_dense, op, forced_long_row_split):
    """The three-launch route (short rows, long rows as a panel stack, combine) gives the oracle's
    result, with alpha / beta and an `out` that holds C_in, and is bit-identical run to run."""
    from flagsparse_b200 import _plan, flagsparse_spmm_csr, set_long_row_policy
    rng = np.random.default_rng(77 + n_dense)
    lengths = np.concatenate([[0, 49, 48, 3000, 1, 0, 700], rng.integers(0, 40, 600),
                              [5000, 0, 0, 64], rng.integers(0, 6, 500), [2100]])
    n_rows, n_cols = lengths.size, 2600
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype, sort=False)
    if op != "non":
        # hand over the transpose of that matrix, so that op(A) is the one with the long rows
        import scipy.sparse as sp
        At = sp.csr_matrix((data, idx, ptr), shape=(n_rows, n_cols)).T.tocsr()
        data, idx, ptr = At.data.astype(dtype), At.indices.astype(np.int64), At.indptr
        n_rows, n_cols = n_cols, n_rows
    k = n_rows if op != "non" else n_cols
    m = n_cols if op != "non" else n_rows
    B = random_values(rng, k * n_dense, dtype).reshape(k, n_dense)
    C0 = random_values(rng, m * n_dense, dtype).reshape(m, n_dense)
    d, i, p = dev(data), dev(idx, torch.int32), dev(ptr, torch.int64)
    C = flagsparse_spmm_csr(d, i, p, dev(B), (n_rows, n_cols), op=op)
    plan = _plan.cache_get(_plan.plan_key("spmm", d, i, p, (n_rows, n_cols)))
    if op != "non":
        plan = plan.transposed(conj=False)
    split = plan.long_row_split(n_dense * B.itemsize)
    assert split is not None and split.n_long >= 3 and split.n_panels >= 2
    assert split.short.nnz + split.stack.nnz == data.size
    assert_parity(host(C), oracle.spmm(data, idx, ptr, B, (n_rows, n_cols), op=op), dtype)
    out = dev(C0)
    got = flagsparse_spmm_csr(d, i, p, dev(B), (n_rows, n_cols), op=op, out=out, alpha=-0.75,
                              beta=1.25)
    assert got is out
    expect = oracle.spmm(data, idx, ptr, B, (n_rows, n_cols), op=op, alpha=-0.75, beta=1.25,
                         C0=C0)
    assert_parity(host(out), expect, dtype)
    again = flagsparse_spmm_csr(d, i, p, dev(B), (n_rows, n_cols), op=op)
    assert torch.equal(C.view(torch.uint8), again.view(torch.uint8))
    # the plain route on the same inputs agrees to rounding
    set_long_row_policy("off")
    from flagsparse_b200 import clear_plan_cache
    clear_plan_cache()
    plain = flagsparse_spmm_csr(d, i, p, dev(B), (n_rows, n_cols), op=op)
    assert_parity(host(C), host(plain), dtype)


def test_long_row_split_is_not_taken_for_small_or_uniform_matrices():
    from flagsparse_b200 import _plan
    assert _plan.long_row_shift(1 << 20, 64) is None            # B of 64 MB fits L2
    assert _plan.long_row_shift(1 << 24, 256) == 17             # 2^17 rows x 256 B = 32 MB
    assert _plan.long_row_shift(1 << 26, 64) == 19
    assert _plan.long_row_shift((1 << 31) - 1, 4096) == 23      # never more than 256 panels
    rng = np.random.default_rng(1)
    data, idx, ptr = csr_from_lengths(rng, rng.integers(0, 20, 500), 300, np.float32)
    plan = _plan.CsrPlan(dev(data), dev(idx, torch.int32), dev(ptr, torch.int64), (500, 300), 19)
    assert plan.long_row_split(1 << 20) is None


@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.complex64], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("n_dense", [4, 32, 64])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64], ids=["i32", "i64"])
def test_spmm_banded_matrix_uses_the_shared_memory_window(dtype, n_dense, idx_dtype):
    """A banded matrix (unsorted columns inside the band, empty rows, one dense row piece) whose
    tiles span few columns: B rows come from the shared-memory window.  Where the windowed kernel
    cuts the same tiles as the plain one it does the same additions in the same order and the
    two results are equal bit for bit; float32 with int32 columns runs longer tiles, so rows that
    cross a tile border are split elsewhere and the results agree to the parity tolerance."""
    from flagsparse_b200 import _lib as _lib_mod
    from flagsparse_b200 import _plan, clear_plan_cache, flagsparse_spmm_csr, set_window_policy
    rng = np.random.default_rng(300 + n_dense)
    n, band = 3000, 10
    rows, cols = [], []
    for r in range(n):
        if r % 97 == 5:
            continue                                   # empty row
        lo, hi = max(0, r - band), min(n, r + band)
        k = hi - lo if r == 1500 else int(rng.integers(8, 21))
        c = rng.choice(np.arange(lo, hi), size=min(k, hi - lo), replace=False)
        rows.append(np.full(c.size, r))
        cols.append(c)                                 # not sorted
    rows, cols = np.concatenate(rows), np.concatenate(cols)
    ptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=n), out=ptr[1:])
    data = random_values(rng, cols.size, dtype)
    B = random_values(rng, n * n_dense, dtype).reshape(n, n_dense)
    C0 = random_values(rng, n * n_dense, dtype).reshape(n, n_dense)
    d, i, p = dev(data), dev(cols, idx_dtype), dev(ptr, torch.int64)
    clear_plan_cache()
    set_window_policy("auto")
    try:
        out = dev(C0)
        flagsparse_spmm_csr(d, i, p, dev(B), (n, n), out=out, alpha=0.5, beta=-1.5)
        plan = _plan.cache_get(_plan.plan_key("spmm", d, i, p, (n, n)))
        lib = _lib_mod.load()
        w_items = lib.b2s_spmm_window_tile_items(plan.vcode, plan.icode)
        same_tiles = w_items == lib.b2s_spmm_tile_items(plan.vcode, plan.icode)
        assert same_tiles == (not (dtype == np.float32 and plan.indices.dtype == torch.int32))
        span = plan.window_rows(w_items)
        assert 0 < span < 200
        if n_dense * data.itemsize <= 128:   # wider B rows may not fit and take the plain kernel
            assert span * n_dense * data.itemsize <= _plan.WINDOW_MAX_BYTES
        expect = oracle.spmm(data, cols, ptr, B, (n, n), alpha=0.5, beta=-1.5, C0=C0)
        assert_parity(host(out), expect, dtype)
        C = flagsparse_spmm_csr(d, i, p, dev(B), (n, n))
        # B as a view with a wider pitch (whole 16-byte packs): the window copies pitch-sized
        # rows but for the last one
        pad = 16 // data.itemsize
        wide = torch.zeros((n, n_dense + pad), dtype=C.dtype, device="cuda")
        wide[:, :n_dense] = dev(B)
        assert torch.equal(flagsparse_spmm_csr(d, i, p, wide[:, :n_dense], (n, n)), C)
        set_window_policy("off")
        clear_plan_cache()
        plain = flagsparse_spmm_csr(d, i, p, dev(B), (n, n))
        if same_tiles:
            assert torch.equal(C.view(torch.uint8), plain.view(torch.uint8))
        else:
            assert_parity(host(C), host(plain), dtype)
    finally:
        set_window_policy("auto")
        clear_plan_cache()


def test_spmm_window_stat_entry_point():
    from flagsparse_b200 import _lib as L
    from flagsparse_b200._plan import CsrPlan
    lib = L.load()
    rng = np.random.default_rng(9)
    data, idx, ptr = csr_from_lengths(rng, rng.integers(0, 9, 4000), 5000, np.float32)
    plan = CsrPlan(dev(data), dev(idx, torch.int64), dev(ptr, torch.int64), (4000, 5000), 8)
    n_tiles, tile_row = plan.tiles(1024)
    widest = 0
    tr = host(tile_row)
    total = 4000 + data.size
    for t in range(n_tiles):
        j0 = min(t * 1024, total) - tr[t]
        j1 = min((t + 1) * 1024, total) - tr[t + 1]
        if j1 > j0:
            widest = max(widest, int(idx[j0:j1].max() - idx[j0:j1].min() + 1))
    assert plan.window_rows(1024) == widest
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = L.stream_handle(out.device)
    table = host(plan.window(1024)[1]) if plan.window(1024)[1] is not None else None
    if table is not None:
        assert int(table[1::2].max()) == widest and int(table[0::2].min()) >= 0
    assert lib.b2s_spmm_window_stat(1, None, 0, 0, None, 1024, L.ptr(out), None, stream) == 0
    assert lib.b2s_spmm_window_stat(1, None, 4, 4, None, 1024, L.ptr(out), None, stream) == 2
    assert lib.b2s_spmm_window_stat(1, None, 4, 4, None, 1024, None, None, stream) == 2
