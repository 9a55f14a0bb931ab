"""The C ABI called directly (ctypes, raw device pointers): tile plan invariants, the CSR -> CSC
kernel against the reference fixtures bit for bit, the status codes."""

import ctypes

import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden
from gpu_util import assert_parity, csr_from_lengths, dev, host, random_values

pytestmark = pytest.mark.gpu

TRANS_CASES = sorted(c for c in load_golden("spmv_reference.npz") if not c.endswith("_non"))


def _lib():
    from flagsparse_b200 import _lib
    return _lib.load(), _lib


def _merge_path_rows(ptr, n_rows, nnz, items):
    """numpy restatement of the merge-path search the plan kernel performs."""
    total = n_rows + nnz
    n_tiles = -(-total // items)
    out = np.empty(n_tiles + 1, dtype=np.int64)
    ends = ptr[1:]
    for t in range(n_tiles + 1):
        d = min(t * items, total)
        lo, hi = max(d - nnz, 0), min(d, n_rows)
        while lo < hi:
            mid = (lo + hi) // 2
            if ends[mid] <= d - mid - 1:
                lo = mid + 1
            else:
                hi = mid
        out[t] = lo
    return out


@pytest.mark.parametrize("items", [64, 1024, 2048])
def test_tile_plan_matches_merge_path(items):
    lib, L = _lib()
    rng = np.random.default_rng(2)
    lengths = np.concatenate([rng.integers(0, 4, 5000), [9000, 0, 0, 1], np.zeros(3000, int),
                              rng.integers(0, 300, 200)])
    ptr = np.zeros(lengths.size + 1, dtype=np.int64)
    np.cumsum(lengths, out=ptr[1:])
    n_rows, nnz = lengths.size, int(ptr[-1])
    for tdt, code in ((torch.int32, L.B2S_I32), (torch.int64, L.B2S_I64)):
        p = dev(ptr, tdt)
        T = lib.b2s_tile_count(n_rows, nnz, items)
        assert T == -(-(n_rows + nnz) // items)
        tile_row = torch.empty(T + 1, dtype=torch.int64, device="cuda")
        st = lib.b2s_tile_plan(L.ptr(p), code, n_rows, nnz, items, L.ptr(tile_row),
                               L.stream_handle(p.device))
        assert st == 0
        got = host(tile_row)
        assert np.array_equal(got, _merge_path_rows(ptr, n_rows, nnz, items))
        # invariants the kernels rely on
        d = np.minimum(np.arange(T + 1) * items, n_rows + nnz)
        j = d - got
        assert got[0] == 0 and got[-1] == n_rows and j[-1] == nnz
        assert np.all(np.diff(got) >= 0) and np.all(np.diff(j) >= 0)
        assert np.all(ptr[got] <= j) and np.all(j <= ptr[np.minimum(got + 1, n_rows)])


@pytest.mark.parametrize("case", TRANS_CASES)
def test_csr2csc_bit_identical_to_reference_transpose(case, spmv_golden):
    """b2s_csr2csc against the output of the reference's _transpose_csr_for_spmv
    (spmv_csr.py:477-515) on the same input: same permutation, same bits."""
    lib, L = _lib()
    c = spmv_golden[case]
    n_rows = c["indptr"].shape[0] - 1
    n_cols = int(case.split("_")[1].split("x")[1])
    conj = case.endswith("_conj")
    data, idx, ptr = dev(c["data"]), dev(c["indices"]), dev(c["indptr"])
    nnz = data.numel()
    t_data, t_idx = torch.empty_like(data), torch.empty_like(idx)
    t_ptr = torch.empty(n_cols + 1, dtype=torch.int64, device="cuda")
    nbytes = lib.b2s_csr2csc_bytes(n_rows, n_cols, nnz)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    st = lib.b2s_csr2csc(L.VALUE_CODE[data.dtype], L.B2S_I64, L.B2S_I64, L.ptr(data), L.ptr(idx),
                         L.ptr(ptr), n_rows, n_cols, nnz, int(conj), L.ptr(t_data), L.ptr(t_idx),
                         L.ptr(t_ptr), L.ptr(ws), nbytes, L.stream_handle(data.device))
    assert st == 0
    assert np.array_equal(host(t_ptr), c["t_indptr"])
    assert np.array_equal(host(t_idx), c["t_indices"])
    assert np.array_equal(host(t_data).view(np.uint8), c["t_data"].view(np.uint8))
    too_small = lib.b2s_csr2csc(L.VALUE_CODE[data.dtype], L.B2S_I64, L.B2S_I64, L.ptr(data),
                                L.ptr(idx), L.ptr(ptr), n_rows, n_cols, nnz, int(conj),
                                L.ptr(t_data), L.ptr(t_idx), L.ptr(t_ptr), L.ptr(ws), 16,
                                L.stream_handle(data.device))
    assert too_small == 6 and b"scratch" in lib.b2s_status_string(too_small)


@pytest.mark.parametrize("n_cols", [1, 255, 257, 70000, 17_000_000])
def test_csr2csc_large_random_vs_oracle(n_cols):
    """1, 2 and 3+ radix passes; several thousand CTAs; unsorted columns with duplicates."""
    from flagsparse_b200._plan import CsrPlan
    rng = np.random.default_rng(n_cols)
    n_rows = 20000
    data, idx, ptr = csr_from_lengths(rng, rng.integers(0, 60, n_rows), n_cols, np.complex64,
                                      sort=False)
    plan = CsrPlan(dev(data), dev(idx, torch.int32), dev(ptr), (n_rows, n_cols), -1)
    t = plan.transposed(conj=True)
    e_data, e_idx, e_ptr, _ = oracle.transpose_csr(data, idx, ptr, (n_rows, n_cols), conj=True)
    assert np.array_equal(host(t.indptr), e_ptr)
    assert np.array_equal(host(t.indices), e_idx)
    assert np.array_equal(host(t.data).view(np.uint8), e_data.view(np.uint8))


def test_raw_spmv_spmm_calls_and_status_codes():
    lib, L = _lib()
    rng = np.random.default_rng(9)
    n_rows, n_cols = 3000, 2000
    data, idx, ptr = csr_from_lengths(rng, rng.integers(0, 50, n_rows), n_cols, np.float64)
    x = random_values(rng, n_cols, np.float64)
    d, i, p, xd = dev(data), dev(idx, torch.int32), dev(ptr, torch.int32), dev(x)
    nnz = d.numel()
    items = lib.b2s_spmv_tile_items(L.B2S_F64, L.B2S_I32)
    T = lib.b2s_tile_count(n_rows, nnz, items)
    tile_row = torch.empty(T + 1, dtype=torch.int64, device="cuda")
    s = L.stream_handle(d.device)
    assert lib.b2s_tile_plan(L.ptr(p), L.B2S_I32, n_rows, nnz, items, L.ptr(tile_row), s) == 0
    carry = torch.empty(T, dtype=torch.float64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.empty(n_rows, dtype=torch.float64, device="cuda")
    one, zero = (ctypes.c_double * 1)(1.0), (ctypes.c_double * 1)(0.0)
    st = lib.b2s_spmv_csr(L.B2S_F64, L.B2S_I32, L.B2S_I32, L.ptr(d), L.ptr(i), L.ptr(p), n_rows,
                          n_cols, nnz, L.ptr(xd), None, L.ptr(y), one, zero, L.ptr(tile_row),
                          L.ptr(carry), L.ptr(status), s)
    assert st == 0
    assert_parity(host(y), oracle.spmv(data, idx, ptr, x, (n_rows, n_cols)), np.float64)
    assert int(status.item()) == 0
    # status codes: bad dtype, beta != 0 without y_in, misaligned pointer
    args = [L.B2S_F64, L.B2S_I32, L.B2S_I32, L.ptr(d), L.ptr(i), L.ptr(p), n_rows, n_cols, nnz,
            L.ptr(xd), None, L.ptr(y), one, zero, L.ptr(tile_row), L.ptr(carry), L.ptr(status), s]
    bad = list(args); bad[0] = 9
    assert lib.b2s_spmv_csr(*bad) == 1
    bad = list(args); bad[13] = one
    assert lib.b2s_spmv_csr(*bad) == 2
    bad = list(args); bad[11] = ctypes.c_void_p(y.data_ptr() + 4)
    assert lib.b2s_spmv_csr(*bad) == 3
    assert lib.b2s_version() == 100

    n_dense = 8
    B = random_values(rng, n_cols * n_dense, np.float64).reshape(n_cols, n_dense)
    Bd = dev(B)
    items = lib.b2s_spmm_tile_items(L.B2S_F64, L.B2S_I32)
    T = lib.b2s_tile_count(n_rows, nnz, items)
    tile_row = torch.empty(T + 1, dtype=torch.int64, device="cuda")
    assert lib.b2s_tile_plan(L.ptr(p), L.B2S_I32, n_rows, nnz, items, L.ptr(tile_row), s) == 0
    carry = torch.empty(T * n_dense, dtype=torch.float64, device="cuda")
    C = torch.empty((n_rows, n_dense), dtype=torch.float64, device="cuda")
    st = lib.b2s_spmm_csr(L.B2S_F64, L.B2S_I32, L.B2S_I32, L.ptr(d), L.ptr(i), L.ptr(p), n_rows,
                          n_cols, nnz, L.ptr(Bd), n_dense, n_dense, None, L.ptr(C), n_dense, one,
                          zero, L.ptr(tile_row), L.ptr(carry), L.ptr(status), s)
    assert st == 0
    assert_parity(host(C), oracle.spmm(data, idx, ptr, B, (n_rows, n_cols)), np.float64)


def test_inspect_reports_contract_violations():
    lib, L = _lib()
    ptr = torch.tensor([0, 3, 2, 2, 7], dtype=torch.int64, device="cuda")
    idx = torch.tensor([5, -2, 9, 1, 1, 1, 4], dtype=torch.int32, device="cuda")
    stats = torch.empty(8, dtype=torch.int64, device="cuda")
    st = lib.b2s_csr_inspect(L.ptr(ptr), L.B2S_I64, L.ptr(idx), L.B2S_I32, 4, 7, L.ptr(stats),
                             L.stream_handle(ptr.device))
    assert st == 0
    assert stats.tolist()[:7] == [0, 7, 1, -2, 9, 5, 1]


def test_bounded_wait_runs_out_with_a_status_bit_not_a_hang():
    """A wait that can never be satisfied gives up after its iteration limit, reports
    B2S_ERR_TIMEOUT through the status word, and leaves the context usable; the Python layer
    turns the bit into an exception."""
    lib, L = _lib()
    from flagsparse_b200._plan import CsrPlan
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.b2s_selftest_wait_timeout(L.ptr(status), 200, L.stream_handle(status.device)) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1 << L.B2S_ERR_TIMEOUT
    assert lib.b2s_selftest_wait_timeout(L.ptr(status), 0, L.stream_handle(status.device)) == 2
    # the context still works, and a plan whose status word carries the bit raises
    ptr = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    plan = CsrPlan(torch.ones(1, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"),
                   ptr, (1, 1), 1)
    plan.status.copy_(status)
    with pytest.raises(RuntimeError, match="bounded wait"):
        plan.check_status()
    assert int(plan.status.item()) == 0
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


def test_csr2csc_with_more_than_2_31_columns_uses_the_64_bit_sort():
    """n_cols just above 2^31 forces the 64-bit keys of the radix sort (the path nnz > 2^31 would
    also take).  Checked against torch's stable sort on the device; needs ~30 GB of HBM."""
    lib, L = _lib()
    if torch.cuda.get_device_properties(0).total_memory < 60 * 2**30:
        pytest.skip("needs a large GPU")
    n_cols = 2**31 + 1000
    n_rows = 3000
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    lengths = torch.randint(0, 700, (n_rows,), generator=g, device="cuda")
    ptr = torch.zeros(n_rows + 1, dtype=torch.int64, device="cuda")
    torch.cumsum(lengths, 0, out=ptr[1:])
    nnz = int(ptr[-1])
    # columns: half spread over the whole range, half piled onto a few columns (long output rows)
    idx = torch.randint(0, n_cols, (nnz,), generator=g, device="cuda", dtype=torch.int64)
    idx[::2] = (idx[::2] % 7) * 300_000_007 % n_cols
    data = torch.randn(nnz, generator=g, device="cuda", dtype=torch.float32)
    t_data, t_idx = torch.empty_like(data), torch.empty_like(idx)
    t_ptr = torch.empty(n_cols + 1, dtype=torch.int64, device="cuda")
    nbytes = lib.b2s_csr2csc_bytes(n_rows, n_cols, nnz)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    st = lib.b2s_csr2csc(L.B2S_F32, L.B2S_I64, L.B2S_I64, L.ptr(data), L.ptr(idx), L.ptr(ptr),
                         n_rows, n_cols, nnz, 0, L.ptr(t_data), L.ptr(t_idx), L.ptr(t_ptr),
                         L.ptr(ws), nbytes, L.stream_handle(data.device))
    assert st == 0
    order = torch.sort(idx, stable=True).indices
    rows = torch.repeat_interleave(torch.arange(n_rows, device="cuda"), lengths)
    assert torch.equal(t_idx, rows[order])
    assert torch.equal(t_data, data[order])
    # column pointers: spot-check against counts (a full bincount would need 17 GB more)
    assert int(t_ptr[0]) == 0 and int(t_ptr[-1]) == nnz
    probe = torch.unique(idx)[:2000]
    counts = (idx.unsqueeze(0) == probe[:50].unsqueeze(1)).sum(1)
    assert torch.equal(t_ptr[probe[:50] + 1] - t_ptr[probe[:50]], counts)
    assert bool((t_ptr[1:200_000] >= t_ptr[:199_999]).all())
    del ws, t_ptr
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.complex64, torch.complex128],
                         ids=lambda d: str(d).replace("torch.", ""))
@pytest.mark.parametrize("n_rows,row_offset", [(1001, 0), (1000, 4), (777, 3), (5, 1)])
def test_panel_combine_peers_stores_the_same_values_as_panel_combine(dtype, n_rows, row_offset):
    """b2s_panel_combine_peers with two buffers of this GPU standing for the peers: every buffer
    receives, at row_offset, exactly what b2s_panel_combine writes (16-byte stores where the
    block is aligned, by value otherwise and at the ragged end), and nothing outside the block."""
    lib, L = _lib()
    g = torch.Generator(device="cuda")
    g.manual_seed(n_rows + row_offset)
    n_panels = 3
    real = torch.float64 if dtype in (torch.float64, torch.complex128) else torch.float32
    def rand(n):
        if dtype.is_complex:
            return torch.complex(torch.randn(n, dtype=real, device="cuda", generator=g),
                                 torch.randn(n, dtype=real, device="cuda", generator=g))
        return torch.randn(n, dtype=dtype, device="cuda", generator=g)
    n_part = 2 * n_rows
    ypart = rand(n_part)
    subpos = torch.randint(-1, n_part, (n_panels * n_rows,), dtype=torch.int32, device="cuda",
                           generator=g)
    y_in = rand(n_rows)
    vcode = L.VALUE_CODE[dtype]
    a, b = L.scalar_buffer(0.75, dtype), L.scalar_buffer(-0.5, dtype)
    stream = L.stream_handle(ypart.device)
    want = torch.empty(n_rows, dtype=dtype, device="cuda")
    assert lib.b2s_panel_combine(vcode, L.ptr(ypart), L.ptr(subpos), n_rows, n_panels,
                                 L.ptr(y_in), L.ptr(want), a, b, stream) == 0
    peer_rows = row_offset + n_rows + 7
    bufs = [torch.full((peer_rows,), 9.0, dtype=dtype, device="cuda") for _ in range(2)]
    arr = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in bufs])
    for grid_limit in (0, 2):
        for t in bufs:
            t.fill_(9.0)
        assert lib.b2s_panel_combine_peers(vcode, L.ptr(ypart), L.ptr(subpos), n_rows, n_panels,
                                           L.ptr(y_in), arr, 2, row_offset, peer_rows, a, b,
                                           grid_limit, stream) == 0
        torch.cuda.synchronize()
        for t in bufs:
            assert torch.equal(t[row_offset:row_offset + n_rows].view(torch.uint8),
                               want.view(torch.uint8))
            assert bool((t[:row_offset] == 9.0).all()) and bool(
                (t[row_offset + n_rows:] == 9.0).all())
    # a block that does not fit the peers' buffers is refused
    assert lib.b2s_panel_combine_peers(vcode, L.ptr(ypart), L.ptr(subpos), n_rows, n_panels,
                                       L.ptr(y_in), arr, 2, 8, n_rows + 7, a, b, 0, stream) == \
        2   # B2S_ERR_ARG


def test_window_entry_points_say_when_the_windowed_kernel_can_run():
    """b2s_spmm_window_tile_items / b2s_spmm_window_usable, and b2s_spmm_csr_windowed refusing a
    window it cannot use instead of running the wrong tile plan."""
    lib, L = _lib()
    assert lib.b2s_spmm_window_tile_items(L.B2S_F32, L.B2S_I32) == 1536
    for v, i in ((L.B2S_F64, L.B2S_I32), (L.B2S_F32, L.B2S_I64), (L.B2S_C64, L.B2S_I32)):
        assert lib.b2s_spmm_window_tile_items(v, i) == lib.b2s_spmm_tile_items(v, i)
    n, N = 4096, 32
    B = torch.zeros((n, N + 4), dtype=torch.float32, device="cuda")
    C = torch.zeros((n, N), dtype=torch.float32, device="cuda")
    ok = lambda b, ldb, nd, c, ldc, rows: lib.b2s_spmm_window_usable(  # noqa: E731
        L.B2S_F32, b, ldb, nd, None, c, ldc, n, rows)
    assert ok(L.ptr(B), N + 4, N, L.ptr(C), N, 100) == 1
    assert ok(L.ptr(B), N + 4, N, L.ptr(C), N, 0) == 0                 # no window
    assert ok(L.ptr(B), N + 4, N, L.ptr(C), N, 300) == 0               # 300 rows x 144 B > 32 KB
    assert ok(L.ptr(B), N + 3, N, L.ptr(C), N, 100) == 0               # pitch not a multiple of 16
    assert ok(L.ptr(B[:, 1:]), N + 4, N, L.ptr(C), N, 100) == 0        # B not 16-byte aligned
    assert ok(L.ptr(B), N + 4, N - 2, L.ptr(C), N, 100) == 0           # ragged last pack
    assert ok(L.ptr(B), N + 4, 256, L.ptr(C), 256, 10) == 0            # more than one column tile
    # a window that cannot be used is refused, not silently run on the plain kernel's tiles
    data = torch.ones(8, dtype=torch.float32, device="cuda")
    col = torch.arange(8, dtype=torch.int32, device="cuda")
    ptr = torch.arange(0, 9, dtype=torch.int32, device="cuda")
    items = lib.b2s_spmm_window_tile_items(L.B2S_F32, L.B2S_I32)
    T = lib.b2s_tile_count(8, 8, items)
    tile_row = torch.zeros(T + 1, dtype=torch.int64, device="cuda")
    table = torch.zeros(2 * T, dtype=torch.int32, device="cuda")
    carry = torch.zeros(T * N, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    s = L.stream_handle(data.device)
    assert lib.b2s_tile_plan(L.ptr(ptr), L.B2S_I32, 8, 8, items, L.ptr(tile_row), s) == 0
    a, b = L.scalar_buffer(1.0, torch.float32), L.scalar_buffer(0.0, torch.float32)
    st = lib.b2s_spmm_csr_windowed(L.B2S_F32, L.B2S_I32, L.B2S_I32, L.ptr(data), L.ptr(col),
                                   L.ptr(ptr), 8, n, 8, L.ptr(B), N + 3, N, None, L.ptr(C), N,
                                   a, b, L.ptr(tile_row), L.ptr(carry), L.ptr(status), 100,
                                   L.ptr(table), s)
    assert st == 2   # B2S_ERR_ARG
    torch.cuda.synchronize()
