"""GPU parity of flagsparse_spmv_csr (CUDA path) against the CPU oracle and the reference
fixtures.  Tolerance: rel-L2 <= 1e-5 (float32 / complex64), <= 1e-12 (float64 / complex128);
results must repeat bit for bit."""

import numpy as np
import pytest
import torch

import oracle
from conftest import ALLCLOSE_TOL, load_golden
from gpu_util import TORCH_OF, assert_parity, csr_from_lengths, dev, host, random_values

pytestmark = pytest.mark.gpu


def _lib_mod():
    from flagsparse_b200 import _lib
    return _lib

SPMV_CASES = sorted(load_golden("spmv_reference.npz"))
DTYPES = [np.float32, np.float64, np.complex64, np.complex128]


def _shape_of(case, c):
    n_rows = c["indptr"].shape[0] - 1
    if case.startswith("spmv_longrows"):
        return n_rows, 3000
    return n_rows, int(case.split("_")[1].split("x")[1])


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64], ids=["int32", "int64"])
@pytest.mark.parametrize("case", SPMV_CASES)
def test_spmv_matches_reference_fixture(case, index_dtype, spmv_golden):
    from flagsparse_b200 import flagsparse_spmv_csr
    c = spmv_golden[case]
    op = case.rsplit("_", 1)[1]
    shape = _shape_of(case, c)
    y = flagsparse_spmv_csr(dev(c["data"]), dev(c["indices"], index_dtype),
                            dev(c["indptr"], index_dtype), dev(c["x"]), shape, op=op)
    assert_parity(host(y), c["y"], c["y"].dtype, case)
    tol = ALLCLOSE_TOL[c["y"].dtype]
    assert np.allclose(host(y), c["y"], rtol=max(tol, 1e-5 if tol > 1e-7 else tol), atol=tol * 8)


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("ptr_dtype", [torch.int32, torch.int64], ids=["p32", "p64"])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64], ids=["i32", "i64"])
@pytest.mark.parametrize("op", ["non", "trans", "conj"])
def test_spmv_ragged_rows_vs_oracle(dtype, idx_dtype, ptr_dtype, op):
    """Row lengths 0, 1, 31, 32, 33, a row longer than several tiles, runs of empty rows."""
    from flagsparse_b200 import flagsparse_spmv_csr
    rng = np.random.default_rng(11)
    lengths = np.concatenate([
        [0, 1, 31, 32, 33, 0, 0, 7000, 2, 1025, 1024, 255, 257, 0],
        rng.integers(0, 6, 3000), np.zeros(2500, dtype=np.int64), rng.integers(0, 70, 500), [0, 0]])
    n_rows, n_cols = lengths.size, 5000
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype)
    x = random_values(rng, n_rows if op != "non" else n_cols, dtype)
    expect = oracle.spmv(data, idx, ptr, x, (n_rows, n_cols), op=op)
    y = flagsparse_spmv_csr(dev(data), dev(idx, idx_dtype), dev(ptr, ptr_dtype), dev(x),
                            (n_rows, n_cols), op=op)
    assert_parity(host(y), expect, dtype)
    y2 = flagsparse_spmv_csr(dev(data), dev(idx, idx_dtype), dev(ptr, ptr_dtype), dev(x),
                             (n_rows, n_cols), op=op)
    assert torch.equal(y.view(torch.uint8), y2.view(torch.uint8)), "not bit-identical run to run"


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
def test_spmv_alpha_beta_epilogue(dtype):
    from flagsparse_b200 import flagsparse_spmv_csr
    rng = np.random.default_rng(5)
    lengths = rng.integers(0, 40, 4000)
    lengths[17] = 9000
    data, idx, ptr = csr_from_lengths(rng, lengths, 3000, dtype)
    x = random_values(rng, 3000, dtype)
    y0 = random_values(rng, 4000, dtype)
    alpha, beta = (1.5, 0.5) if np.dtype(dtype).kind != "c" else (1.5 - 0.25j, 0.5 + 2j)
    expect = oracle.spmv(data, idx, ptr, x, (4000, 3000), alpha=alpha, beta=beta, y0=y0)
    out = dev(y0)
    y = flagsparse_spmv_csr(dev(data), dev(idx), dev(ptr), dev(x), (4000, 3000), out=out,
                            alpha=alpha, beta=beta)
    assert y is out
    assert_parity(host(y), expect, dtype)
    with pytest.raises(ValueError, match="beta != 0 requires out"):
        flagsparse_spmv_csr(dev(data), dev(idx), dev(ptr), dev(x), (4000, 3000), beta=0.5)
    # beta == 0 must not read out: NaNs in it may not leak
    nan_out = torch.full((4000,), float("nan"), dtype=TORCH_OF[np.dtype(dtype)], device="cuda")
    y = flagsparse_spmv_csr(dev(data), dev(idx), dev(ptr), dev(x), (4000, 3000), out=nan_out)
    assert_parity(host(y), oracle.spmv(data, idx, ptr, x, (4000, 3000)), dtype)


def test_spmv_edge_shapes():
    from flagsparse_b200 import flagsparse_spmv_csr
    f = torch.float32
    # zero rows
    y = flagsparse_spmv_csr(torch.empty(0, dtype=f, device="cuda"),
                            torch.empty(0, dtype=torch.int32, device="cuda"),
                            torch.zeros(1, dtype=torch.int32, device="cuda"),
                            torch.ones(4, dtype=f, device="cuda"), (0, 4))
    assert y.shape == (0,)
    # rows but no entries -> zeros
    y = flagsparse_spmv_csr(torch.empty(0, dtype=f, device="cuda"),
                            torch.empty(0, dtype=torch.int64, device="cuda"),
                            torch.zeros(5001, dtype=torch.int64, device="cuda"),
                            torch.ones(4, dtype=f, device="cuda"), (5000, 4))
    assert y.shape == (5000,) and float(y.abs().sum()) == 0.0
    # duplicate + unsorted columns are summed; misaligned views are accepted
    data = torch.tensor([9.0, 1.0, 2.0, 3.0, 4.0], device="cuda")[1:]
    idx = torch.tensor([0, 2, 0, 0, 1], dtype=torch.int32, device="cuda")[1:]
    ptr = torch.tensor([0, 0, 3, 3, 4], dtype=torch.int64, device="cuda")
    x = torch.tensor([7.0, 1.0, 10.0, 100.0], device="cuda")[1:]
    y = flagsparse_spmv_csr(data, idx, ptr, x, (4, 3))
    assert y.tolist() == [0.0, 105.0, 0.0, 40.0]
    # strided (non-contiguous) inputs
    big = torch.arange(12, dtype=f, device="cuda")
    y = flagsparse_spmv_csr(big[::3], torch.tensor([0, 1, 2, 0], dtype=torch.int32, device="cuda"),
                            torch.tensor([0, 2, 4], dtype=torch.int32, device="cuda"),
                            torch.ones(6, dtype=f, device="cuda")[::2], (2, 3))
    assert y.tolist() == [3.0, 15.0]


def test_spmv_cfg1_full_size_vs_oracle():
    """float32/int32 65,536^2, 1-32 entries per row: the CPU-sized configuration, full size."""
    from flagsparse_b200 import flagsparse_spmv_csr, workloads
    p = workloads.cfg1_uniform_spmv(device="cuda")
    y = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape)
    expect = oracle.spmv(host(p.data), host(p.indices), host(p.indptr), host(p.x), p.shape)
    assert_parity(host(y), expect, np.float32)


@pytest.mark.parametrize("scale", [64])
def test_spmv_cfg2_scaled_vs_oracle(scale):
    """float64/int64 power-law rows (Zipf 1.8, longest row tens of thousands of entries),
    alpha=1.5 beta=0.5, at 1/64 of the benchmark's row count."""
    from flagsparse_b200 import flagsparse_spmv_csr, workloads
    p = workloads.cfg2_powerlaw_spmv(device="cuda", scale=scale)
    out = p.y0.clone()
    y = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, out=out, alpha=p.alpha,
                            beta=p.beta)
    expect = oracle.spmv(host(p.data), host(p.indices), host(p.indptr), host(p.x), p.shape,
                         alpha=p.alpha, beta=p.beta, y0=host(p.y0))
    assert_parity(host(y), expect, np.float64)
    out2 = p.y0.clone()
    flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, out=out2, alpha=p.alpha,
                        beta=p.beta)
    assert torch.equal(out, out2)


def test_spmv_cfg2_full_size_properties():
    """Full 2^24-row power-law matrix: compared with torch's own CSR product (an independent
    implementation), linearity in x, and bit-identical repeats."""
    from flagsparse_b200 import flagsparse_spmv_csr, workloads
    p = workloads.cfg2_powerlaw_spmv(device="cuda")
    y = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape)
    A = torch.sparse_csr_tensor(p.indptr, p.indices, p.data, size=p.shape)
    ref = (A @ p.x.unsqueeze(1)).squeeze(1)
    err = float(torch.linalg.vector_norm(y - ref) / torch.linalg.vector_norm(ref))
    assert err <= 1e-12, err
    x2 = torch.randn_like(p.x)
    y2 = flagsparse_spmv_csr(p.data, p.indices, p.indptr, x2, p.shape)
    y12 = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x + x2, p.shape)
    lin = float(torch.linalg.vector_norm(y12 - (y + y2)) / torch.linalg.vector_norm(y12))
    assert lin <= 1e-12, lin
    again = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape)
    assert torch.equal(y, again)


def test_spmv_prepared_and_contract_errors():
    import flagsparse_b200.spmv as mod
    from flagsparse_b200 import flagsparse_spmv_csr, prepare_spmv_csr
    rng = np.random.default_rng(3)
    data, idx, ptr = csr_from_lengths(rng, rng.integers(0, 9, 64), 48, np.float32)
    d, i, p = dev(data), dev(idx, torch.int32), dev(ptr, torch.int32)
    x = dev(random_values(rng, 48, np.float32))
    xt = dev(random_values(rng, 64, np.float32))
    prep = prepare_spmv_csr(d, i, p, (64, 48))
    y = flagsparse_spmv_csr(x=x, prepared=prep)
    assert_parity(host(y), oracle.spmv(data, idx, ptr, host(x), (64, 48)), np.float32)
    prep_t = prepare_spmv_csr(d, i, p, (64, 48), op="trans")
    assert prep_t.transpose and prep_t.shape == (48, 64)
    yt = flagsparse_spmv_csr(x=xt, prepared=prep_t)
    assert_parity(host(yt), oracle.spmv(data, idx, ptr, host(xt), (64, 48), op="trans"),
                  np.float32)
    # tests/pytest/test_spmv_csr_accuracy.py:128-149
    with pytest.raises(ValueError, match="does not match prepared.transpose"):
        flagsparse_spmv_csr(x=x, prepared=prep, transpose=True)
    with pytest.raises(ValueError, match="does not match prepared.op"):
        flagsparse_spmv_csr(x=x, prepared=prep, op="trans")
    with pytest.raises(ValueError, match="transpose conflicts with op"):
        flagsparse_spmv_csr(d, i, p, x, (64, 48), op="non", transpose=True)
    with pytest.raises(ValueError, match="op must be one of"):
        flagsparse_spmv_csr(d, i, p, x, (64, 48), op="bad")
    with pytest.raises(TypeError, match="x dtype must match"):
        flagsparse_spmv_csr(d, i, p, x.double(), (64, 48))
    with pytest.raises(ValueError, match="x length must be n_cols=48"):
        flagsparse_spmv_csr(d, i, p, xt, (64, 48))
    with pytest.raises(TypeError, match="data dtype must be one of"):
        flagsparse_spmv_csr(d.to(torch.int32), i, p, x.to(torch.int32), (64, 48))
    with pytest.raises(ValueError, match="must be CUDA tensors"):
        flagsparse_spmv_csr(d.cpu(), i.cpu(), p.cpu(), x, (64, 48))
    with pytest.raises(ValueError, match="indptr must start at zero"):
        flagsparse_spmv_csr(d, i, p + 1, x, (64, 48))
    bad = p.clone()
    bad[-1] += 1
    with pytest.raises(ValueError, match="must equal nnz"):
        flagsparse_spmv_csr(d, i, bad, x, (64, 48))
    bad = p.clone()
    bad[3], bad[4] = int(p[4]) + 1, int(p[3])
    with pytest.raises(ValueError, match="non-decreasing"):
        flagsparse_spmv_csr(d, i, bad, x, (64, 48))
    bad_i = i.clone()
    bad_i[0] = 48
    with pytest.raises(IndexError, match="indices out of range"):
        flagsparse_spmv_csr(d, bad_i, p, x, (64, 48))
    with pytest.raises(ValueError, match="out shape/dtype must match result"):
        flagsparse_spmv_csr(d, i, p, x, (64, 48), out=torch.empty(63, device="cuda"))
    # timing / meta tuples (spmv_csr.py:901-913)
    y, ms, meta = flagsparse_spmv_csr(d, i, p, x, (64, 48), return_time=True, return_meta=True)
    assert ms == pytest.approx(meta["op_total_ms"]) and meta["symbolic_ms"] == 0.0
    assert set(meta) == {"symbolic_ms", "compute_ms", "op_total_ms", "bucket_count"}
    assert mod._INDEX_LIMIT_INT32 == 2**31 - 1


def test_spmv_int64_fallback_policy(monkeypatch):
    """The retry contract of tests/pytest/test_spmv_csr_accuracy.py:152-234: a failing int64
    launch is retried on int32 copies under 'auto', re-raised under 'strict', and refused when an
    index does not fit."""
    import flagsparse_b200.spmv as mod
    from flagsparse_b200 import flagsparse_spmv_csr
    rng = np.random.default_rng(4)
    data, idx, ptr = csr_from_lengths(rng, rng.integers(0, 9, 32), 20, np.float64)
    d, i, p, x = dev(data), dev(idx), dev(ptr), dev(random_values(rng, 20, np.float64))
    real_impl = mod._b200_spmv_csr_impl_prepared
    calls = []

    def flaky(prepared, x, **kw):
        calls.append(prepared.kernel_indices.dtype)
        if prepared.kernel_indices.dtype == torch.int64:
            raise RuntimeError("forced native int64 failure")
        return real_impl(prepared, x, **kw)

    # the reference's test patches the launcher under its Triton name; both names work here
    monkeypatch.setattr(mod, "_triton_spmv_csr_impl_prepared", flaky)
    y = flagsparse_spmv_csr(d, i, p, x, (32, 20), index_fallback_policy="auto")
    assert calls == [torch.int64, torch.int32]
    assert_parity(host(y), oracle.spmv(data, idx, ptr, host(x), (32, 20)), np.float64)
    with pytest.raises(RuntimeError, match="forced native int64 failure"):
        flagsparse_spmv_csr(d, i, p, x, (32, 20), index_fallback_policy="strict")
    prepared = mod.prepare_spmv_csr(d, i, p, (32, 20))
    prepared.n_rows = mod._INDEX_LIMIT_INT32 + 1
    with pytest.raises(RuntimeError, match="int32 fallback is unsafe"):
        mod._run_spmv_prepared_with_fallback(prepared, x)


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64], ids=["i32", "i64"])
@pytest.mark.parametrize("target_elems", [32, 512, 2048])
def test_spmv_column_panel_layout_vs_oracle(monkeypatch, dtype, idx_dtype, target_elems):
    """The column-panel layout (normally used only when x outgrows L2) forced onto a small
    matrix: 2 .. 200 panels, panels with no entries, tiles that straddle several panels, rows
    longer than a tile, alpha / beta, bit-identical repeats."""
    import flagsparse_b200._plan as plan_mod
    from flagsparse_b200 import clear_plan_cache, flagsparse_spmv_csr
    monkeypatch.setattr(plan_mod, "PANEL_TRIGGER_BYTES", 0)
    monkeypatch.setattr(plan_mod, "PANEL_TARGET_BYTES", target_elems * np.dtype(dtype).itemsize)
    monkeypatch.setattr(plan_mod, "PANEL_MIN_NNZ", 0)
    clear_plan_cache()
    rng = np.random.default_rng(target_elems)
    lengths = np.concatenate([[0, 1, 5000, 0, 33], rng.integers(0, 12, 3000), [2500, 0]])
    n_rows, n_cols = lengths.size, 6000
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype, sort=False)
    idx[idx >= 5000] //= 7      # leave the last panels (almost) empty
    x = random_values(rng, n_cols, dtype)
    y0 = random_values(rng, n_rows, dtype)
    alpha, beta = (1.5, 0.5) if np.dtype(dtype).kind != "c" else (1.5 - 0.25j, 0.5 + 2j)
    expect = oracle.spmv(data, idx, ptr, x, (n_rows, n_cols), alpha=alpha, beta=beta, y0=y0)
    args = (dev(data), dev(idx, idx_dtype), dev(ptr, idx_dtype), dev(x), (n_rows, n_cols))
    out = dev(y0)
    y = flagsparse_spmv_csr(*args, out=out, alpha=alpha, beta=beta)
    plan = plan_mod.cache_get(plan_mod.plan_key("spmv", args[0], args[1], args[2], args[4]))
    assert plan is not None and plan.panels() is not None and plan.panels().n_panels >= 2
    assert_parity(host(y), expect, dtype)
    out2 = dev(y0)
    flagsparse_spmv_csr(*args, out=out2, alpha=alpha, beta=beta)
    assert torch.equal(out.view(torch.uint8), out2.view(torch.uint8))
    yt = flagsparse_spmv_csr(*args[:3], dev(random_values(rng, n_rows, dtype)), args[4], op="trans")
    assert yt.shape == (n_cols,)
    clear_plan_cache()


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64], ids=["i32", "i64"])
@pytest.mark.parametrize("slice_cols", [64, 1024])
def test_spmv_long_rows_from_shared_memory_slices(monkeypatch, dtype, idx_dtype, slice_cols):
    """The long rows of a panel-layout matrix are multiplied from shared-memory slices of x
    (b2s_spmv_stack_shared).  Forced onto a small matrix: narrow panels of 64 / 1024 columns
    (so 94 / 6 slices), several CTAs per slice, rows that span many tiles, rows that end
    exactly on tile borders, alpha / beta, bit-identical repeats."""
    import flagsparse_b200._plan as plan_mod
    from flagsparse_b200 import clear_plan_cache, flagsparse_spmv_csr
    monkeypatch.setattr(plan_mod, "PANEL_TRIGGER_BYTES", 0)
    monkeypatch.setattr(plan_mod, "PANEL_TARGET_BYTES", 2048 * np.dtype(dtype).itemsize)
    monkeypatch.setattr(plan_mod, "PANEL_MIN_NNZ", 0)
    monkeypatch.setattr(plan_mod, "LONG_SPMV_SLICE_COLS", slice_cols)
    monkeypatch.setattr(plan_mod, "LONG_SPMV_MIN_PER_PANEL", 2.0)
    monkeypatch.setattr(plan_mod, "LONG_SPMV_TILES_PER_UNIT", 2)
    clear_plan_cache()
    rng = np.random.default_rng(slice_cols)
    lengths = np.concatenate([[0, 1, 5000, 0, 33, 256, 512, 1024], rng.integers(0, 12, 3000),
                              [2500, 0, 9000, 3]])
    n_rows, n_cols = lengths.size, 6000
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype, sort=False)
    x = random_values(rng, n_cols, dtype)
    y0 = random_values(rng, n_rows, dtype)
    alpha, beta = (1.5, 0.5) if np.dtype(dtype).kind != "c" else (1.5 - 0.25j, 0.5 + 2j)
    expect = oracle.spmv(data, idx, ptr, x, (n_rows, n_cols), alpha=alpha, beta=beta, y0=y0)
    args = (dev(data), dev(idx, idx_dtype), dev(ptr, idx_dtype), dev(x), (n_rows, n_cols))
    out = dev(y0)
    y = flagsparse_spmv_csr(*args, out=out, alpha=alpha, beta=beta)
    plan = plan_mod.cache_get(plan_mod.plan_key("spmv", args[0], args[1], args[2], args[4]))
    lay = plan.panels()
    assert lay is not None and lay.long_rows is not None
    assert 3 <= lay.long_rows.n_long <= 8 and lay.long_rows.n_units > 1
    assert_parity(host(y), expect, dtype)
    out2 = dev(y0)
    flagsparse_spmv_csr(*args, out=out2, alpha=alpha, beta=beta)
    assert torch.equal(out.view(torch.uint8), out2.view(torch.uint8))
    clear_plan_cache()


@pytest.mark.parametrize("dtype", DTYPES, ids=lambda d: np.dtype(d).name)
def test_spmv_stack_launched_panel_by_panel_equals_one_launch(monkeypatch, dtype):
    """Several GPUs receive x one column panel at a time and launch the wide-panel kernel once
    per panel (b2s_spmv_stack_tiles), each launch behind the arrival of its slice.  Here the
    arrival hook only records its calls: the partial sums must equal those of the single launch
    bit for bit, panels must be asked for in ascending order and all of x at the end."""
    import flagsparse_b200._plan as plan_mod
    from flagsparse_b200 import clear_plan_cache, prepare_spmv_csr
    from flagsparse_b200.spmv import _launch_stack_partials, _spmv_launch_record
    monkeypatch.setattr(plan_mod, "PANEL_TRIGGER_BYTES", 0)
    monkeypatch.setattr(plan_mod, "PANEL_TARGET_BYTES", 1024 * np.dtype(dtype).itemsize)
    monkeypatch.setattr(plan_mod, "PANEL_MIN_NNZ", 0)
    clear_plan_cache()
    rng = np.random.default_rng(77)
    lengths = np.concatenate([rng.integers(0, 40, 2500), [3000, 0, 1]])
    n_rows, n_cols = lengths.size, 5000
    data, idx, ptr = csr_from_lengths(rng, lengths, n_cols, dtype, sort=False)
    d, i, p = dev(data), dev(idx, torch.int64), dev(ptr, torch.int64)
    x = dev(random_values(rng, n_cols, dtype))
    plan = prepare_spmv_csr(d, i, p, (n_rows, n_cols)).plan()
    rec = _spmv_launch_record(plan)
    assert rec[0] == "stack"
    lay = rec[1]
    assert lay.n_panels >= 4
    bounds = lay.panel_tile_bounds()
    assert len(bounds) == lay.n_panels and bounds[-1] == lay.n_tiles
    assert all(a <= b for a, b in zip(bounds, bounds[1:]))
    stream = torch.cuda.current_stream().cuda_stream
    whole = _launch_stack_partials(plan, lay, x, stream).clone()
    asked = []
    piecewise = _launch_stack_partials(plan, lay, x, stream, x_ready=asked.append)
    torch.cuda.synchronize()
    assert asked == list(range(lay.n_panels)) + [None]
    assert torch.equal(whole.view(torch.uint8), piecewise.view(torch.uint8))
    # ranges the C entry point refuses
    lib = _lib_mod().load()
    L = _lib_mod()
    carry = plan.scratch_on("spmv_stack_carry", lay.n_tiles, stream)
    st = lib.b2s_spmv_stack_tiles(
        plan.vcode, L.ptr(lay.vals), L.ptr(lay.cols), lay.n_entries, lay.n_stacked, plan.n_cols,
        lay.n_panels, lay.shift, L.ptr(lay.panel_start), L.ptr(lay.tile_panel),
        L.ptr(lay.tile_ord), L.ptr(x), L.ptr(whole), L.ptr(carry), L.ptr(plan.status),
        lay.n_tiles - 1, 2, 1, stream)
    assert st == 2   # B2S_ERR_ARG: the range runs past the last tile
    clear_plan_cache()


def test_spmv_and_spmm_accept_inference_mode_tensors():
    """Tensors made under torch.inference_mode() have no version counter; the plan cache must
    not trip over that (the reference works there)."""
    from flagsparse_b200 import clear_plan_cache, flagsparse_spmm_csr, flagsparse_spmv_csr
    rng = np.random.default_rng(5)
    lengths = rng.integers(0, 9, 300)
    data, idx, ptr = csr_from_lengths(rng, lengths, 200, np.float32)
    x = random_values(rng, 200, np.float32)
    B = random_values(rng, 200 * 8, np.float32).reshape(200, 8)
    with torch.inference_mode():
        d, i, p, xd, Bd = dev(data), dev(idx, torch.int32), dev(ptr, torch.int32), dev(x), dev(B)
        y = flagsparse_spmv_csr(d, i, p, xd, (300, 200))
        C = flagsparse_spmm_csr(d, i, p, Bd, (300, 200))
        y_again = flagsparse_spmv_csr(d, i, p, xd, (300, 200))
    assert_parity(host(y), oracle.spmv(data, idx, ptr, x, (300, 200)), np.float32)
    assert_parity(host(C), oracle.spmm(data, idx, ptr, B, (300, 200)), np.float32)
    assert torch.equal(y, y_again)
    clear_plan_cache()


def test_prepared_handle_follows_in_place_value_updates_on_the_panel_layout(monkeypatch):
    """A prepared handle keeps the caller's data tensor, as the reference's does
    (spmv_csr.py:55-79): values changed in place afterwards are the ones multiplied, also when
    the kernels read a re-laid-out private copy of the matrix."""
    import flagsparse_b200._plan as plan_mod
    from flagsparse_b200 import clear_plan_cache, flagsparse_spmv_csr, prepare_spmv_csr
    monkeypatch.setattr(plan_mod, "PANEL_TRIGGER_BYTES", 0)
    monkeypatch.setattr(plan_mod, "PANEL_TARGET_BYTES", 512 * 8)
    monkeypatch.setattr(plan_mod, "PANEL_MIN_NNZ", 0)
    clear_plan_cache()
    rng = np.random.default_rng(9)
    lengths = rng.integers(0, 20, 2000)
    data, idx, ptr = csr_from_lengths(rng, lengths, 4000, np.float64)
    x = random_values(rng, 4000, np.float64)
    d, i, p = dev(data), dev(idx, torch.int64), dev(ptr, torch.int64)
    prepared = prepare_spmv_csr(d, i, p, (2000, 4000))
    y1 = flagsparse_spmv_csr(x=dev(x), prepared=prepared)
    assert prepared.plan().panels() is not None
    assert_parity(host(y1), oracle.spmv(data, idx, ptr, x, (2000, 4000)), np.float64)
    d.mul_(-3.0)
    y2 = flagsparse_spmv_csr(x=dev(x), prepared=prepared)
    assert_parity(host(y2), oracle.spmv(-3.0 * data, idx, ptr, x, (2000, 4000)), np.float64)
    clear_plan_cache()


def test_plan_cache_is_bounded_by_bytes():
    import flagsparse_b200._plan as plan_mod
    from flagsparse_b200 import (clear_plan_cache, flagsparse_spmv_csr, set_plan_cache_bytes)
    clear_plan_cache()
    rng = np.random.default_rng(3)
    try:
        set_plan_cache_bytes(1)          # nothing but the newest plan fits
        for k in range(3):
            data, idx, ptr = csr_from_lengths(rng, rng.integers(1, 9, 500), 300, np.float32)
            flagsparse_spmv_csr(dev(data), dev(idx, torch.int32), dev(ptr, torch.int32),
                                dev(random_values(rng, 300, np.float32)), (500, 300))
            assert len(plan_mod._CACHE) == 1
    finally:
        set_plan_cache_bytes(None)
        clear_plan_cache()


def test_spmv_coo_front_door_and_public_transpose():
    """flagsparse_spmv_coo_tocsr (spmv_csr.py:988-1057): unsorted COO with duplicates, the
    prepared form, and csr_to_csc against the oracle's stable transpose."""
    from flagsparse_b200 import (csr_to_csc, flagsparse_spmv_coo_tocsr, prepare_spmv_coo_tocsr)
    rng = np.random.default_rng(77)
    n_rows, n_cols, nnz = 500, 300, 6000
    row = rng.integers(0, n_rows, nnz)
    col = rng.integers(0, n_cols, nnz)
    for dtype in (np.float32, np.float64, np.complex64):
        data = random_values(rng, nnz, dtype)
        x = random_values(rng, n_cols, dtype)
        order = np.lexsort((col, row))
        ptr = np.zeros(n_rows + 1, dtype=np.int64)
        np.cumsum(np.bincount(row, minlength=n_rows), out=ptr[1:])
        # sums inside a row may be reordered by the unstable sort: compare within tolerance
        expect = oracle.spmv(data[order], col[order], ptr, x, (n_rows, n_cols))
        y = flagsparse_spmv_coo_tocsr(dev(data), dev(row), dev(col), dev(x), (n_rows, n_cols))
        assert_parity(host(y), expect, dtype)
        prep = prepare_spmv_coo_tocsr(dev(data), dev(row), dev(col), (n_rows, n_cols))
        y2 = flagsparse_spmv_coo_tocsr(x=dev(x), prepared=prep)
        assert_parity(host(y2), expect, dtype)
        with pytest.raises(ValueError, match="does not match prepared.shape"):
            flagsparse_spmv_coo_tocsr(x=dev(x), prepared=prep, shape=(n_rows, n_cols + 1))
        t_data, t_idx, t_ptr, t_shape = csr_to_csc(dev(data[order]), dev(col[order]), dev(ptr),
                                                   (n_rows, n_cols), conj=True)
        e_data, e_idx, e_ptr, e_shape = oracle.transpose_csr(data[order], col[order], ptr,
                                                             (n_rows, n_cols), conj=True)
        assert t_shape == e_shape
        assert np.array_equal(host(t_ptr), e_ptr) and np.array_equal(host(t_idx), e_idx)
        assert np.array_equal(host(t_data).view(np.uint8), e_data.view(np.uint8))
    with pytest.raises(TypeError, match="x dtype must match data dtype"):
        flagsparse_spmv_coo_tocsr(dev(data), dev(row), dev(col), dev(x).to(torch.complex128),
                                  (n_rows, n_cols))


def test_spmv_calls_can_be_captured_in_a_cuda_graph():
    """More captured launches than the period of the scheduled status read: inside a capture the
    read (a copy to the host and an event query) is skipped, so the capture stays valid; the
    replayed products equal the eager one bit for bit."""
    from flagsparse_b200 import clear_plan_cache, flagsparse_spmv_csr
    from flagsparse_b200._plan import CsrPlan
    rng = np.random.default_rng(11)
    lengths = rng.integers(0, 30, 4000)
    data, idx, ptr = csr_from_lengths(rng, lengths, 3000, np.float32)
    d, i, p = dev(data), dev(idx, torch.int32), dev(ptr, torch.int32)
    x = dev(random_values(rng, 3000, np.float32))
    out = torch.empty(4000, dtype=torch.float32, device="cuda")
    eager = flagsparse_spmv_csr(d, i, p, x, (4000, 3000)).clone()
    n_calls = 3 * CsrPlan.STATUS_EVERY + 5
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        flagsparse_spmv_csr(d, i, p, x, (4000, 3000), out=out)   # scratch of this stream exists
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(n_calls):
                flagsparse_spmv_csr(d, i, p, x, (4000, 3000), out=out)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    assert torch.equal(flagsparse_spmv_csr(d, i, p, x, (4000, 3000)), eager)   # eager again
    clear_plan_cache()
