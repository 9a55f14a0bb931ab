"""Host-side logic that needs no GPU: panel-width choice of the SpMM long-row split, its policy
switch, and the cache of widened float16 / bfloat16 value arrays."""

import pytest
import torch


def test_long_row_panel_width_and_policy():
    from flagsparse_b200 import _plan, set_long_row_policy
    saved = (_plan.LONG_ROW_POLICY, _plan.LONG_ROW_MIN, _plan.LONG_ROW_TRIGGER_BYTES,
             _plan.LONG_ROW_TARGET_BYTES, _plan.LONG_ROW_MIN_SHARE, _plan.LONG_ROW_MIN_NNZ)
    try:
        set_long_row_policy("auto")
        assert _plan.long_row_shift(1 << 20, 64) is None            # B of 64 MB: not a candidate
        assert _plan.long_row_shift(1 << 24, 256) == 17             # 2^17 rows x 256 B = 32 MB
        assert _plan.long_row_shift(1 << 26, 64) == 19
        assert _plan.long_row_shift((1 << 31) - 1, 4096) == 23      # never more than 256 panels
        assert _plan.long_row_shift(1 << 24, 0) is None
        for n_cols, row_bytes in ((1 << 22, 128), (3_000_000, 512), (1 << 28, 16)):
            shift = _plan.long_row_shift(n_cols, row_bytes)
            n_panels = ((n_cols - 1) >> shift) + 1
            assert 2 <= n_panels <= 256
            assert (1 << shift) * row_bytes <= _plan.LONG_ROW_TARGET_BYTES or n_panels == 256
        set_long_row_policy("off")
        assert _plan.long_row_shift(1 << 24, 256) is None
        set_long_row_policy("auto", min_len=64, trigger_bytes=0, target_bytes=1 << 12,
                            min_share=0.0, min_nnz=0)
        assert (_plan.LONG_ROW_MIN, _plan.LONG_ROW_MIN_NNZ) == (64, 0)
        assert _plan.long_row_shift(4096, 16) == 8                  # 256 rows x 16 B = 4 KB
        with pytest.raises(ValueError, match="'auto' or 'off'"):
            set_long_row_policy("sometimes")
    finally:
        set_long_row_policy(saved[0], *saved[1:])
    assert _plan.LONG_ROW_MIN == saved[1] and _plan.LONG_ROW_POLICY == saved[0]


def test_half_dtypes_have_value_codes_and_float32_scalars():
    """float16 / bfloat16 are value dtypes of their own at the C ABI (no widened copies): their
    codes, and alpha / beta passed as float32."""
    import ctypes

    from flagsparse_b200 import _half, _lib
    assert _lib.VALUE_CODE[torch.float16] == 4 and _lib.VALUE_CODE[torch.bfloat16] == 5
    h = torch.ones(8, dtype=torch.float16)
    assert _half.is_half(h) and not _half.is_half(h.float()) and not _half.is_half(None)
    buf = _lib.scalar_buffer(0.5, torch.bfloat16)
    assert isinstance(buf, ctypes.Array) and ctypes.sizeof(buf) == 4 and buf[0] == 0.5


def test_panel_width_follows_from_the_value_type_alone():
    """Every rank of a partitioned matrix must cut x into the same panels: the width depends on
    the value size only (largest power of two whose x slice is at most 40 MB)."""
    import torch

    from flagsparse_b200 import _plan
    assert _plan.panel_shift(torch.float64) == 22
    assert _plan.panel_shift(torch.float32) == 23
    assert _plan.panel_shift(torch.complex64) == 22
    assert _plan.panel_shift(torch.complex128) == 21


def test_panel_tile_bounds_give_a_straddling_tile_to_the_later_panel():
    """Tiles launched behind the arrival of panel p's slice of x are those that need no x beyond
    panel p; a tile that starts in one panel and ends in the next waits for the next."""
    import torch

    from flagsparse_b200._plan import StackLayout
    tile, n_tiles = 256, 4
    vals = torch.zeros(tile * n_tiles)
    cols = torch.zeros(tile * n_tiles, dtype=torch.int32)
    panel_start = torch.tensor([0, 300, 300, 1000], dtype=torch.int64)   # panel 1 is empty
    lay = StackLayout(vals, cols, 10, torch.zeros(n_tiles + 1, dtype=torch.int64),
                      torch.zeros(n_tiles, dtype=torch.int32), panel_start, 3, 4, None, tile)
    # tile 0 = entries 0..255 lies in panel 0; tile 1 = 256..511 straddles panels 0 and 2
    assert lay.panel_tile_bounds() == [1, 1, 4]
    assert lay.panel_tile_bounds() is lay.panel_tile_bounds()          # read back once


def test_algorithmic_bytes_of_the_headline_configuration():
    """The bench line's numerator: each array once at the caller's widths.  The headline
    configuration (float64 / int64, 2^24 rows and columns, 268,532,588 non-zeros, beta != 0) is
    4,833,392,328 bytes per product; SpMM N = 32 on the same matrix 13,020,673,736."""
    import sys
    from pathlib import Path

    from flagsparse_b200 import workloads as W
    n, nnz = 1 << 24, 268_532_588
    assert W.spmv_bytes(n, n, nnz, 8, 8, 8, beta_nonzero=True) == 4_833_392_328
    assert W.spmm_bytes(n, n, nnz, 32, 8, 8, 8, beta_nonzero=False) == 13_020_673_736
    assert W.sp_flops(nnz) == 2 * nnz and W.sp_flops(10, 4, complex_values=True) == 320
    # bench.problem_bytes_flops applies the same formulas to a problem object (CPU tensors)
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    p = W.cfg2_powerlaw_spmv(device="cpu", scale=4096)
    p.extra.update(alpha=p.alpha, beta=p.beta, y0=p.y0, op="non")
    nbytes, flops = bench.problem_bytes_flops(p, "spmv")
    assert nbytes == W.spmv_bytes(p.shape[0], p.shape[1], p.nnz, 8, 8, 8, beta_nonzero=True)
    assert flops == 2 * p.nnz
