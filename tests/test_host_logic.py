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
