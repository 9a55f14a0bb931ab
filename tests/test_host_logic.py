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


def test_widened_half_values_are_made_once_per_tensor_state():
    from flagsparse_b200 import _half
    _half.clear_widened()
    d = torch.arange(8, dtype=torch.float32).to(torch.bfloat16)
    w1 = _half.widened_values(d)
    assert w1.dtype == torch.float32 and torch.equal(w1, d.float())
    assert _half.widened_values(d) is w1                 # same tensor, same version: cached
    d.mul_(2)                                            # in-place change bumps the version
    w2 = _half.widened_values(d)
    assert w2 is not w1 and torch.equal(w2, d.float())
    h = torch.ones(8, dtype=torch.float16)
    assert _half.widened_values(h).dtype == torch.float32
    assert _half.is_half(h) and not _half.is_half(w2) and not _half.is_half(None)
    for k in range(20):                                  # bounded: old entries fall out
        _half.widened_values(torch.full((4,), float(k), dtype=torch.float16))
    assert len(_half._WIDE) <= _half._WIDE_CAPACITY
    out = torch.zeros(8, dtype=torch.float16)
    r = torch.arange(8, dtype=torch.float32)
    assert _half.narrow_result(r, torch.float16, out) is out and torch.equal(out.float(), r)
    assert _half.narrow_result(r, torch.bfloat16, None).dtype == torch.bfloat16
    _half.clear_widened()
