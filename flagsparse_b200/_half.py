"""float16 / bfloat16 values.

FlagSparse lists both among its value dtypes (_common.py:21-29) and computes them in float32: its
launchers widen the matrix values and the dense operand, run the float32 kernel and round the
result once (spmv_csr.py:124-129 and :679-704, spmm_csr.py:2716-2719).  Here the kernels read
the 16-bit arrays themselves (value codes B2S_F16 / B2S_BF16 of the C ABI): two bytes per matrix
value and per element of x / B instead of four, float32 sums, one rounding of y / C -- also for
rows that cross tile borders, whose pieces are added in float32 before the row is rounded.
No widened copies are kept.  The column-panel layouts of SpMV and the long-row split of SpMM
are not used for these dtypes.
"""

from __future__ import annotations

import torch

from ._contract import HALF_VALUE_DTYPES


def is_half(t):
    return torch.is_tensor(t) and t.dtype in HALF_VALUE_DTYPES
