"""float16 / bfloat16 values.

FlagSparse lists both among its value dtypes (_common.py:21-29) and computes them in float32:
its launchers widen the matrix values (cached per prepared handle) and the dense operand, run the
float32 kernel and round the result once (spmv_csr.py:124-129 and :679-704,
spmm_csr.py:2716-2719).  This package does the same around its float32 kernels: the widened copy
of a matrix's values is made once and found again by the identity of the caller's tensor, the
dense operand is widened per call, the result is rounded to the caller's dtype.  The value stream
the kernels read is therefore float32; kernels that read 16-bit values directly are not built.
"""

from __future__ import annotations

from collections import OrderedDict

import torch

HALF_VALUE_DTYPES = (torch.float16, torch.bfloat16)
_WIDE = OrderedDict()   # identity of the caller's tensor -> (float32 copy, the caller's tensor)
_WIDE_CAPACITY = 8


def is_half(t):
    return torch.is_tensor(t) and t.dtype in HALF_VALUE_DTYPES


def widened_values(data):
    """float32 copy of a float16 / bfloat16 value array, made once per tensor (and per in-place
    modification of it).  The entry keeps the caller's tensor alive, so its address cannot be
    reused by another tensor while the entry exists."""
    from ._plan import tensor_version
    key = (data.data_ptr(), data.numel(), data.dtype, tensor_version(data), str(data.device),
           tuple(data.stride()))
    hit = _WIDE.get(key)
    if hit is not None:
        _WIDE.move_to_end(key)
        return hit[0]
    wide = data.to(torch.float32)
    _WIDE[key] = (wide, data)
    while len(_WIDE) > _WIDE_CAPACITY:
        _WIDE.popitem(last=False)
    return wide


def clear_widened():
    _WIDE.clear()


def narrow_result(result, dtype, out):
    """Round a float32 result to `dtype`; with `out` (the caller's 16-bit tensor) the rounded
    values are written there and `out` itself is returned."""
    if out is not None:
        out.copy_(result)
        return out
    return result.to(dtype)
