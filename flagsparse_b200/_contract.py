"""The argument contract FlagSparse's CSR SpMV / SpMM share: op codes and dtype tables.

Exception types and message texts follow the reference so that code written against
``flagsparse.sparse_operations`` sees the same errors:
op handling -- spmv_csr.py:18-52 and spmm_csr.py:11-45 (identical logic);
dtype tables -- _common.py:21-31.
"""

from __future__ import annotations

import torch

OP_NON = 0
OP_TRANS = 1
OP_CONJ_TRANS = 2
OP_NAMES = {OP_NON: "non", OP_TRANS: "trans", OP_CONJ_TRANS: "conj"}
_NAME_TO_OP = {v: k for k, v in OP_NAMES.items()}
_OP_MESSAGE = "op must be one of: 0=non, 1=trans, 2=conj"

# The value dtypes of FlagSparse (_common.py:21-29).  float16 / bfloat16 are stored as they are
# (matrix values, dense operand and result) and summed in float32 with one rounding at the end,
# the arithmetic the reference's launchers do on float32 copies (spmv_csr.py:124-129,
# spmm_csr.py:2716-2719).
HALF_VALUE_DTYPES = (torch.float16, torch.bfloat16)
SUPPORTED_VALUE_DTYPES = (torch.float32, torch.float64, torch.complex64, torch.complex128)
ALL_VALUE_DTYPES = HALF_VALUE_DTYPES + SUPPORTED_VALUE_DTYPES
SUPPORTED_INDEX_DTYPES = (torch.int32, torch.int64)
INDEX_LIMIT_INT32 = 2**31 - 1

REFERENCE_VALUE_DTYPE_NAMES = "float16, bfloat16, float32, float64, complex64, complex128"


def normalize_op(op=None, transpose=False):
    """Map op (0/1/2, 'non'/'trans'/'conj', any case, surrounding blanks) or the legacy
    ``transpose`` flag to an op code."""
    if op is None:
        return OP_TRANS if bool(transpose) else OP_NON
    if isinstance(op, str):
        code = _NAME_TO_OP.get(op.strip().lower())
        if code is None:
            raise ValueError(_OP_MESSAGE)
        return code
    try:
        code = int(op)
    except (TypeError, ValueError) as exc:
        raise ValueError(_OP_MESSAGE) from exc
    if code not in OP_NAMES:
        raise ValueError(_OP_MESSAGE)
    return code


def op_name(op):
    return OP_NAMES[normalize_op(op)]


def op_transposes(op):
    return normalize_op(op) != OP_NON


def resolve_op(op, transpose):
    """The (op, transpose) pair of the public functions -> op code, with the reference's
    conflict rule (spmv_csr.py:838-844, spmm_csr.py:3312-3322)."""
    code = normalize_op(op, transpose=False if transpose is None else bool(transpose))
    if op is not None and transpose is not None and bool(transpose) != op_transposes(code):
        raise ValueError("transpose conflicts with op")
    return code


def is_complex(dtype):
    return dtype in (torch.complex64, torch.complex128)


def check_scalar(value, dtype, name):
    """alpha / beta: a Python or 0-d tensor scalar representable in the value dtype."""
    if torch.is_tensor(value):
        if value.numel() != 1:
            raise ValueError(f"{name} must be a scalar")
        value = value.item()
    if isinstance(value, complex) and not is_complex(dtype):
        if value.imag != 0.0:
            raise TypeError(f"{name} is complex but the matrix dtype is real")
        value = value.real
    return value
