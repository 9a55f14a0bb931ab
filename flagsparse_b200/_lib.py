"""ctypes binding of libb200sparse.so (declarations: include/b200sparse.h).

There is no fallback: if the library is missing or a call returns a non-zero status, a
RuntimeError is raised.  Build it with ``python -m flagsparse_b200._build``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_void_p
from pathlib import Path

import torch

# B200SPARSE_CHECKED=1 selects the bounds-checked build of the same sources (see _build.py)
CHECKED = os.environ.get("B200SPARSE_CHECKED", "") not in ("", "0")
LIB_PATH = Path(__file__).resolve().parent / (
    "libb200sparse_checked.so" if CHECKED else "libb200sparse.so")

# dtype codes of include/b200sparse.h
B2S_F32, B2S_F64, B2S_C64, B2S_C128, B2S_F16, B2S_BF16 = 0, 1, 2, 3, 4, 5
B2S_I32, B2S_I64 = 0, 1
B2S_ERR_TIMEOUT = 5
B2S_ERR_BOUNDS = 9

VALUE_CODE = {
    torch.float32: B2S_F32,
    torch.float64: B2S_F64,
    torch.complex64: B2S_C64,
    torch.complex128: B2S_C128,
    torch.float16: B2S_F16,
    torch.bfloat16: B2S_BF16,
}
INDEX_CODE = {torch.int32: B2S_I32, torch.int64: B2S_I64}

# every symbol include/b200sparse.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "b2s_version": (c_int, []),
    "b2s_status_string": (c_char_p, [c_int]),
    "b2s_selftest_wait_timeout": (c_int, [c_void_p, c_int, c_void_p]),
    "b2s_csr_inspect": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_void_p,
                                c_void_p]),
    "b2s_tile_count": (c_int64, [c_int64, c_int64, c_int]),
    "b2s_tile_plan": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "b2s_spmv_tile_items": (c_int, [c_int, c_int]),
    "b2s_spmm_tile_items": (c_int, [c_int, c_int]),
    "b2s_spmm_window_tile_items": (c_int, [c_int, c_int]),
    "b2s_spmm_window_usable": (c_int, [c_int, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                       c_int64, c_int64, c_int64]),
    "b2s_spmv_csr": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                             c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p]),
    "b2s_spmv_csr_fixed_max_items": (c_int64, []),
    "b2s_spmv_csr_fixed": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                   c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p]),
    "b2s_panel_bytes": (c_int64, [c_int64, c_int64]),
    "b2s_panel_build": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_int, c_void_p, c_void_p, c_int64, c_void_p]),
    "b2s_panel_build_global": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_int, c_void_p, c_void_p, c_int64, c_void_p]),
    "b2s_spmv_stack_tile_items": (c_int, [c_int]),
    "b2s_spmv_stack_shared_cols": (c_int, [c_int]),
    "b2s_spmv_stack": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p]),
    "b2s_spmv_stack_tiles": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                     c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "b2s_spmv_stack_shared": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                      c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p]),
    "b2s_spmv_stack_rows_combine": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                            c_int64, c_void_p, c_void_p, c_void_p]),
    "b2s_panel_combine": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p]),
    "b2s_panel_combine_peers": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p,
                                        c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                        c_int, c_void_p]),
    "b2s_panel_combine_multicast": (c_int, [c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p,
                                            c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                            c_int, c_void_p]),
    "b2s_spmm_csr_colmajor_c": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                        c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p]),
    "b2s_spmm_rows_combine": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64,
                                      c_void_p, c_int64, c_void_p, c_void_p]),
    "b2s_dense_transpose": (c_int, [c_int, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                    c_void_p]),
    "b2s_peer_scatter": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int64, c_int64,
                                 c_void_p]),
    "b2s_panel_compact_bytes": (c_int64, [c_int64]),
    "b2s_panel_compact": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                  c_void_p, c_int64, c_void_p]),
    "b2s_spmm_csr": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                             c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b2s_spmm_csr_windowed": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                      c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int64, c_void_p, c_void_p]),
    "b2s_spmm_window_stat": (c_int, [c_int, c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p,
                                     c_void_p, c_void_p]),
    "b2s_csr2csc_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "b2s_csr2csc": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                            c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                            c_void_p]),
}

_lib = None


def load():
    """Return the loaded library; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built "
            "(run `python -m flagsparse_b200._build`). There is no CPU or Triton fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().b2s_status_string(int(status)).decode()
        raise RuntimeError(f"{what} failed: b2s status {status} ({msg})")


def ptr(t):
    """Device address of a tensor (None -> NULL)."""
    if t is None:
        return None
    return c_void_p(t.data_ptr())


def stream_handle(device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def scalar_buffer(value, dtype):
    """Host buffer holding one scalar of the value dtype (alpha / beta are host pointers)."""
    if dtype in (torch.float32, torch.float16, torch.bfloat16):   # 16-bit values: float32 sums
        return (ctypes.c_float * 1)(float(value))
    if dtype == torch.float64:
        return (ctypes.c_double * 1)(float(value))
    z = complex(value)
    if dtype == torch.complex64:
        return (ctypes.c_float * 2)(z.real, z.imag)
    if dtype == torch.complex128:
        return (ctypes.c_double * 2)(z.real, z.imag)
    raise TypeError(f"unsupported value dtype {dtype}")
