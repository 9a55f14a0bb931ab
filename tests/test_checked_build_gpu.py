"""The bounds-checked build of the library (-DB2S_CHECKED, libb200sparse_checked.so).

A memory checker cannot be run on every machine this library is tested on; its stand-in is a
second compile of the same sources in which every column index, row pointer, stacked-row ordinal
and work-table entry a kernel reads is range-checked before it is used as an address.  A
violation sets bit B2S_ERR_BOUNDS in the device status word and the access is skipped.  Here the
parity suites are run once more against that build (in a child process, since a process loads
one of the two libraries), and a corrupted matrix is shown to be reported instead of followed.
"""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED_LIB = os.path.join(ROOT, "flagsparse_b200", "libb200sparse_checked.so")

SUITES = ["tests/test_spmv_gpu.py", "tests/test_spmm_gpu.py", "tests/test_fuzz_gpu.py",
          "tests/test_cabi_gpu.py", "tests/test_half_gpu.py"]


def _env():
    env = dict(os.environ)
    env["B200SPARSE_CHECKED"] = "1"
    return env


def test_parity_suites_pass_on_the_bounds_checked_build():
    if not os.path.exists(CHECKED_LIB):
        from flagsparse_b200 import _build
        _build.build(checked=True)
    res = subprocess.run([sys.executable, "-m", "pytest", *SUITES, "-m", "gpu", "-x", "-q",
                          "-p", "no:cacheprovider"], cwd=ROOT, env=_env(), capture_output=True,
                         text=True, timeout=1800)
    tail = (res.stdout or "")[-2000:] + (res.stderr or "")[-1000:]
    assert res.returncode == 0, tail
    assert " passed" in res.stdout and " failed" not in res.stdout, tail


_CORRUPT = r"""
import sys, ctypes, torch
sys.path.insert(0, {root!r})
from flagsparse_b200 import _lib as L
assert L.CHECKED and L.LIB_PATH.name == "libb200sparse_checked.so"
lib = L.load()
n_rows, n_cols = 2000, 1000
g = torch.Generator(device="cuda"); g.manual_seed(1)
lens = torch.randint(0, 9, (n_rows,), device="cuda", generator=g)
ptr = torch.zeros(n_rows + 1, dtype=torch.int64, device="cuda"); ptr[1:] = torch.cumsum(lens, 0)
nnz = int(ptr[-1])
col = torch.randint(0, n_cols, (nnz,), dtype=torch.int64, device="cuda", generator=g)
col[nnz // 2] = n_cols + 12345            # a column outside x: raw C-ABI callers can pass this
val = torch.ones(nnz, dtype=torch.float64, device="cuda")
x = torch.ones(n_cols, dtype=torch.float64, device="cuda")
y = torch.zeros(n_rows, dtype=torch.float64, device="cuda")
items = lib.b2s_spmv_tile_items(L.B2S_F64, L.B2S_I64)
T = lib.b2s_tile_count(n_rows, nnz, items)
tile_row = torch.empty(T + 1, dtype=torch.int64, device="cuda")
carry = torch.empty(T, dtype=torch.float64, device="cuda")
status = torch.zeros(1, dtype=torch.int32, device="cuda")
s = L.stream_handle(val.device)
assert lib.b2s_tile_plan(L.ptr(ptr), L.B2S_I64, n_rows, nnz, items, L.ptr(tile_row), s) == 0
one, zero = (ctypes.c_double * 1)(1.0), (ctypes.c_double * 1)(0.0)
st = lib.b2s_spmv_csr(L.B2S_F64, L.B2S_I64, L.B2S_I64, L.ptr(val), L.ptr(col), L.ptr(ptr), n_rows,
                      n_cols, nnz, L.ptr(x), None, L.ptr(y), one, zero, L.ptr(tile_row),
                      L.ptr(carry), L.ptr(status), s)
assert st == 0
torch.cuda.synchronize()
bits = int(status.item())
assert bits == 1 << L.B2S_ERR_BOUNDS, bits
# every other row is still right: the bad entry was skipped, nothing else was touched
good = torch.ones(nnz, dtype=torch.float64, device="cuda"); good[nnz // 2] = 0.0
rows = torch.repeat_interleave(torch.arange(n_rows, device="cuda"), lens)
want = torch.zeros(n_rows, dtype=torch.float64, device="cuda").index_add_(0, rows, good)
assert torch.equal(y, want)
print("reported")
"""


def test_a_column_outside_x_is_reported_not_followed():
    if not os.path.exists(CHECKED_LIB):
        from flagsparse_b200 import _build
        _build.build(checked=True)
    res = subprocess.run([sys.executable, "-c", _CORRUPT.format(root=ROOT)], cwd=ROOT, env=_env(),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "reported" in res.stdout, res.stdout[-1500:] + res.stderr[-1500:]
