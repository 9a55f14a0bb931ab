"""FlagSparse's own CSR SpMV / SpMM accuracy suites, byte for byte as FlagSparse ships them
(tests/pytest/test_spmv_csr_accuracy.py, tests/pytest/test_spmm_csr_accuracy.py), run against
this repository's kernels.

The suites import ``flagsparse`` and reach into ``flagsparse.sparse_operations.spmv_csr`` by
name; a child pytest process loads the plugin ``flagsparse_b200._install_plugin`` first, which
calls ``install(replace_modules=True)``, so every name the suites touch resolves to this
package.  The suites and the unmodified package come from baseline/_ref, which
baseline/install_reference.py fills from a FlagSparse checkout; without it the tests skip.

Selection is by the suites' own markers: ``spmv_csr``, ``spmm_csr`` and ``spmv_coo_tocsr``.  The cases marked
``spmm_csr_opt`` exercise FlagSparse's separate "opt" entry points, which install() leaves alone.
"""

from __future__ import annotations

import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REF = os.path.join(_ROOT, "baseline", "_ref")


def _run_suite(file_name, marker):
    suite = os.path.join(_REF, "tests", "pytest", file_name)
    if not (os.path.isfile(suite) and os.path.isdir(os.path.join(_REF, "flagsparse"))):
        pytest.skip("FlagSparse package / suites not installed under baseline/_ref")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([_REF, _ROOT])
    proc = subprocess.run(
        [sys.executable, "-m", "pytest", "-p", "flagsparse_b200._install_plugin",
         "-p", "no:cacheprovider", "-q", "-m", marker, "--rootdir", _REF,
         "-W", "ignore::pytest.PytestUnknownMarkWarning", suite],
        cwd=_REF, env=env, capture_output=True, text=True, timeout=1500)
    tail = proc.stdout[-4000:] + proc.stderr[-2000:]
    assert proc.returncode == 0, tail
    summary = re.search(r"(\d+) passed", proc.stdout)
    assert summary is not None, tail
    return int(summary.group(1)), tail


def test_flagsparse_spmv_csr_accuracy_suite_passes_unmodified():
    # 3 shapes x 4 value types x 2 index types x 3 ops, and 5 behaviour cases (prepared-handle
    # mismatches, the int64 -> int32 retry under 'auto', no retry under 'strict', no retry when
    # an index does not fit int32)
    passed, tail = _run_suite("test_spmv_csr_accuracy.py", "spmv_csr")
    assert passed == 3 * 4 * 2 * 3 + 5, tail


def test_flagsparse_spmm_csr_accuracy_suite_passes_unmodified():
    # 2 shapes x 4 value types, 2 shapes x 4 value types x 2 index types x 3 ops, and 3
    # behaviour cases (timing meta of the transpose path, of the plain path, argument errors)
    passed, tail = _run_suite("test_spmm_csr_accuracy.py", "spmm_csr")
    assert passed == 2 * 4 + 2 * 4 * 2 * 3 + 3, tail


def test_flagsparse_coo_tocsr_cases_of_the_coo_suite_pass_unmodified():
    # the COO -> CSR front door (flagsparse_spmv_coo_tocsr / prepare_spmv_coo_tocsr), which feeds
    # the CSR kernels: 3 shapes x 2 value types against torch, and the prepared path.  The
    # suite's other cases exercise FlagSparse's COO kernels, which install() leaves alone.
    passed, tail = _run_suite("test_spmv_coo_accuracy.py", "spmv_coo_tocsr")
    assert passed == 3 * 2 + 1, tail
