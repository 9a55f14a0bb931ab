"""Install the unmodified FlagSparse package, and the accuracy suites of its own test tree that
cover CSR SpMV / SpMM and the COO -> CSR front door, under baseline/_ref (git-ignored; never
committed).

    python baseline/install_reference.py <path of a FlagSparse checkout>

The package goes in with pip from the local wheelhouse (no index, no dependency resolution); the
test files are copied byte for byte into baseline/_ref/tests/pytest/ so that
tests/test_reference_suites_gpu.py can run them, unmodified, against this repository's kernels
on a machine that has no checkout.  Nothing in the product imports anything from baseline/_ref.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

DEST = Path(__file__).resolve().parent / "_ref"

# tests/pytest/ of the checkout: the two suites and what they import
SUITE_FILES = ("__init__.py", "conftest.py", "accuracy_utils.py", "param_shapes.py",
               "test_spmv_csr_accuracy.py", "test_spmm_csr_accuracy.py",
               "test_spmv_coo_accuracy.py")


def install_package(checkout: Path) -> None:
    if (DEST / "flagsparse").is_dir():
        return
    with tempfile.TemporaryDirectory() as tmp:           # the build writes into its source tree
        src = Path(tmp) / "flagsparse_src"
        shutil.copytree(checkout, src, ignore=shutil.ignore_patterns(".git"))
        subprocess.run([sys.executable, "-m", "pip", "install", "--no-index",
                        "--no-build-isolation", "--no-deps", "--find-links", "/opt/wheelhouse",
                        "--target", str(DEST), str(src)], check=True)


def stage_suites(checkout: Path) -> None:
    out = DEST / "tests" / "pytest"
    out.mkdir(parents=True, exist_ok=True)
    (DEST / "tests" / "__init__.py").write_bytes((checkout / "tests" / "__init__.py").read_bytes()
                                                 if (checkout / "tests" / "__init__.py").exists()
                                                 else b"")
    for name in SUITE_FILES:
        shutil.copyfile(checkout / "tests" / "pytest" / name, out / name)


def main(argv) -> int:
    if len(argv) != 2:
        print(__doc__)
        return 2
    checkout = Path(argv[1]).resolve()
    install_package(checkout)
    stage_suites(checkout)
    print(f"reference package and suites are under {DEST}")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
