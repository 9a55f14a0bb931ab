"""B200-native CSR SpMV / SpMM behind FlagSparse's Python signatures.

    from flagsparse_b200 import flagsparse_spmv_csr, flagsparse_spmm_csr

The two functions accept what ``flagsparse.flagsparse_spmv_csr`` / ``flagsparse_spmm_csr``
accept (plus trailing ``alpha`` / ``beta``) and run hand-written sm_100a kernels from
``libb200sparse.so`` (C ABI: ``include/b200sparse.h``).  ``install()`` rebinds the names inside an
importable ``flagsparse`` package so existing code picks the B200 path up unchanged.
"""

from __future__ import annotations

from ._contract import (
    SUPPORTED_INDEX_DTYPES,
    SUPPORTED_VALUE_DTYPES,
)
from ._plan import (
    clear_plan_cache,
    set_long_row_policy,
    set_long_spmv_policy,
    set_panel_policy,
    set_plan_cache_bytes,
    set_plan_cache_capacity,
    set_window_policy,
)
from .spmm import (
    SPMM_OP_CONJ_TRANS,
    SPMM_OP_NON,
    SPMM_OP_TRANS,
    flagsparse_spmm_csr,
    spmm_csr,
)
from .spmm_route import (
    PreparedCsrSpmmRoute,
    SpmmCsrAlgorithmUnavailable,
    flagsparse_spmm_csr_run,
    list_spmm_csr_algorithms,
    prepare_spmm_csr_route,
    resolve_spmm_csr_algorithm,
)
from .spmv import (
    SPMV_OP_CONJ_TRANS,
    SPMV_OP_NON,
    SPMV_OP_TRANS,
    PreparedCsrSpmv,
    coo_to_csr_for_spmv,
    csr_to_csc,
    flagsparse_spmv_coo_tocsr,
    flagsparse_spmv_csr,
    prepare_spmv_coo_tocsr,
    prepare_spmv_csr,
    spmv_csr,
)

__version__ = "0.1.0"

__all__ = [
    "flagsparse_spmv_csr",
    "flagsparse_spmm_csr",
    "prepare_spmv_csr",
    "PreparedCsrSpmv",
    "spmv_csr",
    "spmm_csr",
    "prepare_spmm_csr_route",
    "flagsparse_spmm_csr_run",
    "PreparedCsrSpmmRoute",
    "SpmmCsrAlgorithmUnavailable",
    "list_spmm_csr_algorithms",
    "resolve_spmm_csr_algorithm",
    "flagsparse_spmv_coo_tocsr",
    "prepare_spmv_coo_tocsr",
    "coo_to_csr_for_spmv",
    "csr_to_csc",
    "install",
    "clear_plan_cache",
    "set_plan_cache_capacity",
    "set_plan_cache_bytes",
    "set_panel_policy",
    "set_long_row_policy",
    "set_long_spmv_policy",
    "set_window_policy",
    "SUPPORTED_VALUE_DTYPES",
    "SUPPORTED_INDEX_DTYPES",
    "SPMV_OP_NON", "SPMV_OP_TRANS", "SPMV_OP_CONJ_TRANS",
    "SPMM_OP_NON", "SPMM_OP_TRANS", "SPMM_OP_CONJ_TRANS",
]

_PATCHED_NAMES = ("flagsparse_spmv_csr", "flagsparse_spmm_csr", "prepare_spmv_csr",
                  "PreparedCsrSpmv", "prepare_spmm_csr_route", "flagsparse_spmm_csr_run",
                  "PreparedCsrSpmmRoute", "flagsparse_spmv_coo_tocsr", "prepare_spmv_coo_tocsr")


def install(flagsparse_module=None, replace_modules=False):
    """Rebind FlagSparse's CSR SpMV / SpMM entry points to this package.

    replace_modules=True additionally registers this package's ``spmv`` / ``spmm`` modules as
    ``flagsparse.sparse_operations.spmv_csr`` / ``.spmm_csr`` (in ``sys.modules`` and as
    attributes of the subpackage), so that code which reaches into those modules by name --
    FlagSparse's own accuracy tests patch ``_triton_spmv_csr_impl_prepared`` and
    ``_run_spmv_prepared`` there (tests/pytest/test_spmv_csr_accuracy.py:152-234) -- acts on
    this implementation.

    FlagSparse resolves its public names lazily from ``flagsparse.sparse_operations``
    (src/flagsparse/__init__.py:247-254) and imports them eagerly into that subpackage
    (sparse_operations/__init__.py:36-72); there is no plugin registry.  This function sets
    the names of ``_PATCHED_NAMES`` on ``flagsparse``, ``flagsparse.sparse_operations`` and the
    ``spmv_csr`` / ``spmm_csr`` submodules.  Returns a dict of the objects it replaced (pass it to
    ``uninstall``).
    """
    import importlib
    import sys

    if flagsparse_module is None:
        flagsparse_module = importlib.import_module("flagsparse")
    here = sys.modules[__name__]
    targets = [flagsparse_module]
    for sub in ("sparse_operations", "sparse_operations.spmv_csr", "sparse_operations.spmm_csr"):
        try:
            targets.append(importlib.import_module(f"{flagsparse_module.__name__}.{sub}"))
        except ImportError:
            pass
    replaced = {}
    for mod in targets:
        for name in _PATCHED_NAMES:
            if name in vars(mod) or mod is flagsparse_module:
                replaced[(mod.__name__, name)] = vars(mod).get(name)
                setattr(mod, name, getattr(here, name))
    if replace_modules:
        ops_name = f"{flagsparse_module.__name__}.sparse_operations"
        ops = sys.modules.get(ops_name)
        for sub, ours in (("spmv_csr", "spmv"), ("spmm_csr", "spmm")):
            mine = importlib.import_module(f"{__name__}.{ours}")
            replaced[("sys.modules", f"{ops_name}.{sub}")] = sys.modules.get(f"{ops_name}.{sub}")
            sys.modules[f"{ops_name}.{sub}"] = mine
            if ops is not None:
                replaced[(ops_name, sub)] = vars(ops).get(sub)
                setattr(ops, sub, mine)
    return replaced


def uninstall(replaced):
    """Undo ``install`` with the dict it returned."""
    import sys

    for (mod_name, name), old in replaced.items():
        if mod_name == "sys.modules":
            if old is None:
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = old
            continue
        mod = sys.modules.get(mod_name)
        if mod is None:
            continue
        if old is None:
            if name in vars(mod):
                delattr(mod, name)
        else:
            setattr(mod, name, old)
