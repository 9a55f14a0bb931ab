"""pytest plugin: ``python -m pytest -p flagsparse_b200._install_plugin ...`` rebinds FlagSparse's
CSR SpMV / SpMM names to this package before any test module is imported, so that FlagSparse's
own test files run unmodified against this implementation (install(replace_modules=True))."""

import flagsparse_b200

flagsparse_b200.install(replace_modules=True)
