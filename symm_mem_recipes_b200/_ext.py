"""Loads the native module and refuses to run GPU paths without it.

There is no pure-PyTorch fallback for any GPU op of this package: if the
shared object is missing the import fails with the build command, so a GPU run
can never silently use another implementation.
"""
from __future__ import annotations

import importlib
import os


def _load():
    try:
        return importlib.import_module("symm_mem_recipes_b200._C")
    except ImportError as first:
        if os.environ.get("SMR_NO_AUTOBUILD") == "1":
            raise ImportError(
                "symm_mem_recipes_b200._C is not built; run "
                "`python -m symm_mem_recipes_b200._build`"
            ) from first
        # Build in tree once (needs nvcc, no GPU), then import again.
        from . import _build

        _build.build()
        importlib.invalidate_caches()
        return importlib.import_module("symm_mem_recipes_b200._C")


C = _load()
