"""Import shim: the package directory is ``gru-triton_b200/`` (not a valid Python
identifier), so ``import gru_triton_b200`` loads this file, which loads that
directory as the package ``gru_triton_b200`` and takes its place in ``sys.modules``."""

import importlib.util
import os
import sys

_pkg_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gru-triton_b200")
_spec = importlib.util.spec_from_file_location(
    "gru_triton_b200", os.path.join(_pkg_dir, "__init__.py"), submodule_search_locations=[_pkg_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["gru_triton_b200"] = _mod
_spec.loader.exec_module(_mod)
