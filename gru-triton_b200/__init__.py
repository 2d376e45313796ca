"""B200-native persistent GRU scan behind the ``gru_qat`` Python API.

Public names mirror ``gru_qat`` (src/gru_qat/__init__.py:21-36).  The scan
modules (``scan``, ``scan_diagonal``, ``scan_monarch``, ``scan_butterfly``) call a
C-ABI CUDA library built for sm_100a; :func:`install_as_gru_qat` makes the package
importable under the reference's module paths for literal drop-in use.
"""

from __future__ import annotations

import sys

from .gru_cell import GRUCellQuant
from .gru_layer import GRULayer
from .quantizers import (PRESETS, FakeQuantize, FakeQuantizePerChannel, FakeQuantizePerGroup,
                         FakeQuantizePerTensor, Identity, QuantizerConfig, QuantRecipe)
from .ste import STEClamp, STERound
from .structure import StructureConfig, make_structured_linear

__all__ = [
    "GRUCellQuant", "GRULayer", "FakeQuantize", "FakeQuantizePerTensor", "FakeQuantizePerChannel",
    "FakeQuantizePerGroup", "Identity", "QuantizerConfig", "QuantRecipe", "PRESETS", "STERound",
    "STEClamp", "StructureConfig", "make_structured_linear", "install_as_gru_qat",
]

__version__ = "0.1.0"


def install_as_gru_qat() -> None:
    """Register this package in ``sys.modules`` as ``gru_qat`` (and its scan modules as
    ``gru_qat.triton_kernels.*``) so code written against the reference imports it unchanged.
    Refuses if a different ``gru_qat`` is already imported."""
    import importlib
    import types

    me = sys.modules[__name__]
    if "gru_qat" in sys.modules and sys.modules["gru_qat"] is not me:
        raise RuntimeError("a different gru_qat is already imported")
    sys.modules["gru_qat"] = me
    for sub in ("gru_cell", "gru_layer", "quantizers", "ste", "structure", "calibration"):
        sys.modules[f"gru_qat.{sub}"] = importlib.import_module(f"{__name__}.{sub}")
    tk = types.ModuleType("gru_qat.triton_kernels")
    tk.is_available = lambda: True
    sys.modules["gru_qat.triton_kernels"] = tk
    for sub in ("scan", "scan_diagonal", "scan_monarch", "scan_butterfly"):
        mod = importlib.import_module(f"{__name__}.{sub}")
        sys.modules[f"gru_qat.triton_kernels.{sub}"] = mod
        setattr(tk, sub, mod)
    me.triton_kernels = tk
