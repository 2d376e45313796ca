"""Shared pytest configuration: the ``gpu`` marker and golden-fixture helpers."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

GOLDEN_DIR = os.path.join(REPO, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "slow: long-running case")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, not failed, where no CUDA device exists."""
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str) -> dict:
    """Load ``tests/golden/<name>.npz`` as torch tensors; quant tuples decoded."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {}
    for k in z.files:
        a = z[k]
        if k in ("q_in", "q_out"):
            d[k] = None if a.size == 0 else (float(a[0]), int(a[1]), int(a[2]))
        else:
            d[k] = torch.from_numpy(np.array(a))
    return d


SCAN_GOLDEN = {
    "dense": ["scan_dense_fp32", "scan_dense_q8", "scan_dense_q8_asym"],
    "diagonal": ["scan_diagonal_fp32", "scan_diagonal_q8"],
    "monarch": ["scan_monarch_fp32", "scan_monarch_q8"],
    "butterfly": ["scan_butterfly_fp32", "scan_butterfly_q8", "scan_butterfly_nb2",
                  "scan_butterfly_pad"],
}
SCAN_GOLDEN_FLAT = [(k, n) for k, names in SCAN_GOLDEN.items() for n in names]

# Butterfly fixtures produced on a GPU by the reference's own Triton kernels
# (tests/golden/make_golden_butterfly_gpu.py): they pin the stage / stride / twiddle convention.
BUTTERFLY_REFERENCE_GOLDEN = ["ref_butterfly_h16", "ref_butterfly_h8_nb2", "ref_butterfly_h12_pad",
                              "ref_butterfly_h32_nb2", "ref_butterfly_h16_q8"]


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max(1e-30, max|b|) -- the reference tests' 'relative' measure."""
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp(min=1e-30))
