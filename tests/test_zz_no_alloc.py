"""The allocation-free diagonal backward (``b200gru_diagonal_backward_noalloc``).

Some users of the library are not allowed to allocate GPU memory -- for instance a
plugin living inside another runtime's memory budget.  This entry point keeps its
scratch in a buffer built into the library.  The test drives it straight through the
C ABI, twice in a row with different shapes (the second call finds the first call's
leftovers in the shared buffer), and compares each result with the ordinary
workspace-taking entry point.  Collected last on purpose: if it fails under ``-x``
every other test has already run.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from conftest import rel_err
from oracle import gru_scan_oracle as orc

pytestmark = pytest.mark.gpu

GRAD_TOL = 1e-4


def _run_pair(T, B, H, seed, quant, first_call_on_device=False):
    from gru_triton_b200 import _lib
    from gru_triton_b200.scan_diagonal import (gru_scan_diagonal_backward_triton,
                                               gru_scan_diagonal_forward_triton)
    lib = _lib.load()
    gi, h0, W, bh, dout = [t.cuda() for t in orc.make_problem("diagonal", T, B, H, seed=seed)]
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    out = gru_scan_diagonal_forward_triton(gi, h0, W, bh, **kw)
    ref = gru_scan_diagonal_backward_triton(gi, h0, W, bh, out, dout, **kw)

    # outputs are pre-filled with NaN so that any element the call fails to write shows up
    dgi = torch.full_like(gi, float("nan"))
    dh0 = torch.full_like(h0, float("nan"))
    dW = torch.full_like(W, float("nan"))
    dbh = torch.full_like(bh, float("nan"))
    qi = _lib._cquant(quant[0] if quant else None)
    qo = _lib._cquant(quant[1] if quant else None)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]               # the driver's view: catches a raw cudaMalloc too
    rc = lib.b200gru_diagonal_backward_noalloc(
        p(gi), p(h0), p(W), p(bh), p(out), p(dout), T, B, H, ctypes.byref(qi), ctypes.byref(qo),
        p(dgi), p(dh0), p(dW), p(dbh), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.b200gru_strerror(rc)
    assert torch.cuda.memory_allocated() == before          # nothing came from torch's allocator
    torch.cuda.synchronize()
    if not first_call_on_device:
        assert torch.cuda.mem_get_info()[0] >= free_before  # nor from the driver (other tenants may free)
    for name, got, want in zip(("dgi", "dh0", "dW", "dbh"), (dgi, dh0, dW, dbh), ref):
        assert not torch.isnan(got).any(), name
        assert rel_err(got, want) <= GRAD_TOL, name


def test_noalloc_backward_matches_workspace_backward_twice_in_a_row():
    q8 = ((0.02, -127, 127), (0.02, -127, 127))
    _run_pair(24, 37, 256, seed=1, quant=q8, first_call_on_device=True)       # larger first ...
    _run_pair(9, 5, 64, seed=2, quant=None)        # ... then a smaller one over its leftovers
    _run_pair(24, 37, 256, seed=3, quant=None)


def test_noalloc_backward_rejects_oversized_problems():
    from gru_triton_b200 import _lib
    lib = _lib.load()
    dummy = torch.zeros(16, device="cuda")
    p = ctypes.c_void_p(dummy.data_ptr())
    # ceil(B/4) * 6 * H * 4 bytes = 6 MiB > 4 MiB: refused before anything is launched
    n0 = lib.b200gru_launch_count()
    rc = lib.b200gru_diagonal_backward_noalloc(p, p, p, p, p, p, 1, 1024, 1024, None, None, p, p, p, p, None)
    assert rc == 5 and b"built-in" in lib.b200gru_strerror(rc)
    assert lib.b200gru_launch_count() == n0


def test_noalloc_backward_accepts_exactly_the_built_in_size():
    """H = 1024: ceil(B/4) * 6 * 1024 * 4 bytes; B = 680 fills the 4 MiB buffer to the byte (170 row
    groups of 24 KiB + ...), one more row group is refused."""
    from gru_triton_b200 import _lib
    lib = _lib.load()
    H = 1024
    groups = (4 << 20) // (6 * H * 4)                        # 170 row groups fit
    for B, want_rc in ((4 * groups, 0), (4 * groups + 1, 5)):
        gi, h0, W, bh, dout = [t.cuda() for t in orc.make_problem("diagonal", 2, B, H, seed=4)]
        out = torch.zeros(2, B, H, device="cuda")
        dgi, dh0, dW, dbh = torch.empty_like(gi), torch.empty_like(h0), torch.empty_like(W), torch.empty_like(bh)
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        rc = lib.b200gru_diagonal_backward_noalloc(
            p(gi), p(h0), p(W), p(bh), p(out), p(dout), 2, B, H, None, None, p(dgi), p(dh0), p(dW), p(dbh),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == want_rc, (B, rc)
    torch.cuda.synchronize()
