"""GPU parity: the CUDA scan (through the C ABI) against the CPU oracle.

Tolerances (the ones the build is held to):
  fp32 forward            |gpu - ref| <= 1e-5 + 1e-5 * |ref|            (FWD_TOL)
  fp32 gradients          max|gpu - ref| / max|ref| <= 1e-4             (GRAD_TOL)
  int8 codes of h         bit-exact, except where the oracle's h_raw / s lies within
                          TIE_WINDOW = 1e-4 code units of a half-way point; then +-1 code.
The code comparison is teacher-forced: the oracle advances ONE step from the
device's own h_{t-1}, so a rounding tie cannot cascade into later steps.  Every
quantised comparison prints its mismatch counts (inside / outside the window) and the
free-running figure: the fraction of sequences whose codes equal the oracle's own
trajectory through all T steps.
"""

from __future__ import annotations

import pytest
import torch

from conftest import BUTTERFLY_REFERENCE_GOLDEN, SCAN_GOLDEN_FLAT, load_golden, rel_err
from oracle import gru_scan_oracle as orc

pytestmark = pytest.mark.gpu

FWD_TOL = 1e-5
GRAD_TOL = 1e-4
TIE_WINDOW = 1e-4
Q8 = ((0.02, -127, 127), (0.02, -127, 127))
Q8_ASYM = ((0.02, -127, 127), (0.013, -127, 127))


def _mods():
    from gru_triton_b200 import scan, scan_butterfly, scan_diagonal, scan_monarch
    return {
        "dense": (scan.gru_scan_forward_persistent, scan.gru_scan_backward_persistent, scan.gru_scan_persistent),
        "diagonal": (scan_diagonal.gru_scan_diagonal_forward_triton,
                     scan_diagonal.gru_scan_diagonal_backward_triton, scan_diagonal.gru_scan_diagonal),
        "monarch": (scan_monarch.gru_scan_monarch_forward_triton,
                    scan_monarch.gru_scan_monarch_backward_triton, scan_monarch.gru_scan_monarch),
        "butterfly": (scan_butterfly.gru_scan_butterfly_forward_triton,
                      scan_butterfly.gru_scan_butterfly_backward_triton,
                      scan_butterfly.gru_scan_butterfly_triton),
    }


def _cuda(*ts):
    return tuple(t.cuda() for t in ts)


def check_forward(kind, out_gpu, gi, h0, W, bh, quant, free_running=True):
    """Assert forward parity; returns (max abs err | None, #code mismatches inside the tie window)."""
    out_gpu = out_gpu.cpu()
    qi, qo = quant if quant else (None, None)
    if qo is None:
        ref = orc.scan_forward(kind, gi, h0, W, bh, qi, qo)
        err = (out_gpu - ref).abs()
        assert bool((err <= FWD_TOL + FWD_TOL * ref.abs()).all()), f"max abs err {err.max().item():.3e}"
        return err.max().item(), 0
    h_prev = torch.cat([h0[None], out_gpu[:-1]], dim=0)
    # float64 after the input quantiser: the reference value of h_raw without the summation-order
    # noise of an fp32 CPU product, so the tie window measures the device's arithmetic only
    raw = orc.scan_forward_teacher_forced(kind, gi, h_prev, W, bh, qi, wide=True)
    codes_ref = orc.quant_codes(raw, qo).float()
    codes_gpu = torch.round(out_gpu / qo[0])
    assert bool((codes_gpu * qo[0] == out_gpu).all()), "device output is not on the quantisation grid"
    bad = codes_ref != codes_gpu
    n_inside = n_outside = 0
    if bool(bad.any()):
        dist = orc.tie_distance(raw, qo)[bad]
        step = (codes_ref - codes_gpu)[bad].abs()
        n_outside = int(((dist > TIE_WINDOW) | (step > 1.0)).sum())
        n_inside = int(bad.sum()) - n_outside
    identical = float("nan")
    if free_running:
        traj = orc.scan_forward(kind, gi, h0, W, bh, qi, qo)
        identical = float((traj == out_gpu).all(dim=2).all(dim=0).float().mean())
    print(f"[codes] {kind} T={gi.shape[0]} B={gi.shape[1]} H={h0.shape[1]}: {codes_gpu.numel()} codes, "
          f"mismatches inside the tie window {n_inside}, outside {n_outside}; "
          f"sequences identical to the free-running oracle through T: {identical:.4f}")
    assert n_outside == 0, f"{n_outside} code mismatches outside the {TIE_WINDOW} tie window"
    return None, n_inside


def check_backward(kind, grads_gpu, gi, h0, W, bh, out_gpu, dout, quant, tol=GRAD_TOL):
    qi, qo = quant if quant else (None, None)
    ref = orc.scan_backward(kind, gi, h0, W, bh, out_gpu.cpu(), dout, qi, qo)
    errs = {}
    for nm, a, b in zip(("dgi", "dh0", "dW", "dbh"), grads_gpu, ref):
        errs[nm] = rel_err(a.cpu(), b)
        assert errs[nm] <= tol, f"{nm}: rel err {errs[nm]:.3e}"
    return errs


GRID = [(1, 1, 32), (8, 4, 32), (8, 32, 128), (64, 4, 128), (64, 32, 512), (5, 3, 96)]


def _kwargs(kind, H):
    if kind == "monarch":
        return {"nblocks": 4}
    return {}


@pytest.mark.parametrize("quant", [None, Q8, Q8_ASYM], ids=["fp32", "q8", "q8asym"])
@pytest.mark.parametrize("T,B,H", GRID)
@pytest.mark.parametrize("kind", ["dense", "diagonal", "monarch", "butterfly"])
def test_scan_parity(kind, T, B, H, quant):
    if kind == "butterfly" and H & (H - 1):
        H = 128                                 # covered separately by the padding test
    fwd, bwd, _ = _mods()[kind]
    gi, h0, W, bh, dout = orc.make_problem(kind, T, B, H, seed=T * 1000 + B * 10 + H, **_kwargs(kind, H))
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], **kw)
    check_forward(kind, out, gi, h0, W, bh, quant)
    grads = bwd(*d[:4], out, d[4], **kw)
    check_backward(kind, grads, gi, h0, W, bh, out, dout, quant)


@pytest.mark.parametrize("quant", [None, Q8], ids=["fp32", "q8"])
@pytest.mark.parametrize("T,B,H,extra", [(8, 4, 32, {}), (16, 32, 512, {}), (5, 3, 48, {"butterfly_nblocks": 2}),
                                         (3, 2, 1024, {})])
def test_butterfly_alternate_kernels(T, B, H, extra, quant):
    """The library keeps two butterfly kernels per direction (staged twiddles, the default, and the
    register / global-twiddle one for unaligned problems); the test hook selects the latter on
    aligned shapes too, so that it keeps parity coverage there."""
    from gru_triton_b200 import _lib
    fwd, bwd, _ = _mods()["butterfly"]
    gi, h0, W, bh, dout = orc.make_problem("butterfly", T, B, H, seed=7 + T + H, **extra)
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh, dout)
    _lib.load().b200gru_test_select_kernels(1, 0)
    try:
        out = fwd(*d[:4], **kw)
        grads = bwd(*d[:4], out, d[4], **kw)
    finally:
        _lib.load().b200gru_test_select_kernels(0, 0)
    check_forward("butterfly", out, gi, h0, W, bh, quant)
    check_backward("butterfly", grads, gi, h0, W, bh, out, dout, quant)


@pytest.mark.parametrize("quant", [None, Q8, Q8_ASYM], ids=["fp32", "q8", "q8asym"])
@pytest.mark.parametrize("T,B,H,h0_gain", [(8, 1, 256, 1.0), (20, 16, 256, 1.0), (33, 17, 512, 1.0), (9, 112, 512, 1.0),
                                           (12, 5, 512, 3.0), (37, 29, 136, 1.0), (41, 27, 520, 1.0), (6, 3, 1000, 1.0), (5, 9, 200, 1.0)])
def test_dense_small_batch_cluster_shapes(T, B, H, h0_gain, quant):
    """Small-batch dense shapes of the cluster kernels (one and several clusters, a ragged last batch
    tile, |h0| above 1) and, in the last two, T*B >= 1024 rows that are no multiple of a k-block with
    H % 8 == 0: the weight gradient then runs as one tensor-core product with a ragged contraction
    tail.  Forward and backward against the oracle; no bounded wait gave up."""
    from gru_triton_b200 import _lib
    fwd, bwd, _ = _mods()["dense"]
    gi, h0, W, bh, dout = orc.make_problem("dense", T, B, H, seed=3 * T + B + H)
    h0 = h0 * h0_gain
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], **kw)
    grads = bwd(*d[:4], out, d[4], **kw)
    check_forward("dense", out, gi, h0, W, bh, quant)
    check_backward("dense", grads, gi, h0, W, bh, out, dout, quant)
    _lib.check_device_status()


@pytest.mark.parametrize("quant", [None, Q8, Q8_ASYM], ids=["fp32", "q8", "q8asym"])
@pytest.mark.parametrize("T,B,H", [(16, 64, 1024), (9, 300, 256)])
def test_diagonal_register_ring_forward_on_aligned_shapes(T, B, H, quant):
    """Shapes that normally take the bulk-copy forward kernel, forced onto the register-ring one."""
    from gru_triton_b200 import _lib
    fwd, _, _ = _mods()["diagonal"]
    gi, h0, W, bh, dout = orc.make_problem("diagonal", T, B, H, seed=T + H)
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh)
    default = fwd(*d, **kw)
    _lib.load().b200gru_test_select_kernels(0, 1)
    try:
        ring = fwd(*d, **kw)
    finally:
        _lib.load().b200gru_test_select_kernels(0, 0)
    assert torch.equal(ring, default)
    check_forward("diagonal", ring[:, :8], gi[:, :8], h0[:8], W, bh, quant)


@pytest.mark.parametrize("quant", [None, Q8, Q8_ASYM], ids=["fp32", "q8", "q8asym"])
@pytest.mark.parametrize("T,B,H", [(5, 128, 544), (6, 134, 576), (3, 130, 1024), (1, 128, 640), (4, 257, 608)])
def test_dense_per_step_path(T, B, H, quant):
    """Dense problems whose weight slice misses a cluster's shared memory, at batch >= 128, run as
    one fused SGEMM launch per time step (forward and backward); ragged batches exercise the
    padded transposed operand buffers."""
    fwd, bwd, auto = _mods()["dense"]
    gi, h0, W, bh, dout = orc.make_problem("dense", T, B, H, seed=T + B + H)
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], **kw)
    check_forward("dense", out, gi, h0, W, bh, quant)
    grads = bwd(*d[:4], out, d[4], **kw)
    check_backward("dense", grads, gi, h0, W, bh, out, dout, quant)
    # autograd route (the forward hands its gate activations to the backward)
    leaves = [t.clone().requires_grad_(True) for t in d[:4]]
    out2 = auto(*leaves, **kw)
    assert torch.equal(out2.detach(), out)
    out2.backward(d[4])
    for g_auto, g_exp in zip([t.grad for t in leaves], grads):
        assert rel_err(g_auto, g_exp) <= GRAD_TOL


@pytest.mark.parametrize("kind,name", SCAN_GOLDEN_FLAT)
def test_golden_vectors_through_the_cuda_path(kind, name):
    g = load_golden(name)
    fwd, bwd, _ = _mods()[kind]
    kw = dict(h_in_quant=g["q_in"], h_out_quant=g["q_out"]) if g["q_in"] else {}
    d = _cuda(g["gi"], g["h0"], g["W"], g["bh"], g["dout"], g["out"])
    out = fwd(*d[:4], **kw).cpu()
    if g["q_out"] is None:
        assert bool(((out - g["out"]).abs() <= FWD_TOL + FWD_TOL * g["out"].abs()).all())
    else:
        check_forward(kind, out, g["gi"], g["h0"], g["W"], g["bh"], (g["q_in"], g["q_out"]))
    grads = bwd(*d[:4], d[5], d[4], **kw)        # backward from the REFERENCE's out
    for nm, a in zip(("dgi", "dh0", "dW", "dbh"), grads):
        assert rel_err(a.cpu(), g[nm]) <= GRAD_TOL, nm


@pytest.mark.parametrize("name", BUTTERFLY_REFERENCE_GOLDEN)
def test_butterfly_against_the_references_own_kernels(name):
    """Fixtures computed on a GPU by the reference's Triton butterfly scan (its only executable
    statement of the stage / twiddle convention): forward and all four gradients."""
    g = load_golden(name)
    fwd, bwd, _ = _mods()["butterfly"]
    kw = dict(h_in_quant=g["q_in"], h_out_quant=g["q_out"]) if g["q_in"] else {}
    d = _cuda(g["gi"], g["h0"], g["W"], g["bh"], g["dout"], g["out"])
    out = fwd(*d[:4], **kw).cpu()
    if g["q_out"] is None:
        assert bool(((out - g["out"]).abs() <= FWD_TOL + FWD_TOL * g["out"].abs()).all())
    else:
        check_forward("butterfly", out, g["gi"], g["h0"], g["W"], g["bh"], (g["q_in"], g["q_out"]))
    grads = bwd(*d[:4], d[5], d[4], **kw)
    for nm, a in zip(("dgi", "dh0", "dW", "dbh"), grads):
        assert rel_err(a.cpu(), g[nm]) <= GRAD_TOL, nm


@pytest.mark.slow
@pytest.mark.parametrize("kind,T,B,H,extra,quant,bsub", [
    ("dense", 512, 8, 128, {}, None, 8), ("dense", 512, 8, 128, {}, Q8, 8),
    ("dense", 512, 130, 576, {}, None, 2), ("dense", 512, 130, 576, {}, Q8, 2),
    ("monarch", 512, 8, 128, {"nblocks": 4}, Q8, 8), ("butterfly", 512, 8, 128, {}, None, 8),
    ("butterfly", 512, 6, 128, {}, Q8, 6), ("diagonal", 512, 8, 128, {}, Q8, 8), ("diagonal", 1024, 4, 64, {}, None, 4),
], ids=lambda v: str(v) if not isinstance(v, (dict, tuple)) else ("q8" if isinstance(v, tuple) else "-"))
def test_long_chains(kind, T, B, H, extra, quant, bsub):
    """T = 512 / 1024 (the reference's slow tier, tests/test_edge_cases.py:598-614): the forward and
    the whole backward chain against the oracle; large problems are checked on a few batch rows."""
    fwd, bwd, _ = _mods()[kind]
    gi, h0, W, bh, dout = orc.make_problem(kind, T, B, H, seed=T + B + H, h0_scale=0.3, **extra)
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], **kw)
    check_forward(kind, out[:, :bsub], gi[:, :bsub], h0[:bsub], W, bh, quant)
    grads = bwd(*d[:4], out, d[4], **kw)
    if bsub == B:
        check_backward(kind, grads, gi, h0, W, bh, out, dout, quant)
    else:
        ref = orc.scan_backward(kind, gi[:, :bsub], h0[:bsub], W, bh, out[:, :bsub].cpu(), dout[:, :bsub],
                                *(quant if quant else (None, None)))
        assert rel_err(grads[0][:, :bsub].cpu(), ref[0]) <= GRAD_TOL
        assert rel_err(grads[1][:bsub].cpu(), ref[1]) <= GRAD_TOL


@pytest.mark.parametrize("kind,T,B,H,extra", [
    ("diagonal", 1, 1, 1, {}), ("diagonal", 9, 3, 2, {}), ("diagonal", 9, 5, 8, {}), ("diagonal", 7, 2, 1023, {}),
    ("diagonal", 19, 70, 1000, {}), ("diagonal", 8, 64, 1024, {}), ("diagonal", 33, 300, 256, {}),
    ("dense", 1, 1, 1, {}), ("dense", 6, 3, 2, {}), ("dense", 6, 5, 8, {}), ("dense", 4, 3, 100, {}),
    ("dense", 3, 2, 1024, {}),
    ("monarch", 6, 3, 8, {"nblocks": 8}), ("monarch", 6, 3, 24, {"nblocks": 2}), ("monarch", 5, 9, 96, {"nblocks": 4}),
    ("monarch", 4, 2, 512, {"nblocks": 2}),
    ("butterfly", 5, 3, 2, {}), ("butterfly", 5, 3, 12, {}), ("butterfly", 4, 2, 8, {"butterfly_nblocks": 2}),
    ("butterfly", 3, 5, 48, {"butterfly_nblocks": 3}), ("butterfly", 3, 2, 1024, {}),
])
@pytest.mark.parametrize("quant", [None, Q8, Q8_ASYM], ids=["fp32", "q8", "q8asym"])
def test_edge_shapes(kind, T, B, H, extra, quant):
    fwd, bwd, _ = _mods()[kind]
    gi, h0, W, bh, dout = orc.make_problem(kind, T, B, H, seed=7 + H, **extra)
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], **kw)
    check_forward(kind, out, gi, h0, W, bh, quant)
    grads = bwd(*d[:4], out, d[4], **kw)
    check_backward(kind, grads, gi, h0, W, bh, out, dout, quant)


@pytest.mark.parametrize("kind", ["dense", "diagonal", "monarch", "butterfly"])
def test_batch_invariance_and_determinism(kind):
    """A row's result does not depend on the batch it rides in, and repeated runs are bit-identical."""
    fwd, bwd, _ = _mods()[kind]
    H = 128
    gi, h0, W, bh, dout = orc.make_problem(kind, 12, 33, H, seed=99, nblocks=4)
    d = _cuda(gi, h0, W, bh, dout)
    full = fwd(*d[:4], h_in_quant=Q8[0], h_out_quant=Q8[1])
    for B in (1, 3, 5, 7, 9, 17):
        part = fwd(d[0][:, :B].contiguous(), d[1][:B].contiguous(), d[2], d[3], h_in_quant=Q8[0], h_out_quant=Q8[1])
        assert torch.equal(part, full[:, :B]), B
    g0 = bwd(*d[:4], full, d[4], h_in_quant=Q8[0], h_out_quant=Q8[1])
    for _ in range(5):
        assert torch.equal(fwd(*d[:4], h_in_quant=Q8[0], h_out_quant=Q8[1]), full)
        g1 = bwd(*d[:4], full, d[4], h_in_quant=Q8[0], h_out_quant=Q8[1])
        for a, b in zip(g0, g1):
            assert torch.equal(a, b)


@pytest.mark.parametrize("kind", ["dense", "diagonal", "monarch", "butterfly"])
@pytest.mark.parametrize("quant", [None, Q8], ids=["fp32", "q8"])
def test_autograd_matches_explicit_backward(kind, quant):
    """autograd (forward saves the gate activations) vs the explicit backward (recomputes them)."""
    fwd, bwd, fn = _mods()[kind]
    gi, h0, W, bh, dout = orc.make_problem(kind, 16, 8, 64, seed=5, nblocks=4)
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    leaves = [t.cuda().requires_grad_(True) for t in (gi, h0, W, bh)]
    out = fn(*leaves, **kw)
    out.backward(dout.cuda())
    explicit = bwd(*[l.detach() for l in leaves], out.detach(), dout.cuda(), **kw)
    assert torch.equal(out.detach(), fwd(*[l.detach() for l in leaves], **kw))
    for leaf, e in zip(leaves, explicit):
        assert rel_err(leaf.grad, e) <= GRAD_TOL
    check_backward(kind, [l.grad for l in leaves], gi, h0, W, bh, out.detach(), dout, quant)


@pytest.mark.parametrize("cls", ["near-saturation", "large-magnitude"])
@pytest.mark.parametrize("kind", ["dense", "diagonal", "monarch", "butterfly"])
def test_adversarial_quant_inputs(kind, cls):
    """Inputs that sit at the int8 clip boundary or far beyond it clip the same way as the oracle."""
    fwd, bwd, _ = _mods()[kind]
    T, B, H = 8, 4, 128
    gi, h0, W, bh, dout = orc.make_problem(kind, T, B, H, seed=3, nblocks=4)
    if cls == "near-saturation":
        gi = torch.linspace(-0.99, 0.99, gi.numel()).reshape(gi.shape) * 2.54 * 3
        h0 = torch.linspace(-0.99, 0.99, h0.numel()).reshape(h0.shape) * 2.54
    else:
        gi, h0 = gi * 5.0, torch.randn(B, H, generator=torch.Generator().manual_seed(1)) * 5.0
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], h_in_quant=Q8[0], h_out_quant=Q8[1])
    check_forward(kind, out, gi, h0, W, bh, Q8)
    grads = bwd(*d[:4], out, d[4], h_in_quant=Q8[0], h_out_quant=Q8[1])
    check_backward(kind, grads, gi, h0, W, bh, out, dout, Q8)


def test_wrapper_validation_on_cuda():
    from gru_triton_b200 import scan, scan_butterfly, scan_diagonal, scan_monarch
    T, B, H = 4, 2, 8
    dev = "cuda"
    gi, h0, bh = torch.randn(T, B, 3 * H, device=dev), torch.zeros(B, H, device=dev), torch.zeros(3 * H, device=dev)
    Wd = torch.randn(3 * H, H, device=dev)
    bad = [
        lambda: scan.gru_scan(gi.double(), h0.double(), Wd.double(), bh.double()),
        lambda: scan.gru_scan(gi, torch.zeros(B + 1, H, device=dev), Wd, bh),
        lambda: scan.gru_scan(gi, h0, torch.randn(3 * H, H + 1, device=dev), bh),
        lambda: scan.gru_scan_persistent(gi, torch.zeros(B + 1, H, device=dev), Wd, bh),
        lambda: scan_diagonal.gru_scan_diagonal(gi, h0, torch.randn(3, H + 1, device=dev), bh),
        lambda: scan_monarch.gru_scan_monarch(gi, h0, torch.randn(3, 2, 5, 5, device=dev), bh),
        lambda: scan_butterfly.gru_scan_butterfly_triton(gi, torch.zeros(B + 1, H, device=dev),
                                                         torch.randn(3, 1, 3, 4, 2, 2, device=dev), bh),
        lambda: scan.gru_scan(gi, h0, Wd, bh, h_in_quant=(0.0, -127, 127)),
    ]
    for f in bad:
        with pytest.raises((ValueError, RuntimeError)) as e:
            f()
        assert not isinstance(e.value, AssertionError)


def _recipe(hidden_bits=32, mode="frozen"):
    from gru_triton_b200 import QuantizerConfig, QuantRecipe
    return QuantRecipe(weight=QuantizerConfig(bits=32, axis=0, name="W"),
                       input_act=QuantizerConfig(bits=32, name="x_id"),
                       hidden=QuantizerConfig(bits=hidden_bits, mode=mode, name="h"))


@pytest.mark.parametrize("kind", ["diagonal", "monarch", "butterfly"])
def test_layer_fast_dispatch_matches_per_step_path(kind):
    """GRULayer on CUDA (one GEMM + one scan launch) against the same layer stepping on CPU."""
    import copy
    from gru_triton_b200 import GRULayer, StructureConfig
    torch.manual_seed(11)
    T, B, H = 12, 5, 64
    lay = GRULayer(H, H, _recipe(), gate_layout="fused", structure_hidden=StructureConfig(kind=kind, nblocks=4))
    x, h0 = torch.randn(T, B, H), torch.randn(B, H) * 0.3
    ref, ref_hT = lay(x, h0)
    ref.sum().backward()
    gl = copy.deepcopy(lay).cuda()
    gl.zero_grad()
    assert gl.use_triton
    out, hT = gl(x.cuda(), h0.cuda())
    out.sum().backward()
    assert bool(((out.cpu() - ref).abs() <= FWD_TOL + FWD_TOL * ref.abs()).all())
    assert torch.equal(hT, out[-1])
    for (n, p), (_, q) in zip(lay.named_parameters(), gl.named_parameters()):
        assert rel_err(q.grad.cpu(), p.grad) <= GRAD_TOL, n
    # batch_first plumbing
    from gru_triton_b200 import GRULayer as GL
    bf = GL(H, H, _recipe(), batch_first=True, gate_layout="fused",
            structure_hidden=StructureConfig(kind=kind, nblocks=4)).cuda()
    bf.load_state_dict(gl.state_dict())
    ob, _ = bf(x.cuda().transpose(0, 1).contiguous(), h0.cuda())
    assert torch.equal(ob.transpose(0, 1), out)


def test_calibrate_freeze_then_cuda_scan():
    """calibrate() (per-step path) -> freeze() -> CUDA scan with the frozen int8 scales."""
    import copy
    from gru_triton_b200 import GRULayer, StructureConfig
    torch.manual_seed(3)
    T, B, H = 16, 6, 64
    lay = GRULayer(H, H, _recipe(8, mode="dynamic"), gate_layout="fused",
                   structure_hidden=StructureConfig(kind="diagonal")).cuda()
    stats = lay.calibrate([torch.randn(T, B, H, device="cuda") for _ in range(3)], n_batches=3)
    assert stats["cell.quant_h_in"]["initialized"] and lay.use_triton
    lay.freeze()
    x = torch.randn(T, B, H, device="cuda")
    out, _ = lay(x)
    cpu = copy.deepcopy(lay).cpu()
    q_in = (float(cpu.cell.quant_h_in.scale), -127, 127)
    q_out = (float(cpu.cell.quant_h_out.scale), -127, 127)
    from gru_triton_b200.scan_diagonal import extract_diagonal_factors
    Wi, bi = cpu.cell.quantize_input_weights()
    gi = torch.nn.functional.linear(x, Wi.cuda(), bi.cuda()).cpu()
    W, bh = extract_diagonal_factors(cpu.cell)
    check_forward("diagonal", out.detach(), gi, torch.zeros(B, H), W.detach(), bh.detach(), (q_in, q_out))


def test_baseline_config_shapes_forward_backward():
    """The benchmark shapes themselves: C1 dense (full), C3 monarch (full), C4 butterfly and
    C2 diagonal (full launch on the device, oracle on a slice of the independent batch rows)."""
    cases = [("dense", 64, 32, 512, {}, None, 32), ("monarch", 64, 32, 512, {"nblocks": 8}, Q8, 32),
             ("butterfly", 128, 64, 1024, {}, None, 4), ("diagonal", 1024, 256, 1024, {}, Q8, 2)]
    for kind, T, B, H, extra, quant, bsub in cases:
        fwd, bwd, _ = _mods()[kind]
        gi, h0, W, bh, dout = orc.make_problem(kind, T, B, H, seed=1, h0_scale=0.1, **extra)
        kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
        d = _cuda(gi, h0, W, bh, dout)
        out = fwd(*d[:4], **kw)
        check_forward(kind, out[:, :bsub], gi[:, :bsub], h0[:bsub], W, bh, quant)
        if kind == "diagonal":
            continue                                    # C2 is forward only
        grads = bwd(*d[:4], out, d[4], **kw)
        sub = bwd(d[0][:, :bsub].contiguous(), d[1][:bsub].contiguous(), d[2], d[3], out[:, :bsub].contiguous(),
                  d[4][:, :bsub].contiguous(), **kw)
        assert torch.equal(sub[0], grads[0][:, :bsub]) and torch.equal(sub[1], grads[1][:bsub])
        check_backward(kind, sub, gi[:, :bsub], h0[:bsub], W, bh, out[:, :bsub], dout[:, :bsub], quant)


@pytest.mark.parametrize("T,B,H,quant", [(5, 3, 1000, Q8), (7, 2, 1024, None), (3, 74, 1024, Q8_ASYM), (6, 1, 1016, None),
                                          (1, 1, 1024, None), (2, 3, 1024, None)])
def test_butterfly_two_cta_forward(T, B, H, quant):
    """H around 1024 with at most 74 rows runs the forward as a pair of CTAs per row (gates r, z in one,
    n in the other, halves exchanged through distributed shared memory): parity with the oracle,
    bit-identity with the one-CTA kernel (the same rows inside a batch too large for pairs), and the
    backward without saved activations, whose gate recompute runs the same forward kernel and whose
    scan runs as pairs as well (gates r, z in one CTA, n in the other, partial sums exchanged)."""
    fwd, bwd, _ = _mods()["butterfly"]
    gi, h0, W, bh, dout = orc.make_problem("butterfly", T, B, H, seed=11, h0_scale=0.3)
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], **kw)
    bsub = min(B, 3)
    check_forward("butterfly", out[:, :bsub], gi[:, :bsub], h0[:bsub], W, bh, quant)
    big = 80                                                 # 2 * 80 CTAs exceed the SM count: one CTA per row block
    reps = (big + B - 1) // B
    gi_big = d[0].repeat(1, reps, 1)[:, :big].contiguous()
    h0_big = d[1].repeat(reps, 1)[:big].contiguous()
    out_big = fwd(gi_big, h0_big, d[2], d[3], **kw)
    assert torch.equal(out_big[:, :B], out)
    grads = bwd(*d[:4], out, d[4], **kw)                     # no `save`: recomputes the gates
    sub = [g[:, :bsub] if g.dim() == 3 else g for g in grads[:1]] + [grads[1][:bsub]]
    ref = orc.scan_backward("butterfly", gi[:, :bsub], h0[:bsub], W, bh, out[:, :bsub].cpu(), dout[:, :bsub],
                            *(quant if quant else (None, None)))
    assert rel_err(sub[0].cpu(), ref[0]) <= GRAD_TOL and rel_err(sub[1].cpu(), ref[1]) <= GRAD_TOL
    # the backward scan runs as pairs too; the same rows inside the large batch take the one-CTA kernel
    dout_big = d[4].repeat(1, reps, 1)[:, :big].contiguous()
    grads_big = bwd(gi_big, h0_big, d[2], d[3], out_big, dout_big, **kw)
    assert torch.equal(grads_big[0][:, :B], grads[0]) and torch.equal(grads_big[1][:B], grads[1])


def test_baseline_config5_shard_shape():
    """C5 as one of eight GPUs sees it (B=512, H=1024, int8 weights and hidden state), T cut to 8:
    the full launch runs on the device, the oracle checks a slice of the independent batch rows
    (forward codes, dgi and dh0); dW and dbh are checked through their linearity in the batch:
    the gradient of the whole batch equals the sum over two halves run separately."""
    T, B, H, bsub = 8, 512, 1024, 3
    fwd, bwd, _ = _mods()["dense"]
    gi, h0, W, bh, dout = orc.make_problem("dense", T, B, H, seed=5, h0_scale=0.1)
    W = orc.per_row_weight_fake_quant(W)                      # int8 grid per output row
    quant = ((0.008, -127, 127), (0.008, -127, 127))
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1])
    d = _cuda(gi, h0, W, bh, dout)
    out = fwd(*d[:4], **kw)
    check_forward("dense", out[:, :bsub], gi[:, :bsub], h0[:bsub], W, bh, quant)
    grads = bwd(*d[:4], out, d[4], **kw)
    ref = orc.scan_backward("dense", gi[:, :bsub], h0[:bsub], W, bh, out[:, :bsub].cpu(), dout[:, :bsub], *quant)
    assert rel_err(grads[0][:, :bsub].cpu(), ref[0]) <= GRAD_TOL
    assert rel_err(grads[1][:bsub].cpu(), ref[1]) <= GRAD_TOL
    halves = []
    for sl in (slice(0, B // 2), slice(B // 2, B)):
        halves.append(bwd(d[0][:, sl].contiguous(), d[1][sl].contiguous(), d[2], d[3], out[:, sl].contiguous(),
                          d[4][:, sl].contiguous(), **kw))
    assert rel_err(halves[0][2] + halves[1][2], grads[2]) <= GRAD_TOL
    assert rel_err(halves[0][3] + halves[1][3], grads[3]) <= GRAD_TOL
    # rows are independent; the contraction of the backward product is split over CTAs according to
    # the batch size, so halves and whole agree to rounding, not bit for bit
    assert rel_err(torch.cat([halves[0][0], halves[1][0]], dim=1), grads[0]) <= 1e-5
    out_half = fwd(d[0][:, :B // 2].contiguous(), d[1][:B // 2].contiguous(), d[2], d[3], **kw)
    assert torch.equal(out_half, out[:, :B // 2])                                     # the forward is bit-exact


@pytest.mark.parametrize("kind,T,B,H,extra", [("dense", 16, 32, 512, {}), ("dense", 6, 3, 1024, {}),
                                              ("monarch", 16, 32, 512, {"nblocks": 8}),
                                              ("monarch", 8, 5, 1024, {"nblocks": 2})])
def test_cluster_exchange_is_race_free(kind, T, B, H, extra):
    """The cluster kernels exchange data through asynchronous DSMEM stores; repeated launches of the
    same problem (weights in shared memory and weights streamed from L2) must agree bit for bit."""
    fwd, bwd, _ = _mods()[kind]
    gi, h0, W, bh, dout = _cuda(*orc.make_problem(kind, T, B, H, seed=21, **extra))
    out0 = fwd(gi, h0, W, bh)
    g0 = bwd(gi, h0, W, bh, out0, dout)
    for _ in range(8):
        assert torch.equal(fwd(gi, h0, W, bh), out0)
        for a, b in zip(bwd(gi, h0, W, bh, out0, dout), g0):
            assert torch.equal(a, b)
    check_forward(kind, out0, *[t.cpu() for t in (gi, h0, W, bh)], None)
    check_backward(kind, g0, *[t.cpu() for t in (gi, h0, W, bh)], out0, dout.cpu(), None)


@pytest.mark.parametrize("quant", [None, Q8], ids=["fp32", "q8"])
@pytest.mark.parametrize("T,B,nb,bs", [(8, 4, 4, 8), (16, 32, 8, 64)])
def test_two_factor_monarch_extension(T, B, nb, bs, quant):
    """gru_scan_monarch2 (two block-diagonal factors around the Monarch permutation, the operator
    BASELINE config 3 words) against the oracle's dense scan on the loop-materialised matrix;
    factor gradients against autograd through that materialisation.  Parity with the reference is
    not defined for this operator."""
    from gru_triton_b200 import scan_monarch
    H = nb * bs
    gen = torch.Generator().manual_seed(T + H)
    gi, h0, _, bh, dout = orc.make_problem("dense", T, B, H, seed=H)
    W1 = torch.randn(3, nb, bs, bs, generator=gen) * bs ** -0.5
    W2 = torch.randn(3, nb, bs, bs, generator=gen) * bs ** -0.5
    Md = orc.monarch2_dense_loops(W1, W2) if H <= 64 else scan_monarch.monarch2_dense(W1.double(), W2.double()).float()
    leaves = [t.cuda().requires_grad_(True) for t in (gi, h0, W1, W2, bh)]
    kw = dict(h_in_quant=quant[0], h_out_quant=quant[1]) if quant else {}
    out = scan_monarch.gru_scan_monarch2(*leaves, **kw)
    check_forward("dense", out.detach(), gi, h0, Md, bh, quant)
    out.backward(dout.cuda())
    qi, qo = quant if quant else (None, None)
    ref = orc.scan_backward("dense", gi, h0, Md, bh, out.detach().cpu(), dout, qi, qo)
    W1l, W2l = W1.clone().requires_grad_(True), W2.clone().requires_grad_(True)
    scan_monarch.monarch2_dense(W1l, W2l).backward(ref[2])
    for nm, a, b in zip(("dgi", "dh0", "dW1", "dW2", "dbh"), [l.grad for l in leaves],
                        (ref[0], ref[1], W1l.grad, W2l.grad, ref[3])):
        assert rel_err(a.cpu(), b) <= GRAD_TOL, nm


def test_zz_no_bounded_wait_gave_up():
    """Runs after the other tests of this file: none of the in-kernel waits timed out."""
    from gru_triton_b200 import _lib
    assert _lib.load().b200gru_device_status(0) == 0
