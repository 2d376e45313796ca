"""Host-side logic on CPU: the layer/cell/quantizer mirror, its plain-PyTorch scan
functions, argument validation, and the C ABI's exported symbols."""

from __future__ import annotations

import ctypes
import os
import re

import pytest
import torch

from conftest import REPO, SCAN_GOLDEN_FLAT, load_golden, rel_err

import gru_triton_b200 as pkg
from gru_triton_b200 import GRULayer, QuantizerConfig, QuantRecipe, StructureConfig
from gru_triton_b200 import _lib, scan, scan_butterfly, scan_diagonal, scan_monarch, torch_ref


def _recipe(hidden_bits=32, weight_bits=32, mode="frozen"):
    return QuantRecipe(weight=QuantizerConfig(bits=weight_bits, axis=0, name="W"),
                       input_act=QuantizerConfig(bits=32, name="x_id"),
                       hidden=QuantizerConfig(bits=hidden_bits, mode=mode, name="h"))


def _load_params(layer, g):
    with torch.no_grad():
        for k, v in g.items():
            if k.startswith("p:"):
                layer.get_parameter(k[2:]).copy_(v)


def _set_scales(layer, q_in, q_out):
    for q, p in ((layer.cell.quant_h_in, q_in), (layer.cell.quant_h_out, q_out)):
        q.scale = torch.tensor(p[0])
        q.zero_point = torch.tensor(0.0)
        q.config.mode = "frozen"


@pytest.mark.parametrize("name,kind,wbits", [("layer_dense_fp32", "dense", 32), ("layer_dense_w8h8", "dense", 8),
                                             ("layer_diagonal_fp32", "diagonal", 32),
                                             ("layer_diagonal_q8", "diagonal", 32)])
def test_layer_per_step_path_matches_reference(name, kind, wbits):
    g = load_golden(name)
    I, H = g["x"].shape[2], g["h0"].shape[1]
    structure = None if kind == "dense" else StructureConfig(kind=kind)
    layer = GRULayer(I, H, _recipe(8 if g["q_in"] else 32, wbits), gate_layout="fused",
                     structure_hidden=structure, use_triton=False)
    _load_params(layer, g)
    if g["q_in"]:
        _set_scales(layer, g["q_in"], g["q_out"])
    out, hT = layer(g["x"], g["h0"])
    out.sum().backward()
    assert (out - g["out"]).abs().max().item() < 1e-5
    assert torch.equal(hT, out[-1])
    for k, v in g.items():
        if k.startswith("g:"):
            assert rel_err(layer.get_parameter(k[2:]).grad, v) < 1e-4, k


def test_calibrate_freeze_flow_matches_reference():
    g = load_golden("calib_diagonal")
    H = g["x0"].shape[2]
    layer = GRULayer(H, H, _recipe(8, 32, mode="dynamic"), gate_layout="fused",
                     structure_hidden=StructureConfig(kind="diagonal"))
    _load_params(layer, g)
    assert layer.use_triton is True
    summary = layer.calibrate([g["x0"], g["x1"], g["x2"]], n_batches=3)
    assert layer.use_triton is True                       # restored after calibration
    layer.freeze()
    assert abs(summary["cell.quant_h_in"]["running_min"] - float(g["rmin_in"])) < 1e-6
    assert abs(summary["cell.quant_h_out"]["running_max"] - float(g["rmax_out"])) < 1e-6
    assert rel_err(layer.cell.quant_h_in.scale, g["s_in"]) < 1e-6
    assert rel_err(layer.cell.quant_h_out.scale, g["s_out"]) < 1e-6
    assert layer.cell.quant_h_in.config.mode == "frozen"
    out, _ = layer(g["x_eval"])                            # CPU input: per-step path
    assert (out - g["out_eval"]).abs().max().item() < 1e-5


@pytest.mark.parametrize("kind,name", SCAN_GOLDEN_FLAT)
def test_package_pytorch_scan_functions(kind, name):
    g = load_golden(name)
    out = torch_ref.scan_forward(kind, g["gi"], g["h0"], g["W"], g["bh"], h_in_quant=g["q_in"],
                                 h_out_quant=g["q_out"])
    assert (out - g["out"]).abs().max().item() < 1e-5
    got = torch_ref.scan_backward(kind, g["gi"], g["h0"], g["W"], g["bh"], g["out"], g["dout"],
                                  h_in_quant=g["q_in"], h_out_quant=g["q_out"])
    for nm, a in zip(("dgi", "dh0", "dW", "dbh"), got):
        assert rel_err(a, g[nm]) < 1e-4, nm


def test_structured_modules_feed_the_extractors():
    torch.manual_seed(0)
    H = 16
    lay = GRULayer(H, H, _recipe(), gate_layout="fused", structure_hidden=StructureConfig(kind="monarch", nblocks=4))
    W, bh = scan_monarch.extract_monarch_factors(lay.cell)
    assert W.shape == (3, 4, 4, 4) and bh.shape == (3 * H,)
    lay = GRULayer(12, 12, _recipe(), gate_layout="fused", structure_hidden=StructureConfig(kind="butterfly"))
    tw, bh = scan_butterfly.extract_butterfly_twiddles(lay.cell)
    assert tw.shape == (3, 1, 4, 8, 2, 2)
    mods, _ = scan_butterfly.extract_butterfly_factors(lay.cell)
    x = torch.randn(5, 3, 36)
    h0 = torch.randn(3, 12)
    a = scan_butterfly.gru_scan_butterfly(x, h0, mods, bh)
    b = torch_ref.scan_forward("butterfly", x, h0, tw, bh)
    assert (a - b).abs().max().item() < 1e-6
    lay = GRULayer(H, H, _recipe(), gate_layout="fused", structure_hidden=StructureConfig(kind="diagonal"))
    Wd, _ = scan_diagonal.extract_diagonal_factors(lay.cell)
    assert Wd.shape == (3, H)
    # the per-step structured cell agrees with the scan-form reference
    x = torch.randn(6, 2, H)
    out, _ = lay(x)
    Wi, bi = lay.cell.quantize_input_weights()
    ref = torch_ref.scan_forward("diagonal", torch.nn.functional.linear(x, Wi, bi), torch.zeros(2, H),
                                 *scan_diagonal.extract_diagonal_factors(lay.cell))
    assert (out - ref).abs().max().item() < 1e-5


def test_layer_argument_errors():
    rec = _recipe()
    with pytest.raises(ValueError):
        GRULayer(8, 8, rec, gate_layout="split", use_triton=True)          # split gates are not dispatchable
    with pytest.raises(ValueError):
        GRULayer(8, 8, rec, pre_batch_input=True)                          # needs fused
    with pytest.raises(ValueError):
        GRULayer(8, 8, rec, gate_layout="fused", structure_hidden=StructureConfig(kind="butterfly"),
                 pre_batch_input=True)
    with pytest.raises(ValueError):
        GRULayer(1, 1, rec, gate_layout="fused", structure_hidden=StructureConfig(kind="butterfly"))
    with pytest.raises(ValueError):
        GRULayer(8, 8, QuantRecipe(weight=QuantizerConfig(bits=8, axis=None)), gate_layout="fused")
    lay = GRULayer(8, 8, rec, gate_layout="fused")
    with pytest.raises(ValueError, match="T"):
        lay(torch.zeros(0, 2, 8))
    with pytest.raises(ValueError, match="B"):
        lay(torch.zeros(3, 0, 8))
    assert GRULayer(8, 8, rec, gate_layout="fused").use_triton is True     # dense + fused: this build's extension
    assert GRULayer(8, 8, rec, gate_layout="split").use_triton is False
    assert GRULayer(8, 8, rec, gate_layout="fused",
                    structure_hidden=StructureConfig(kind="diagonal")).use_triton is True
    assert GRULayer(8, 8, rec, gate_layout="split",
                    structure_hidden=StructureConfig(kind="diagonal")).use_triton is False


_ENTRY_POINTS = [
    (scan.gru_scan, "dense"), (scan.gru_scan_persistent, "dense"), (scan.gru_scan_forward, "dense"),
    (scan.gru_scan_forward_persistent, "dense"), (scan_diagonal.gru_scan_diagonal, "diagonal"),
    (scan_monarch.gru_scan_monarch, "monarch"), (scan_butterfly.gru_scan_butterfly_triton, "butterfly"),
]


@pytest.mark.parametrize("fn,kind", _ENTRY_POINTS)
def test_scan_entry_points_reject_cpu_tensors(fn, kind):
    """No CPU fallback: a CPU tensor is an error, and never an AssertionError."""
    T, B, H = 4, 2, 8
    W = {"dense": torch.randn(3 * H, H), "diagonal": torch.randn(3, H),
         "monarch": torch.randn(3, 2, 4, 4), "butterfly": torch.randn(3, 1, 3, 4, 2, 2)}[kind]
    with pytest.raises((ValueError, RuntimeError)) as e:
        fn(torch.randn(T, B, 3 * H), torch.zeros(B, H), W, torch.zeros(3 * H))
    assert not isinstance(e.value, AssertionError)


def test_reference_module_aliases():
    for mod, names in ((scan, ["gru_scan_backward_triton", "gru_scan_backward_persistent",
                               "_gru_scan_backward_pytorch", "GRUScanFunction", "GRUScanPersistentFunction"]),
                       (scan_diagonal, ["gru_scan_diagonal_forward_triton", "gru_scan_diagonal_backward_triton",
                                        "gru_scan_diagonal_forward_pytorch", "gru_scan_diagonal_backward_pytorch",
                                        "GRUScanDiagonalFunction", "extract_diagonal_factors"]),
                       (scan_monarch, ["gru_scan_monarch_forward_triton", "gru_scan_monarch_backward_triton",
                                       "gru_scan_monarch_forward_pytorch", "gru_scan_monarch_backward_pytorch",
                                       "GRUScanMonarchFunction", "extract_monarch_factors"]),
                       (scan_butterfly, ["gru_scan_butterfly_forward_triton", "gru_scan_butterfly_backward_triton",
                                         "gru_scan_butterfly", "GRUScanButterflyTritonFunction",
                                         "extract_butterfly_factors", "extract_butterfly_twiddles"])):
        for n in names:
            assert hasattr(mod, n), (mod.__name__, n)
    for n in pkg.__all__:
        assert hasattr(pkg, n)


def test_library_exports_every_declared_symbol():
    """The shared library loads and exports each function include/b200gru.h declares."""
    header = open(os.path.join(REPO, "include", "b200gru.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(b200gru_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    lib = _lib.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.b200gru_version() >= 100
    assert lib.b200gru_strerror(1) == b"invalid argument"
    # host-only queries (no device work)
    shp = _lib.make_shape("diagonal", 8, 4, 16)
    assert lib.b200gru_workspace_bytes(ctypes.byref(shp), 0) == 0
    assert lib.b200gru_workspace_bytes(ctypes.byref(shp), 1) > 0
    bad = _lib.make_shape("monarch", 8, 4, 10, nblocks=3)
    assert lib.b200gru_workspace_bytes(ctypes.byref(bad), 0) == ctypes.c_size_t(-1).value
    dense = _lib.make_shape("dense", 8, 4, 16)
    assert lib.b200gru_save_bytes(ctypes.byref(dense)) == 4 * 8 * 4 * 16 * 4
    # argument errors are reported before any device work
    assert lib.b200gru_scan_forward(ctypes.byref(dense), None, None, None, None, None, None, None, None,
                                    None, 0, None) == 1


def test_device_status_check_raises_on_a_reported_timeout(monkeypatch):
    """The Python side of the health word: a non-zero b200gru_device_status becomes DeviceWaitTimeout,
    a CUDA error a RuntimeError, zero nothing (driven with a stand-in for the library: no GPU)."""
    class Fake:
        def __init__(self, v):
            self.v, self.resets = v, []

        def b200gru_device_status(self, reset):
            self.resets.append(reset)
            return self.v

        def b200gru_last_cuda_error(self):
            return b"unspecified launch failure"

    for v, exc in ((1, _lib.DeviceWaitTimeout), (-1, RuntimeError)):
        fake = Fake(v)
        monkeypatch.setattr(_lib, "load", lambda fake=fake: fake)
        with pytest.raises(exc):
            _lib.check_device_status()
        assert fake.resets == [1]
    fake = Fake(0)
    monkeypatch.setattr(_lib, "load", lambda: fake)
    _lib.check_device_status(reset=False)
    assert fake.resets == [0]


@pytest.mark.parametrize("nb,bs", [(2, 2), (3, 4), (4, 2), (8, 8)])
def test_two_factor_monarch_materialisation(nb, bs):
    """The vectorised dense form of P^T B2 P B1 against the oracle's index-loop form (the checker of
    the two-factor extension; parity with the reference is undefined: it has one factor per gate)."""
    from oracle import gru_scan_oracle as orc
    gen = torch.Generator().manual_seed(nb * 10 + bs)
    W1 = torch.randn(3, nb, bs, bs, generator=gen, dtype=torch.float64)
    W2 = torch.randn(3, nb, bs, bs, generator=gen, dtype=torch.float64)
    assert (scan_monarch.monarch2_dense(W1, W2) - orc.monarch2_dense_loops(W1, W2)).abs().max() < 1e-12
    # a single factor is the special case B2 = I with the permutation undone
    eye = torch.eye(bs, dtype=torch.float64).expand(3, nb, bs, bs).contiguous()
    single = torch.cat([torch.block_diag(*W1[g]) for g in range(3)], 0)
    if nb == bs:
        assert (scan_monarch.monarch2_dense(W1, eye) - single).abs().max() < 1e-12
