"""The JSON line of ``bench.py``: keys of the contract, checked on the reference arm (CPU only) and on
the helpers the device arm shares with it."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest

from conftest import REPO


def _reference_line(extra=()):
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", *extra], capture_output=True, text=True, timeout=600, env=env, cwd=REPO)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_prints_the_contract_keys():
    oracle_ref = os.path.join(REPO, "oracle", "_ref", "gru_qat", "__init__.py")
    if not os.path.isfile(oracle_ref):
        pytest.skip("reference package not installed under oracle/_ref")
    d = _reference_line()
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["unit"] == "seq-steps/s" and d["value"] > 0
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"]
    assert e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    # seq-steps/s = T * B / step time
    cfg = d["config"]
    assert abs(d["value"] - cfg["T"] * cfg["B_per_gpu"] / (d["ms_per_step"] * 1e-3)) <= 1e-6 * d["value"]


def test_both_arms_describe_the_workload_with_the_same_keys():
    sys.path.insert(0, REPO)
    import bench
    for name, cfg in bench.CONFIGS.items():
        a = bench.config_dict(name, cfg, cfg["B"], 1, False)
        assert {"workload", "T", "B_per_gpu", "H", "hidden_kind", "int8_hidden", "weight_bits", "train_step",
                "parallelism", "l2"} == set(a), name
        assert a["workload"].startswith(name + ":")
    # the default workload is the headline configuration: dense fp32 train step T=64 B=32 H=512
    c1 = bench.CONFIGS["c1"]
    assert (c1["kind"], c1["T"], c1["B"], c1["H"], c1["train"], c1["quant"]) == ("dense", 64, 32, 512, True, False)
