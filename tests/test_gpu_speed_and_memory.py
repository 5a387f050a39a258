"""Smoke test of the sweep script: two sizes, the reference's CSV columns
(Experiments/speed_and_memory/bench.py:139-150 without the pykeops version), skip-if-done on a second run."""

import csv
import importlib.util
import os

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sweep_writes_the_reference_columns_and_skips_done_rows(tmp_path):
    spec = importlib.util.spec_from_file_location(
        "speed_and_memory", os.path.join(ROOT, "quasi-linear-kernel-attention_b200", "kernel_attention", "speed_and_memory.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = str(tmp_path / "sweep.csv")
    argv = ["--sizes", "128", "256", "--runs", "2", "--warmups", "1", "--B", "1", "--H", "2", "--out", out]
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    with_ref = os.path.exists(os.path.join(ref_dir, "ref_abs_ext", "ref_abs_ext.so")) and os.path.exists(os.path.join(ref_dir, "ref_laplace_ext", "ref_laplace_ext.so"))
    if with_ref:
        argv += ["--ref-ext-dir", ref_dir]
    written = mod.main(argv)
    rows = list(csv.DictReader(open(out)))
    assert written == len(rows) > 0
    for col in ("method", "backend", "dtype", "B", "H", "D", "C", "N", "mode", "gpu", "time_mean_ms", "time_std_ms",
                "peak_mem_mb", "runs", "warmups", "hostname", "torch", "cuda", "cudnn", "date"):
        assert col in rows[0], col
    ours = [r for r in rows if r["backend"] == "qlka"]
    assert {r["method"] for r in ours} == {"add_laplace", "add_riesz"}
    assert {r["mode"] for r in ours} == {"fwd", "fwd+bwd"}
    assert all(float(r["time_mean_ms"]) > 0 for r in ours)
    if with_ref:
        assert any(r["backend"] == "ref-ext" and float(r["time_mean_ms"]) > 0 for r in rows)
    assert mod.main(argv) == 0          # everything is already in the file
