"""The arithmetic behind the bench record (bytes a decode step reads, FLOPs of a prefill, peaks), and what
the bench says when asked for more than one GPU. No GPU is needed."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


@pytest.fixture()
def shape():
    saved = dict(bench.MODEL)
    yield lambda name: bench.MODEL.update(bench.SHAPES[name])
    bench.MODEL.clear()
    bench.MODEL.update(saved)


def test_step_bytes_and_prefill_flops_of_the_three_shapes(shape):
    # per layer: (q + 2 kv heads) * hd * hidden + hidden * q * hd + 3 * hidden * intermediate matrix parameters
    n = bench.model_numbers(24)                                  # 0.5B: 357.83 M in the layers + 136.13 M head
    assert n["per_layer_params"] == (14 + 4) * 64 * 896 + 896 * 14 * 64 + 3 * 896 * 4864
    assert round(n["weight_bytes"] / 1e6) == 988
    assert n["kv_bytes_per_token"] == 12 * 1024
    assert abs(n["prefill_flops"](2048) / 1e12 - 1.65) < 0.01
    shape("1.5b")
    n = bench.model_numbers(28)
    assert round(n["weight_bytes"] / 1e6) == 3087 and n["kv_bytes_per_token"] == 28 * 1024
    assert abs(n["prefill_flops"](2048) / 1e12 - 5.73) < 0.01
    shape("7b")
    n = bench.model_numbers(28)
    assert round(n["weight_bytes"] / 1e9, 2) == 14.14 and n["kv_bytes_per_token"] == 56 * 1024
    assert abs(n["prefill_flops"](2048) / 1e12 - 27.57) < 0.02
    assert bench.model_numbers(4)["weight_bytes"] < n["weight_bytes"]      # fewer layers: fewer bytes, named in config


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.peaks() == bench.FALLBACK_PEAKS and bench.peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"hbm_gbs": 6900.5, "bf16_tflops": 1610, "bf16_tflops_sustained": {"value": 1405.0}, "clocks": {"sm": 1900}}))
    p = bench.peaks()
    assert (p["hbm_gbs"], p["bf16_tflops"], p["bf16_tflops_sustained"], p["source"]) == (6900.5, 1610.0, 1405.0, "measured")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 7000}))
    p = bench.peaks()
    assert p["hbm_gbs"] == 7000.0 and p["bf16_tflops"] == 1590.0 and "partly" in p["source"]
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert bench.peaks()["source"] == "fallback"


def test_more_than_one_gpu_is_refused_with_one_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 2
    lines = [line for line in r.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and json.loads(lines[0])["n_gpus"] == 2


def test_launches_are_sorted_into_the_parts_of_a_layer():
    """The breakdown names a launch by its kernel, its epilogue and its place in the layer's order."""
    epi = {"qkv": "qkv", "o": "add", "gate_up": "swiglu", "down": "add", "head": "f32"}
    order = [("embed", None), ("gemm_smallm", "qkv"), ("attention_decode", None), ("gemm_smallm", "o"), ("rmsnorm", None),
             ("gemm_smallm", "gate_up"), ("gemm_tc", "down"), ("rmsnorm", None), ("gemm_tc", "qkv"), ("rope_store", None),
             ("attention_decode", None), ("gemm_tc", "o"), ("rmsnorm", None), ("gemm_tc", "gate_up"), ("gemm_tc", "down"),
             ("rmsnorm", None), ("gemm_tc", "head"), ("argmax", None)]
    state, kinds = {}, []
    for kernel, what in order:
        state["tag"] = epi.get(what)
        kinds.append(bench._kind_of(kernel, "", state))
    assert kinds == ["embed", "qkv", "attention", "o_proj", "rmsnorm", "gate_up", "down", "rmsnorm", "qkv", "rope_store",
                     "attention", "o_proj", "rmsnorm", "gate_up", "down", "rmsnorm", "lm_head", "argmax"]
    n = bench.model_numbers(24)
    assert n["kinds"]["qkv"] == 1152 * 896 and n["kinds"]["gate_up"] == 2 * 896 * 4864
    assert sum(n["kinds"][k] for k in ("qkv", "o_proj", "gate_up", "down")) == n["per_layer_params"]
    assert n["kv_bytes_per_token_layer"] * 24 == n["kv_bytes_per_token"]
