"""The replay program's handling of its input and output (steps as JSON lines, ``done`` lines, one file per
step with wanted rows, requests that skip steps, bring nothing or end), run in-process on the CPU: the
engine it builds is given the host backend of the tests instead of the CUDA kernels. The numerics of
replay on the real kernels are covered by the GPU tests."""
import dataclasses
import io
import json
import os
import runpy
import sys

import numpy as np

from plain_qwen2 import PlainModel
from torch_ops import TorchOps

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_trace_run_protocol(model_dirs, tmp_path, monkeypatch, capsys):
    import nanoinfer_b200.engine.engine as engine_module
    d, page = model_dirs["B"]
    real_init = engine_module.Engine.__init__

    def init_on_host(self, model_dir, cfg, ops=None):
        real_init(self, model_dir, dataclasses.replace(cfg, device="cpu"), ops=TorchOps())
    monkeypatch.setattr(engine_module.Engine, "__init__", init_on_host)

    a, b = [5, 17, 3, 9, 11, 7, 400], [1, 2, 3]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:5], "want": [0, 4]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[5:6], "want": [0]}, {"id": "b", "tokens": b[:2], "want": []},
                                {"id": "c", "tokens": [], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[2:], "want": []}], "end": ["c"]},      # a sits this step out
        {"step": 3, "entries": [{"id": "a", "tokens": a[6:], "want": [0]}, {"id": "b", "tokens": [9], "want": [0]}],
         "end": ["a", "b"]},
        {"step": 4, "entries": [], "end": []},
        {"step": 5, "entries": [{"id": "a", "tokens": b, "want": [2]}], "end": ["a"]},         # the id is used again
    ]
    out = tmp_path / "out"
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n\n"))
    monkeypatch.setattr(sys, "argv", ["trace_run", "--model", d, "--dtype", "float32", "--out", str(out),
                                      "--max-tokens", "128", "--page-size", str(page)])
    try:
        runpy.run_path(os.path.join(ROOT, "bin", "trace_run"), run_name="__main__")
    except SystemExit as e:
        assert e.code == 0
    assert capsys.readouterr().out.split("\n")[:6] == [f"done {i}" for i in range(6)]
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "3.f32", "5.f32"]       # nothing was wanted in 2 and 4
    plain = PlainModel(d)
    la, lb, lb9 = plain.logits(a), plain.logits(b), plain.logits(b + [9])

    def rows(step, n):
        return np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(n, -1)
    for got, want in ((rows(0, 2)[0], la[0]), (rows(0, 2)[1], la[4]), (rows(1, 1)[0], la[5]), (rows(3, 2)[0], la[6]),
                      (rows(3, 2)[1], lb9[3]), (rows(5, 1)[0], lb[2])):
        assert np.abs(got - want.numpy()).max() < 1e-4
