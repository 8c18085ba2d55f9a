"""The command-line tools as a user runs them: bin/generate and bin/serve as child processes on the GPU, with
the product's kernels, in 32-bit (tokens equal to the plain implementation's greedy run) and in bfloat16
(equal up to the first token whose margin in the plain implementation is within bfloat16's rounding)."""
import os
import subprocess
import sys

import pytest
import torch

from gpu_util import assert_diverges_only_at_a_close_call
from plain_qwen2 import PlainModel

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_tool(name, argv):
    env = dict(os.environ, PYTHONUNBUFFERED="1")
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bin", name)] + argv, capture_output=True, text=True,
                          timeout=600, env=env)
    assert done.returncode == 0, done.stderr[-2000:]
    return done.stdout


def completions(text):
    return [[int(t) for t in line.split("Completion: ", 1)[1].split()]
            for line in text.splitlines() if line.startswith("Completion: ")]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_tool_on_the_gpu(model_dirs, dtype):
    d, page = model_dirs["A"]
    plain = PlainModel(d)
    prompt = [5, 17, 3, 250, 9]
    want = plain.greedy(prompt, 24)
    for extra in ([], ["--no-cache"]):
        out = run_tool("generate", ["--model-dir", d, "--prompt", " ".join(map(str, prompt)), "--max-tokens", "24",
                                    "--dtype", dtype, "--block-size", str(page), "--num-blocks", "16"] + extra)
        assert f"Prompt: {' '.join(map(str, prompt))}" in out
        (got,) = completions(out)
        assert len(got) == 24
        if dtype == "float32":
            assert got == want, extra
        else:
            assert_diverges_only_at_a_close_call(plain, prompt, got, want, f"generate {extra}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_serve_tool_on_the_gpu(model_dirs, dtype):
    d, page = model_dirs["B"]
    plain = PlainModel(d)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, plain.cfg["vocab"], (n,), generator=g).tolist() for n in (3, 40, 1, 77, 19)]
    argv = ["--model-dir", d, "--max-batch", "3", "--max-tokens", "12", "--dtype", dtype, "--block-size", str(page),
            "--num-blocks", "24", "--max-tokens-per-step", "32"]
    for p in prompts:
        argv += ["--prompt", " ".join(map(str, p))]
    out = run_tool("serve", argv)
    assert "served 5 prompts, max_batch=3" in out and "peak_batch=3" in out
    got = completions(out)
    assert len(got) == 5
    for p, row in zip(prompts, got):
        want = plain.greedy(p, 12)
        if dtype == "float32":
            assert row == want
        else:
            assert_diverges_only_at_a_close_call(plain, p, row, want, "serve")
