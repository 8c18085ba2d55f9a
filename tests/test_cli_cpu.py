"""The command-line tools (options with the reference's names, what they print, what they refuse), run
in-process on the CPU: the engine they build is given the host backend of the tests instead of the CUDA
kernels. Prompts are token ids, as they are for a model folder without a tokenizer."""
import dataclasses
import json

import pytest

from plain_qwen2 import PlainModel
from tiny_configs import TINY_A
from torch_ops import TorchOps


@pytest.fixture()
def host_engine(monkeypatch):
    import nanoinfer_b200.engine.engine as engine_module
    real_init = engine_module.Engine.__init__

    def init_on_host(self, model_dir, cfg, ops=None):
        real_init(self, model_dir, dataclasses.replace(cfg, device="cpu", dtype="float32"), ops=TorchOps())
    monkeypatch.setattr(engine_module.Engine, "__init__", init_on_host)


def completions(text):
    return [line.split("Completion: ", 1)[1] for line in text.splitlines() if line.startswith("Completion: ")]


def test_generate_cli(model_dirs, host_engine, capsys):
    from nanoinfer_b200.cli import generate
    d, page = model_dirs["A"]
    plain = PlainModel(d)
    want = " ".join(map(str, plain.greedy([5, 17, 3], 9)))
    for extra in ([], ["--no-cache"], ["--weights-dir", d], ["--model", d]):
        argv = ["--prompt", "5 17 3", "--max-tokens", "9", "--block-size", str(page), "--num-blocks", "16"]
        argv += extra if extra and extra[0] != "--no-cache" else ["--model-dir", d] + extra
        assert generate.main(argv) == 0
        out = capsys.readouterr().out
        assert "Prompt: 5 17 3" in out and completions(out) == [want], extra
    # sampling options are taken and reproducible under a seed
    argv = ["--model-dir", d, "--prompt", "5,17,3", "--max-tokens", "9", "--temperature", "0.9", "--top-k", "40",
            "--top-p", "0.95", "--repetition-penalty", "1.1", "--seed", "7", "--num-blocks", "16"]
    generate.main(argv)
    first = completions(capsys.readouterr().out)
    generate.main(argv)
    assert completions(capsys.readouterr().out) == first and len(first[0].split()) == 9


def test_generate_cli_writes_random_weights_and_refuses_what_it_cannot_do(tmp_path, host_engine, capsys, monkeypatch):
    import tempfile
    from nanoinfer_b200.cli import generate
    monkeypatch.setattr(tempfile, "tempdir", str(tmp_path))      # the model folder it writes goes away with the test
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    assert generate.main(["--random-weights", str(cfg), "--prompt", "1 2", "--max-tokens", "3", "--seed", "3",
                          "--num-blocks", "8"]) == 0
    captured = capsys.readouterr()
    assert len(completions(captured.out)[0].split()) == 3 and "random-weights model" in captured.err
    with pytest.raises(SystemExit, match="no CPU path"):
        generate.main(["--model-dir", str(tmp_path), "--device", "cpu", "--prompt", "1"])
    with pytest.raises(SystemExit, match="not a folder"):
        generate.main(["--model", "Qwen/Qwen2.5-0.5B", "--prompt", "1"])
    with pytest.raises(SystemExit, match="--model-dir DIR or --random-weights"):
        generate.main(["--prompt", "1"])


def test_serve_cli(model_dirs, host_engine, capsys):
    from nanoinfer_b200.cli import serve
    d, page = model_dirs["A"]
    plain = PlainModel(d)
    prompts = ["5 17 3", "9", "200 100 50 25 12 6 3"]
    argv = ["--model-dir", d, "--max-batch", "2", "--max-tokens", "6", "--block-size", str(page), "--num-blocks", "12"]
    for p in prompts:
        argv += ["--prompt", p]
    assert serve.main(argv) == 0
    out = capsys.readouterr().out
    assert "served 3 prompts, max_batch=2" in out and "peak_batch=2" in out and "18 tokens" in out
    assert "tokens a step, at most " in out and "% of the budget of " in out and "MiB in 32-bit" in out
    want = [" ".join(map(str, plain.greedy([int(t) for t in p.split()], 6))) for p in prompts]
    assert completions(out) == want
    assert [line for line in out.splitlines() if line.startswith("Prompt: ")] == [f"Prompt: {p}" for p in prompts]


def test_text_prompts_with_a_tokenizer_file_and_ids_without(model_dirs, host_engine, capsys, tmp_path):
    """With ``tokenizer.json`` in the model folder prompts and completions are text; without it a prompt that
    is no list of ids is refused in one line."""
    import shutil
    from tokenizers import Tokenizer, models, pre_tokenizers
    from nanoinfer_b200.cli import generate, serve
    d, page = model_dirs["A"]
    with pytest.raises(SystemExit, match="list of token ids"):
        generate.main(["--model-dir", d, "--prompt", "the cat", "--num-blocks", "8"])
    with pytest.raises(SystemExit, match="list of token ids"):
        serve.main(["--model-dir", d, "--prompt", "1 2", "--prompt", "the cat", "--num-blocks", "8"])
    capsys.readouterr()
    folder = tmp_path / "with_tokenizer"
    shutil.copytree(d, folder)
    vocab = {f"w{i}": i for i in range(256)}
    vocab.update({"the": 5, "cat": 17, "sat": 3})
    del vocab["w5"], vocab["w17"], vocab["w3"]
    tok = Tokenizer(models.WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(folder / "tokenizer.json"))
    assert generate.main(["--model-dir", str(folder), "--prompt", "the cat sat", "--max-tokens", "5",
                          "--block-size", str(page), "--num-blocks", "8"]) == 0
    words = completions(capsys.readouterr().out)[0].split()
    by_id = {i: w for w, i in vocab.items()}
    assert words == [by_id[t] for t in PlainModel(d).greedy([5, 17, 3], 5)]
