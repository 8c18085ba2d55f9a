"""The engine's host-side logic (batch building, cache, step) on the CPU, with every kernel replaced
by its plain PyTorch statement (tests/torch_ops.py): the cutting of requests into steps must not
change the logits."""
import numpy as np
import pytest
import torch

from plain_qwen2 import PlainModel
from torch_ops import TorchOps

from nanoinfer_b200.config import EngineConfig
from nanoinfer_b200.engine import Engine, StepEntry


def make_engine(model_dir, page, num_pages=64, dtype="float32", max_batch=4):
    cfg = EngineConfig(dtype=dtype, page_size=page, num_pages=num_pages, max_batch=max_batch, device="cpu")
    return Engine(model_dir, cfg, ops=TorchOps())


def run_cut(engine, ids, cuts):
    """Feed ``ids`` in portions of the given sizes, wanting every place; returns logits [T, vocab]."""
    rc = engine.open("r")
    out, pos = [], 0
    for n in cuts:
        chunk = ids[pos:pos + n]
        out.append(engine.step([StepEntry(rc, chunk, list(range(len(chunk))))]).double().cpu())
        pos += n
    assert pos == len(ids)
    engine.close(rc)
    engine.cache.check()
    return torch.cat(out)


@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_whole_and_cut_equal_plain(model_dirs, name):
    d, page = model_dirs[name]
    plain = PlainModel(d)
    eng = make_engine(d, page)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, eng.vocab_size, (45,), generator=g).tolist()
    want = plain.logits(ids)
    whole = run_cut(eng, ids, [45])
    assert (whole - want).abs().max().item() < 1e-4
    for cuts in ([13, 32], [40] + [1] * 5, [2, 3, 5, 7, 11, 17], [1] * 45):
        got = run_cut(eng, ids, cuts)
        assert (got - want).abs().max().item() < 1e-4, cuts
    assert eng.cache.num_free(0) == eng.cache.num_pages


def test_mixed_batch_with_page_reuse(model_dirs):
    d, page = model_dirs["B"]
    plain = PlainModel(d)
    eng = make_engine(d, page, num_pages=20)       # 160 positions for up to four live requests
    g = torch.Generator().manual_seed(4)
    prompts = {k: torch.randint(0, eng.vocab_size, (n,), generator=g).tolist()
               for k, n in (("a", 37), ("b", 50), ("c", 21), ("d", 44), ("e", 30))}
    want = {k: plain.logits(v) for k, v in prompts.items()}
    got = {k: [] for k in prompts}
    fed = {k: 0 for k in prompts}
    live = {}
    waiting = list(prompts)
    chunk = {"a": 13, "b": 7, "c": 2, "d": 16, "e": 5}
    rounds = 0
    while waiting or live:
        rounds += 1
        while waiting and len(live) < 4:
            k = waiting[0]
            need = -(-len(prompts[k]) // page)
            held = sum(-(-len(prompts[j]) // page) for j in live)
            if held + need > 20:
                break
            live[waiting.pop(0)] = eng.open(k)
        entries, keys = [], []
        for k, rc in live.items():
            n = chunk[k] if fed[k] < len(prompts[k]) - 8 else 1
            toks = prompts[k][fed[k]:fed[k] + n]
            entries.append(StepEntry(rc, toks, list(range(len(toks)))))
            keys.append((k, len(toks)))
        logits = eng.step(entries).double().cpu()
        row = 0
        for k, n in keys:
            got[k].append(logits[row:row + n])
            row += n
            fed[k] += n
        for k in [k for k in live if fed[k] == len(prompts[k])]:
            eng.close(live.pop(k))
        eng.cache.check()
    for k in prompts:
        assert (torch.cat(got[k]) - want[k]).abs().max().item() < 1e-4, k
    assert eng.cache.num_free(0) == 20


def test_step_errors(model_dirs):
    from nanoinfer_b200.cache import OutOfPages
    d, page = model_dirs["A"]
    eng = make_engine(d, page, num_pages=2)
    rc = eng.open("x")
    with pytest.raises(ValueError):
        eng.step([StepEntry(rc, [], [])])
    with pytest.raises(ValueError):
        eng.step([StepEntry(rc, [999], [0])])
    with pytest.raises(ValueError):
        eng.step([StepEntry(rc, [1, 2], [2])])
    with pytest.raises(OutOfPages):
        eng.step([StepEntry(rc, list(range(40)), [])])
    assert rc.length == 0 and eng.cache.num_free(0) == 2
    assert eng.step([StepEntry(rc, list(range(32)), [])]) is None
    with pytest.raises(OutOfPages):
        eng.step([StepEntry(rc, [1], [0])])
    eng.close(rc)
    eng.cache.check()
