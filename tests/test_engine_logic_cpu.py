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
    # ids that are no ids, alone (a decoded token takes a path of its own) and inside a portion
    for bad in (-1, 256, 2 ** 40, 1.5, "7", None, True):
        with pytest.raises(ValueError, match="outside the vocabulary"):
            eng.step([StepEntry(rc, [bad], [0])])
        if bad is not True:         # (beside integers numpy reads it as 1, as Python does)
            with pytest.raises(ValueError, match="outside the vocabulary"):
                eng.step([StepEntry(rc, [3, bad, 5], [0])])
    assert rc.length == 0 and eng.cache.num_free(0) == 2
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


@pytest.mark.parametrize("name", ["B", "W"])
def test_graph_input_mirror_equals_the_built_context(model_dirs, name):
    """A captured decode graph reads its inputs from a buffer that a host mirror refreshes row by row. Whatever
    happens to the rows (requests decode on, one ends and the others move up, a new one takes the first
    row, the batch shrinks and grows, a window gives pages back), the mirror must hold exactly what
    ``Engine.build_context`` builds for the same padded batch."""
    from nanoinfer_b200.engine.graphs import _InputMirror
    d, page = model_dirs[name]
    eng = make_engine(d, page, num_pages=96)
    vocab = PlainModel(d).cfg["vocab"]
    rng = np.random.default_rng(5)
    rb, widths = 4, [16 for _ in eng.cache.groups]
    mirror = _InputMirror(rb, widths, torch.device("cpu"), eng.storage.pad_slot)
    assert eng.storage.pad_slot == eng.cache.max_requests      # the spare slot that no request is ever given
    static = torch.empty(mirror.size, dtype=torch.int32)
    live = {}

    def prompt(k, n):
        live[k] = eng.open(k)
        eng.step([StepEntry(live[k], rng.integers(0, vocab, n).tolist(), [])])

    def decode(order, steps):
        for _ in range(steps):
            entries = [StepEntry(live[k], [int(rng.integers(0, vocab))], [0]) for k in order]
            for e in entries:                        # what Engine.step does before it builds the inputs
                eng.cache.extend(e.request, 1)
            eng.build_context(entries, pad_to=rb, widths=widths, static=static)
            mirror.fill(entries)
            assert torch.equal(mirror.host, static), f"{name}: rows {order}"
            for e in entries:
                eng.cache.commit(e.request, 1)

    prompt("a", 30); prompt("b", 7); prompt("c", 19)
    decode("abc", 20)
    eng.close(live.pop("a"))
    decode("bc", 6)
    prompt("d", 3)
    decode("dbc", 30)               # W: the window passes whole pages here and their entries become -1
    decode("c", 5)
    decode("cbd", 10)
    for rc in live.values():
        eng.close(rc)
    eng.cache.check()


@pytest.mark.parametrize("name,seed", [("A", 0), ("B", 1), ("W", 2), ("B", 3), ("W", 4), ("A", 5)])
def test_random_traces_equal_plain(model_dirs, name, seed):
    """Seeded random traces: up to four live requests, each step a random subset of them (a request may sit
    a step out) with random portions from one token up, random wanted places, and a pool that only just
    holds the live requests so that pages change hands. Every wanted row equals the plain model's."""
    import random
    rnd = random.Random(77 + seed)
    d, page = model_dirs[name]
    plain = PlainModel(d)
    eng_probe = make_engine(d, page, num_pages=4)
    vocab = eng_probe.vocab_size
    g = torch.Generator().manual_seed(100 + seed)
    lengths = [rnd.randint(1, 70) for _ in range(7)]
    prompts = {f"q{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    want = {k: plain.logits(v) for k, v in prompts.items()}
    pages_of = {k: -(-len(v) // page) for k, v in prompts.items()}
    top4 = sum(sorted(pages_of.values())[-4:])
    num_pages = max(max(pages_of.values()), top4 - rnd.randint(0, top4 // 3))
    eng = make_engine(d, page, num_pages=num_pages)
    fed = {k: 0 for k in prompts}
    live, waiting = {}, list(prompts)
    worst = 0.0
    steps = 0
    while waiting or live:
        steps += 1
        assert steps < 5000
        while waiting and len(live) < 4:
            k = waiting[0]
            if sum(pages_of[j] for j in live) + pages_of[k] > num_pages:
                break
            live[waiting.pop(0)] = eng.open(k)
        chosen = [k for k in live if rnd.random() < 0.8] or [next(iter(live))]
        entries, keys = [], []
        for k in chosen:
            left = len(prompts[k]) - fed[k]
            n = min(left, rnd.choice([1, 1, 2, 3, 7, 16, 29]))
            places = sorted(rnd.sample(range(n), rnd.randint(0, n)))
            entries.append(StepEntry(live[k], prompts[k][fed[k]:fed[k] + n], places))
            keys.append((k, fed[k], places))
            fed[k] += n
        logits = eng.step(entries)
        row = 0
        for k, start, places in keys:
            for p in places:
                worst = max(worst, (logits[row].double().cpu() - want[k][start + p]).abs().max().item())
                row += 1
        assert (0 if logits is None else logits.shape[0]) == row
        for k in [k for k in live if fed[k] == len(prompts[k])]:
            eng.close(live.pop(k))
        eng.cache.check()
    assert worst < 1e-4, worst
    assert eng.cache.num_free(0) == num_pages


def test_decoded_tokens_are_laid_out_first_whatever_the_callers_order(model_dirs):
    """A step's rows begin with the entries of one token (the attention sends the leading one-token requests to its
    decode kernel), in whatever order the caller names the entries; the logits come back in the caller's order."""
    d, page = model_dirs["A"]
    plain = PlainModel(d)
    eng = make_engine(d, page)
    g = torch.Generator().manual_seed(9)
    ids = {k: torch.randint(0, eng.vocab_size, (n,), generator=g).tolist() for k, n in (("a", 30), ("b", 12), ("c", 41))}
    want = {k: plain.logits(v) for k, v in ids.items()}
    reqs = {k: eng.open(k) for k in ids}
    eng.step([StepEntry(reqs["a"], ids["a"][:20], []), StepEntry(reqs["c"], ids["c"][:7], [])])
    # a: one decoded token; b: its whole prompt; c: a portion. Named portion first, decoded token in the middle.
    entries = [StepEntry(reqs["b"], ids["b"], [0, 11]), StepEntry(reqs["a"], [ids["a"][20]], [0]),
               StepEntry(reqs["c"], ids["c"][7:30], [22, 0])]
    ctx, want_rows, want_list = eng.build_context(entries)
    assert ctx.host.q_lens == [1, 12, 23] and want_list == [1, 12, 0, 13 + 22, 13]
    logits = eng.step(entries).double().cpu()
    ref = torch.stack([want["b"][0], want["b"][11], want["a"][20], want["c"][29], want["c"][7]])
    assert (logits - ref).abs().max().item() < 1e-4
    for rc in reqs.values():
        eng.close(rc)
    eng.cache.check()
