"""The scheduler's decisions, and its results against generation alone, on the CPU with the kernels
replaced by their plain PyTorch statements."""
import pytest
import torch

from plain_qwen2 import PlainModel
from torch_ops import TorchOps

from nanoinfer_b200 import Model, Request, SamplingParams, Scheduler
from nanoinfer_b200.config import EngineConfig


def make_model(model_dir, page, num_pages=64, max_batch=4, budget=64):
    cfg = EngineConfig(dtype="float32", page_size=page, num_pages=num_pages, max_batch=max_batch,
                       max_tokens_per_step=budget, device="cpu")
    return Model(model_dir, cfg, ops=TorchOps())


def prompts(vocab, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def test_greedy_equals_plain_full_recompute(model_dirs):
    d, page = model_dirs["A"]
    model = make_model(d, page)
    plain = PlainModel(d)
    for p in prompts(256, [1, 7, 33]):
        assert model.generate(p, max_tokens=16) == plain.greedy(p, 16)
    assert model.engine.cache.num_free() == 64
    model.engine.cache.check()


def test_budget_cuts_prompts_and_decodes_come_first(model_dirs):
    d, page = model_dirs["A"]
    model = make_model(d, page, budget=10, max_batch=3)
    s = Scheduler(model)
    a, b = prompts(256, [25, 8], seed=1)
    s.add(Request("a", a, max_tokens=4))
    plan = s.step()
    assert [(e.seq.req.request_id, e.start, e.count, e.samples) for e in plan.entries] == [("a", 0, 10, False)]
    s.add(Request("b", b, max_tokens=4))
    plan = s.step()      # a goes on with its prompt; nothing is left for b
    assert [(e.seq.req.request_id, e.start, e.count) for e in plan.entries] == [("a", 10, 10)]
    plan = s.step()      # a's last 5 prompt tokens -> first token; b gets the other 5
    assert [(e.seq.req.request_id, e.start, e.count, e.samples) for e in plan.entries] == \
        [("a", 20, 5, True), ("b", 0, 5, False)]
    plan = s.step()      # a decodes (first in the batch), b finishes its prompt
    assert [(e.seq.req.request_id, e.count, e.samples) for e in plan.entries] == [("a", 1, True), ("b", 3, True)]
    out = s.run()
    assert len(out["a"]) == 4 and len(out["b"]) == 4
    st = s.stats()      # four steps carried a prompt's portion: 10, 10, 10 and 4 tokens of a budget of 10
    assert (st["prompt_steps"], st["peak_step_tokens"], st["peak_batch"]) == (4, 10, 2)
    assert st["budget_use"] == pytest.approx(34 / 40)
    assert st["tokens_run"] == 25 + 8 + 3 + 3 and st["tokens_per_step"] == pytest.approx(st["tokens_run"] / st["steps"])
    plain = PlainModel(d)
    assert out["a"] == plain.greedy(a, 4) and out["b"] == plain.greedy(b, 4)


def test_continuous_batching_equals_alone_and_frees_everything(model_dirs):
    d, page = model_dirs["B"]
    plain = PlainModel(d)
    ps = prompts(503, [2, 9, 17, 64, 100], seed=2)
    alone = [plain.greedy(p, 6) for p in ps]
    for budget, max_batch, num_pages in ((13, 3, 40), (64, 5, 40), (5, 2, 16)):
        model = make_model(d, page, num_pages=num_pages, max_batch=max_batch, budget=budget)
        s = Scheduler(model)
        for i, p in enumerate(ps):
            s.add(Request(f"r{i}", p, max_tokens=6))
        out = s.run()
        assert [out[f"r{i}"] for i in range(5)] == alone, (budget, max_batch)
        assert s.peak_batch <= max_batch
        model.engine.cache.check()
        assert model.engine.cache.num_free() == num_pages and not model.engine.cache.live


def test_when_pages_run_out_the_last_admitted_is_preempted_and_recomputed(model_dirs):
    d, page = model_dirs["B"]             # page 8
    plain = PlainModel(d)
    ps = prompts(503, [30, 30, 30], seed=3)
    # 14 pages = 112 positions: three prompts of 30 are admitted (4 pages each + watermark), but their
    # 20 decoded tokens each (3 more pages each) cannot all be held.
    model = make_model(d, page, num_pages=14, max_batch=3, budget=64)
    s = Scheduler(model)
    for i, p in enumerate(ps):
        s.add(Request(f"r{i}", p, max_tokens=20))
    preempted = []
    while s.has_work():
        plan = s.step()
        preempted += [v.req.request_id for v in plan.preempted]
        model.engine.cache.check()
    assert preempted and set(preempted) <= {"r1", "r2"} and "r0" not in preempted
    for i, p in enumerate(ps):
        assert s.finished[f"r{i}"] == plain.greedy(p, 20)
    assert model.engine.cache.num_free() == 14


def test_admission_errors_and_edge_cases(model_dirs):
    d, page = model_dirs["A"]
    model = make_model(d, page, num_pages=4)
    s = Scheduler(model)
    with pytest.raises(ValueError, match="pages"):
        s.add(Request("big", list(range(60)), max_tokens=10))
    with pytest.raises(ValueError):
        s.add(Request("bad", [1], temperature=-1.0))
    s.add(Request("empty", [], max_tokens=5))
    s.add(Request("none", [1, 2, 3], max_tokens=0))
    out = s.run()
    assert out["empty"] == [] and out["none"] == []
    assert model.engine.cache.num_free() == 4


def test_lookahead_equals_alone_under_every_interruption(model_dirs):
    """Lookahead decoding (the next step starts from the device's copy of the last tokens): requests of
    different lengths that finish by count at different steps, one that stops at EOS, a tight pool that
    preempts, late arrivals, a cancel: the outputs equal generation alone, and nothing is left held."""
    d, page = model_dirs["B"]
    plain = PlainModel(d)
    ps = prompts(503, [2, 9, 17, 30, 5], seed=6)
    limits = [9, 4, 12, 7, 10]
    alone = [plain.greedy(p, n) for p, n in zip(ps, limits)]
    eos = alone[2][5]
    stop = alone[2].index(eos)
    for budget, max_batch, num_pages in ((64, 5, 40), (13, 3, 40), (16, 4, 12)):
        model = make_model(d, page, num_pages=num_pages, max_batch=max_batch, budget=budget)
        s = Scheduler(model, lookahead=True)
        for i in range(3):
            s.add(Request(f"r{i}", ps[i], max_tokens=limits[i], eos_id=eos if i == 2 else -1))
        for _ in range(5):
            s.step()
        for i in range(3, 5):
            s.add(Request(f"r{i}", ps[i], max_tokens=limits[i]))
        for _ in range(4):
            s.step()
        assert s.cancel("r4")
        out = s.run()
        assert s._inflight is None and s.steps_ahead > 0
        assert out["r0"] == alone[0] and out["r1"] == alone[1] and out["r3"] == alone[3], (budget, max_batch)
        assert out["r2"] == alone[2][:stop]
        assert out["r4"] == alone[4][:len(out["r4"])] and len(out["r4"]) < limits[4]
        model.engine.cache.check()
        assert model.engine.cache.num_free() == num_pages and not model.engine.cache.live


def test_eos_ends_generation_and_is_not_emitted(model_dirs):
    d, page = model_dirs["B"]
    model = make_model(d, page)
    p = prompts(503, [5], seed=4)[0]
    first = PlainModel(d).greedy(p, 12)
    k = next(i for i in range(1, 12) if first[i] not in first[:i])    # the first new token after the first
    assert model.generate(p, max_tokens=12, eos_id=first[k]) == first[:k]
    assert model.generate(p, max_tokens=12, eos_id=first[0]) == []


def test_cancel(model_dirs):
    d, page = model_dirs["A"]
    model = make_model(d, page, max_batch=1)
    s = Scheduler(model)
    s.add(Request("x", [1, 2, 3], max_tokens=50))
    s.add(Request("y", [4, 5], max_tokens=50))
    for _ in range(4):
        s.step()
    assert s.cancel("y") and s.finished["y"] == []
    assert s.cancel("x") and len(s.finished["x"]) == 4
    assert not s.cancel("x") and not s.has_work()
    assert model.engine.cache.num_free() == 64


def test_sampling_is_reproducible_and_independent_of_the_batch(model_dirs):
    d, page = model_dirs["B"]
    ps = prompts(503, [9, 17, 40], seed=5)
    def run(max_batch, budget, lookahead=False):
        model = make_model(d, page, max_batch=max_batch, budget=budget)
        s = Scheduler(model, lookahead=lookahead)
        for i, p in enumerate(ps):
            s.add(Request(f"r{i}", p, max_tokens=12, temperature=0.7, seed=11 + i, top_k=50, top_p=0.9))
        out = s.run()
        assert (s.steps_ahead > 0) == (lookahead and max_batch > 1)
        return out
    a, b = run(1, 64), run(3, 7)
    assert a == b
    assert run(3, 64, lookahead=True) == a       # the draw's counter is the same when the step starts early
    model = make_model(d, page)
    alone = model.generate(ps[1], max_tokens=12, params=SamplingParams(temperature=0.7, top_k=50, top_p=0.9, seed=12))
    assert alone == a["r1"]
    other = model.generate(ps[1], max_tokens=12, params=SamplingParams(temperature=0.7, top_k=50, top_p=0.9, seed=13))
    assert other != alone


def test_greedy_sampled_and_penalised_requests_share_steps_ahead(model_dirs):
    """A batch that holds greedy and sampled requests, with and without a repetition penalty, is decoded ahead like
    any other (one sampling launch takes both kinds; the id that the host has not read yet is penalised from the
    device's copy): every request's tokens equal what it generates alone, one step at a time."""
    d, page = model_dirs["A"]
    ps = prompts(256, [5, 12, 21, 8, 30, 3], seed=8)
    kinds = [SamplingParams(), SamplingParams(temperature=0.9, top_k=20, seed=3), SamplingParams(),
             SamplingParams(temperature=1.2, top_p=0.85, seed=4), SamplingParams(repetition_penalty=40.0),
             SamplingParams(temperature=0.8, repetition_penalty=1.4, seed=5)]

    def requests():
        return [Request(f"r{i}", p, max_tokens=14, temperature=k.temperature, top_k=k.k, top_p=k.p,
                        repetition_penalty=k.repetition_penalty, seed=k.seed or 0) for i, (p, k) in enumerate(zip(ps, kinds))]
    alone = []
    for r in requests():
        s = Scheduler(make_model(d, page), lookahead=False)
        s.add(r)
        alone.append(s.run()[r.request_id])
        assert s.steps_ahead == 0
    plain = PlainModel(d)
    assert alone[0] == plain.greedy(ps[0], 14)
    assert alone[4] != plain.greedy(ps[4], 14)          # the penalty does something here
    s = Scheduler(make_model(d, page, max_batch=6), lookahead=True)
    for r in requests():
        s.add(r)
    out = s.run()
    assert s.steps_ahead >= 10
    assert [out[f"r{i}"] for i in range(6)] == alone


def test_prompt_portions_are_views_of_one_array(model_dirs):
    import numpy as np
    from nanoinfer_b200.engine.scheduler import Sequence
    seq = Sequence(Request("x", list(range(40)), max_tokens=8), 0)
    a, b = seq.tokens(0, 16), seq.tokens(16, 24)
    assert a.dtype == np.int32 and a.base is b.base and a.tolist() == list(range(16)) and b.tolist() == list(range(16, 40))
    seq.emit(7)
    assert seq.tokens(38, 3) == [38, 39, 7] and seq.tokens(40, 1) == [7] and seq.tokens(39, 1) == [39]
    # a prompt that holds something else than integers stays a list, and the step names the id
    d, page = model_dirs["A"]
    s = Scheduler(make_model(d, page))
    s.add(Request("bad", [5, 6.5, 7], max_tokens=2))
    with pytest.raises(ValueError, match="6.5"):
        s.step()


def test_a_sequence_keeps_its_distinct_ids_up_to_date():
    from nanoinfer_b200.engine.scheduler import Sequence
    seq = Sequence(Request("x", [5, 3, 5, 9] * 40, max_tokens=200, repetition_penalty=1.2), 0)
    assert seq.distinct_ids().tolist() == [5, 3, 9]
    for tok in [3, 70, 5, 71] + list(range(100, 200)):
        seq.emit(tok)
    assert seq.distinct_ids().tolist() == [5, 3, 9, 70, 71] + list(range(100, 200))
    row = seq.sample_row(7)
    assert row.distinct and row.context.tolist() == seq.distinct_ids().tolist() and row.generated == 7


@pytest.mark.parametrize("seed", range(8))
def test_random_arrivals_cancels_and_tight_pools(model_dirs, seed):
    """A seeded random run: requests arrive at random steps, some are cancelled at random steps, the pool,
    the batch and the token budget are drawn small enough that prompts are cut and requests preempted,
    with and without lookahead. Whatever happens, every output is generation alone (cut short where the
    request was cancelled), the manager's books balance after every step and nothing stays held."""
    import random
    rnd = random.Random(1000 + seed)
    name = "B" if seed % 2 else "A"
    d, page = model_dirs[name]
    vocab = 503 if name == "B" else 256
    plain = PlainModel(d)
    n_req = rnd.randint(5, 8)
    lengths = [rnd.choice([1, 2, 3, 5, 9, 17, 26, 33]) for _ in range(n_req)]
    limits = [rnd.randint(1, 12) for _ in range(n_req)]
    ps = prompts(vocab, lengths, seed=50 + seed)
    alone = [plain.greedy(p, n) for p, n in zip(ps, limits)]
    largest = max(-(-(l + n) // page) for l, n in zip(lengths, limits))
    num_pages = largest + rnd.randint(1, 2 * largest)          # the largest request fits; not all of them
    max_batch = rnd.randint(1, 4)
    budget = max(max_batch, rnd.choice([2, 5, 13, 64]))      # at least one token for each decoding request
    model = make_model(d, page, num_pages=num_pages, max_batch=max_batch, budget=budget)
    s = Scheduler(model, lookahead=bool(seed & 2))
    arrive = sorted((rnd.randint(0, 25), i) for i in range(n_req))
    cancel_at = {i: rnd.randint(1, 40) for i in range(n_req) if rnd.random() < 0.3}
    cancelled = set()
    step = 0
    while arrive or s.has_work():
        while arrive and arrive[0][0] <= step:
            _, i = arrive.pop(0)
            s.add(Request(f"r{i}", ps[i], max_tokens=limits[i]))
        for i, at in cancel_at.items():
            if at == step and s.cancel(f"r{i}"):
                cancelled.add(i)
        if s.has_work():
            s.step()
        model.engine.cache.check()
        step += 1
        assert step < 2000, "the scheduler makes no progress"
    for i in range(n_req):
        out = s.finished[f"r{i}"]
        if i in cancelled:
            assert out == alone[i][:len(out)], (seed, i)
        else:
            assert out == alone[i], (seed, i, name, num_pages, max_batch, budget)
    assert s._inflight is None
    assert model.engine.cache.num_free() == num_pages and not model.engine.cache.live


def test_generation_without_the_cache_gives_the_same_tokens(model_dirs):
    """``use_cache=False`` (the reference's --no-cache) recomputes the whole sequence for every token, in
    portions under the token budget; greedy, sampled and penalised generation equal the cached way, and
    no page stays held."""
    d, page = model_dirs["B"]
    model = make_model(d, page, num_pages=40, budget=16)
    p = prompts(503, [23], seed=9)[0]
    for params in (SamplingParams(), SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=5),
                   SamplingParams(repetition_penalty=1.3)):
        cached = model.generate(p, max_tokens=7, params=params)
        assert len(cached) == 7
        assert model.generate(p, max_tokens=7, params=params, use_cache=False) == cached
    eos = model.generate(p, max_tokens=7)[3]
    stop = model.generate(p, max_tokens=7).index(eos)
    assert model.generate(p, max_tokens=7, eos_id=eos, use_cache=False) == model.generate(p, max_tokens=7)[:stop]
    assert model.generate([], max_tokens=3, use_cache=False) == []
    assert model.engine.cache.num_free() == 40 and not model.engine.cache.live


def test_sampled_workload_of_the_second_tiny_configuration(model_dirs):
    """Five prompts of 2, 9, 17, 64 and 100 ids, 24 tokens each at temperature 0.7 with a fixed seed, prompts
    cut into portions of 13 beside the other requests' decoded tokens: every request's tokens equal a plain
    loop of its own (whole-sequence logits, the sampling distribution of the plain implementation, the
    draw's uniform number from (seed, tokens generated), inverse CDF in vocabulary order)."""
    import numpy as np
    from plain_qwen2 import sampling_distribution
    from nanoinfer_b200.sampling.sampler import uniform_for
    d, page = model_dirs["B"]
    plain = PlainModel(d)
    ps = prompts(503, [2, 9, 17, 64, 100], seed=21)

    def plain_sampled(prompt, n, seed):
        ids, out = list(prompt), []
        for step in range(n):
            probs = sampling_distribution(plain.logits(ids)[-1].numpy(), ids, 0.7)
            cdf = np.cumsum(probs)
            tok = int(np.searchsorted(cdf, uniform_for(seed, step) * cdf[-1], side="right"))
            out.append(tok)
            ids.append(tok)
        return out

    want = [plain_sampled(p, 24, 100 + i) for i, p in enumerate(ps)]
    for lookahead in (False, True):
        model = make_model(d, page, num_pages=80, max_batch=5, budget=13)
        s = Scheduler(model, lookahead=lookahead)
        for i, p in enumerate(ps):
            s.add(Request(f"r{i}", p, max_tokens=24, temperature=0.7, seed=100 + i))
        out = s.run()
        assert [out[f"r{i}"] for i in range(5)] == want, lookahead
        assert model.engine.cache.num_free() == 80
