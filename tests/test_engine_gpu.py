"""The engine on the GPU, in-process: long decoding, the first tokens of a sequence, greedy generation
through the entry point, continuous batching against generation alone, and each part alone against the
plain implementation's function for it. In 32-bit and in bfloat16."""

import dataclasses

import pytest
import torch

from gpu_util import assert_close
from plain_qwen2 import PlainModel, apply_rope, causal_attention_fast, linear, rms_norm, rope_tables, swiglu

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def engine_for(model_dir, page, dtype, num_pages=128, max_batch=4, **kw):
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine
    return Engine(model_dir, EngineConfig(dtype=dtype, page_size=page, num_pages=num_pages, max_batch=max_batch, **kw))


def tdt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "W", "C"])
def test_long_decoding_token_by_token(model_dirs, name, dtype):
    from nanoinfer_b200.engine import StepEntry
    d, page = model_dirs[name]
    plain = PlainModel(d)
    n = min(plain.cfg["max_pos"], 400)
    ids = torch.randint(0, plain.cfg["vocab"], (n,), generator=torch.Generator().manual_seed(1)).tolist()
    want = plain.logits(ids)
    eng = engine_for(d, page, dtype)
    rc = eng.open("long")
    rows = [eng.step([StepEntry(rc, [t], [0])])[0].clone() for t in ids]
    got = torch.stack(rows)
    assert_close(got, want, tdt(dtype), f"long decode {name}")
    eng.close(rc)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(model_dirs, dtype):
    """Positions 0, 1, 2: one visible key, then two, then three; alone and as a three-token portion."""
    from nanoinfer_b200.engine import StepEntry
    d, page = model_dirs["B"]
    plain = PlainModel(d)
    eng = engine_for(d, page, dtype)
    for ids in ([7], [7, 300], [7, 300, 12]):
        want = plain.logits(ids)
        rc = eng.open("f")
        got = eng.step([StepEntry(rc, ids, list(range(len(ids))))])
        assert_close(got, want, tdt(dtype), f"first tokens {ids}")
        eng.close(rc)
        rc = eng.open("f")
        got = torch.cat([eng.step([StepEntry(rc, [t], [0])]) for t in ids])
        assert_close(got, want, tdt(dtype), f"first tokens one by one {ids}")
        eng.close(rc)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(model_dirs, name, dtype):
    from nanoinfer_b200 import load_model
    d, page = model_dirs[name]
    plain = PlainModel(d)
    model = load_model(d, dtype=dtype, page_size=page, num_pages=64, max_batch=2)
    g = torch.Generator().manual_seed(2)
    for n in (1, 7, 33):
        prompt = torch.randint(0, plain.cfg["vocab"], (n,), generator=g).tolist()
        got = model.generate(prompt, max_tokens=16)
        # follow the engine's own tokens with the plain model: at every step the chosen token must be the
        # plain argmax, or (bfloat16 only) within the rounding of it
        ids = list(prompt)
        for tok in got:
            ref = plain.logits(ids)[-1]
            if dtype == "float32":
                assert tok == int(ref.argmax()), (n, ids)
            else:
                assert ref[tok] >= ref.max() - 0.06 * ref.pow(2).mean().sqrt(), (n, ids)
            ids.append(tok)
        assert len(got) == 16
    assert model.engine.cache.num_free() == 64


@pytest.mark.parametrize("dtype", DTYPES)
def test_scheduler_equals_alone_with_few_pages(model_dirs, dtype):
    """Six staggered requests under a small token budget and a pool that forces queueing, reuse of pages
    and preemption: every output equals generation alone (cpp/tests/python/run_serve.py:44-69 is the
    reference's form of this test)."""
    from nanoinfer_b200 import Request, Scheduler, load_model
    d, page = model_dirs["B"]
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 503, (n,), generator=g).tolist() for n in (30, 9, 30, 64, 2, 30)]
    model = load_model(d, dtype=dtype, page_size=page, num_pages=14, max_batch=3, max_tokens_per_step=24)
    alone = [model.generate(p, max_tokens=20) for p in prompts]
    sched = Scheduler(model)
    for i, p in enumerate(prompts[:3]):
        sched.add(Request(f"r{i}", p, max_tokens=20))
    for _ in range(3):
        sched.step()
    for i, p in enumerate(prompts[3:], start=3):
        sched.add(Request(f"r{i}", p, max_tokens=20))
    out = sched.run()
    if dtype == "float32":
        assert [out[f"r{i}"] for i in range(6)] == alone
    else:
        # bfloat16 rounds differently in different batches, so a near tie may turn another way and the
        # continuation then differs. What must hold: every token emitted is, under the plain model fed
        # the same tokens, within twice the element tolerance of the best one.
        from gpu_util import assert_diverges_only_at_a_close_call, bf16_slack
        plain = PlainModel(d)
        for i, p in enumerate(prompts):
            for got in (out[f"r{i}"], alone[i]):
                assert len(got) == 20
                ref = plain.logits(p + got).double()
                for j, tok in enumerate(got):
                    row = ref[len(p) + j - 1]
                    assert row.max().item() - row[tok].item() <= bf16_slack(row), f"request {i} token {j}: not the best within rounding"
            # and the batched run leaves the lone run only where the plain model's best two are within rounding
            assert_diverges_only_at_a_close_call(plain, p, out[f"r{i}"], alone[i], f"request {i}")
    assert sched.preemptions > 0
    model.engine.cache.check()
    assert model.engine.cache.num_free() == 14


@pytest.mark.parametrize("dtype", DTYPES)
def test_lookahead_scheduling_generates_the_same(model_dirs, dtype):
    """With ``lookahead`` the next decode step starts from the tokens on the device while the host still
    reads the previous ones. Requests of different lengths, one that stops at an EOS token in the middle
    (it has run one step too many by then: that token is dropped), a late arrival that interrupts the
    pipeline, few pages: the outputs equal those of the plain scheduler."""
    from nanoinfer_b200 import Request, Scheduler, load_model
    d, page = model_dirs["B"]
    g = torch.Generator().manual_seed(13)
    prompts = [torch.randint(0, 503, (n,), generator=g).tolist() for n in (20, 5, 33, 9)]
    limits = [25, 12, 30, 18]
    model = load_model(d, dtype=dtype, page_size=page, num_pages=40, max_batch=4, max_tokens_per_step=64)

    def run(lookahead, eos, temperature=0.0):
        sched = Scheduler(model, lookahead=lookahead)
        for i in range(3):
            sched.add(Request(f"r{i}", prompts[i], max_tokens=limits[i], eos_id=eos if i == 0 else -1,
                              temperature=temperature, top_k=40, top_p=0.95, seed=100 + i))
        for _ in range(6):
            sched.step()
        sched.add(Request("r3", prompts[3], max_tokens=limits[3], temperature=temperature, seed=7))
        out = sched.run()
        assert sched._inflight is None and not sched.running and (sched.steps_ahead > 0) == lookahead
        model.engine.cache.check()
        assert model.engine.cache.num_free() == 40
        return [out[f"r{i}"] for i in range(4)]

    plain = run(False, -1)
    assert [len(o) for o in plain] == limits
    eos = plain[0][10]                       # the first request will stop where this token first appears
    stop = plain[0].index(eos)
    for look in (True,):
        got = run(look, -1)
        with_eos = run(look, eos)
        if dtype == "float32":
            assert got == plain
            assert with_eos[0] == plain[0][:stop] and with_eos[1:] == plain[1:]
            assert run(True, -1, temperature=0.8) == run(False, -1, temperature=0.8)      # sampled rows start early too

            def mixed(lookahead):       # greedy, sampled, greedy with a penalty, sampled with a penalty in one batch
                sched = Scheduler(model, lookahead=lookahead)
                kinds = [dict(), dict(temperature=0.9, top_k=30, seed=3), dict(repetition_penalty=25.0),
                         dict(temperature=0.7, top_p=0.9, repetition_penalty=1.6, seed=4)]
                for i, kw in enumerate(kinds):
                    sched.add(Request(f"m{i}", prompts[i], max_tokens=16, **kw))
                out = sched.run()
                assert (sched.steps_ahead >= 10) == lookahead
                return [out[f"m{i}"] for i in range(4)]
            ahead = mixed(True)
            assert ahead == mixed(False)
            assert ahead[0] == plain[0][:16] and ahead[2] != plain[2][:16]      # the penalty changed what is generated
        else:   # bfloat16: another batch may round a near tie the other way; lengths and stop rules must hold
            assert [len(o) for o in got] == limits
            assert eos not in with_eos[0] and len(with_eos[0]) <= limits[0]
            from gpu_util import assert_diverges_only_at_a_close_call
            oracle = PlainModel(d)
            for i, (a, b) in enumerate(zip(got, plain)):
                assert_diverges_only_at_a_close_call(oracle, prompts[i], a, b, f"request {i} with lookahead")


def test_two_engines_in_one_process_keep_their_own_kernel_options(model_dirs):
    """The options that pin kernel paths belong to an engine: one engine on the general attention kernel and the
    CUDA-core products, one on the library's own choice, side by side, each used while the other exists. Both are
    held against the plain implementation; neither sees the other's options."""
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.config import KernelOptions
    d, page = model_dirs["A"]
    plain = PlainModel(d)
    pinned = KernelOptions(force_general_attention=True, force_simt_gemm=True, fuse_qkv=False)
    a = load_model(d, dtype="bfloat16", page_size=page, num_pages=32, kernel_options=pinned)
    b = load_model(d, dtype="bfloat16", page_size=page, num_pages=32)
    assert a.engine.rt.ops.options == pinned and b.engine.rt.ops.options == KernelOptions()
    assert a.engine.rt.ops is not b.engine.rt.ops
    prompt = [5, 17, 3, 250, 9, 77, 41]
    from gpu_util import assert_diverges_only_at_a_close_call
    want = plain.greedy(prompt, 12)
    for model in (a, b, a):
        assert_diverges_only_at_a_close_call(plain, prompt, model.generate(prompt, max_tokens=12), want, "two engines")
    with pytest.raises(dataclasses.FrozenInstanceError):
        a.engine.rt.ops.options.gemm_route = "tc"


# ------------------------------------------------------------------------------- parts alone
def _runtime(dtype):
    from nanoinfer_b200.csrc.lib import load_kernels
    from nanoinfer_b200.parts.base import Runtime
    return Runtime(torch.device("cuda:0"), tdt(dtype), load_kernels())


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", DTYPES)
def test_part_rmsnorm(dtype):
    from nanoinfer_b200.parts.norm import RMSNorm
    rt = _runtime(dtype)
    gain = (1 + 0.1 * _rand((200,), 1)).to(torch.bfloat16)
    part = RMSNorm(RMSNorm.spec(200, 3e-4, "g"), {"gain": gain}, rt)
    x = _rand((19, 200), 2, 2.0).cuda()
    assert_close(part.forward(x), rms_norm(x.double().cpu(), gain.double(), 3e-4), rt.dtype, "rmsnorm part")


def test_part_rotary_tables():
    from nanoinfer_b200.parts.position import RotaryEncoding
    rt = _runtime("float32")
    part = RotaryEncoding(RotaryEncoding.spec(48, 50000.0, 300), {}, rt)
    cos, sin, dim = part.rotary()
    c, s = rope_tables(torch.arange(300), 48, 50000.0)
    assert dim == 48 and (cos.cpu().double() - c[:, :24]).abs().max() < 1e-7 and (sin.cpu().double() - s[:, :24]).abs().max() < 1e-7


@pytest.mark.parametrize("dtype", DTYPES)
def test_part_swiglu(dtype):
    from nanoinfer_b200.parts.feedforward import SwiGLU
    rt = _runtime(dtype)
    w = {"gate_w": _rand((200, 144), 3, 0.08).to(torch.bfloat16), "up_w": _rand((200, 144), 4, 0.08).to(torch.bfloat16),
         "down_w": _rand((144, 200), 5, 0.08).to(torch.bfloat16)}
    part = SwiGLU(SwiGLU.spec("mlp", 144, 200), w, rt)
    h = _rand((23, 144), 6).to(rt.dtype).cuda()
    res = _rand((23, 144), 7).cuda()
    want = res.double().cpu() + swiglu(h.double().cpu(), w["gate_w"].double(), w["up_w"].double(), w["down_w"].double())
    part.forward(h, res, None)
    assert_close(res, want, rt.dtype, "swiglu part")


@pytest.mark.parametrize("dtype", DTYPES)
def test_part_embedding_and_head(dtype):
    from nanoinfer_b200.parts.embedding import LinearHead, TokenEmbedding
    rt = _runtime(dtype)
    table = _rand((311, 72), 8, 0.5).to(torch.bfloat16)
    emb = TokenEmbedding(TokenEmbedding.spec("e", 311, 72), {"table": table}, rt)
    head = LinearHead(LinearHead.spec("e", 311, 72), {"weight": table}, rt)
    ids = torch.tensor([0, 310, 5, 5], dtype=torch.int32, device="cuda")
    x = emb.forward(ids, None)
    assert torch.equal(x.cpu(), table[ids.long().cpu()].float())
    h = _rand((4, 72), 9).to(rt.dtype).cuda()
    assert_close(head.forward(h), linear(h.double().cpu(), table.double()), rt.dtype, "head part")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,window,bias", [(6, 2, 32, 0, True), (3, 3, 48, 9, False), (14, 2, 64, 0, True)])
def test_part_attention_whole_and_cut(dtype, heads, kv_heads, hd, window, bias):
    """The attention part alone: a whole sequence in one step equals the plain attention; the same
    sequence cut into a portion and single tokens gives the same rows."""
    from gpu_util import make_paged_batch
    from nanoinfer_b200.parts.attention import GroupedQueryAttention
    from nanoinfer_b200.parts.base import LayerCache
    from nanoinfer_b200.parts.position import RotaryEncoding
    rt = _runtime(dtype)
    hidden, page, T = 80, 8, 45
    spec = GroupedQueryAttention.spec("a", hidden, heads, kv_heads, hd, bias, "rot", window)
    w = {role: _rand(ts.shape, 10 + i, 0.1).to(torch.bfloat16) for i, (role, ts) in enumerate(spec.tensors.items())}
    part = GroupedQueryAttention(spec, w, rt)
    part.bind_positions({"rot": RotaryEncoding(RotaryEncoding.spec(hd, 1e4, 64), {}, rt)})
    h = _rand((T, hidden), 30).to(rt.dtype)
    # plain
    wd = {k: v.double() for k, v in w.items()}
    hd64 = h.double()
    q = linear(hd64, wd["q_w"], wd.get("q_b")).view(T, heads, hd)
    k = linear(hd64, wd["k_w"], wd.get("k_b")).view(T, kv_heads, hd)
    v = linear(hd64, wd["v_w"], wd.get("v_b")).view(T, kv_heads, hd)
    cos, sin = rope_tables(torch.arange(T), hd, 1e4)
    a = causal_attention_fast(apply_rope(q, cos, sin), apply_rope(k, cos, sin), v, window)
    want = linear(a.reshape(T, -1), wd["o_w"])

    shape = (16, kv_heads, page, hd)
    for cuts in ([T], [20, 1, 1, 13, 10]):
        kp, vp = torch.zeros(shape, dtype=rt.dtype, device="cuda"), torch.zeros(shape, dtype=rt.dtype, device="cuda")
        outs, done = [], 0
        for n in cuts:
            ctx, bt = make_paged_batch([n], [done], page, 16, "cuda", shuffle=False)
            res = torch.zeros(n, hidden, device="cuda")
            part.forward(h[done:done + n].cuda().contiguous(), res, ctx, LayerCache({"k": kp, "v": vp}, bt, page, True, None))
            outs.append(res)
            done += n
        assert_close(torch.cat(outs), want, rt.dtype, f"attention part cuts={cuts}")


# ------------------------------------------------------------------------------- sampling kernels
@pytest.mark.parametrize("vocab", [13, 503, 4100, 151936])      # a row smaller than the cluster's slices; odd; aligned; the real one
def test_sampling_kernels_follow_the_plain_pipeline(vocab):
    import numpy as np
    from plain_qwen2 import greedy_pick, sampling_distribution
    from nanoinfer_b200.csrc.lib import load_kernels
    from nanoinfer_b200.sampling import SampleRow, Sampler, SamplingParams, uniform_for
    sampler = Sampler(load_kernels(), "cuda:0")
    g = torch.Generator().manual_seed(5)
    base = torch.randn(1, vocab, generator=g) * 3.0
    base[0, 7] = base[0, 11] = base.max() + 0.5       # a tie at the top
    context = [7, 3, 3, min(100, vocab - 3), vocab - 1]
    cases = [SamplingParams(temperature=0.7), SamplingParams(temperature=1.3, top_k=40),
             SamplingParams(temperature=0.9, top_p=0.8), SamplingParams(temperature=1.0, top_k=200, top_p=0.5),
             SamplingParams(temperature=0.5, repetition_penalty=1.7, top_k=5), SamplingParams(temperature=2.0, top_k=1)]
    for ci, params in enumerate(cases):
        rows, n = [], 24
        for i in range(n):
            rows.append(SampleRow(params, context, generated=i, seed=100 + ci))
        logits = base.repeat(n, 1).cuda().contiguous()
        toks = sampler.sample(logits, rows)
        probs = sampling_distribution(base[0].double().numpy(), context, params.temperature, params.k, params.p,
                                      params.repetition_penalty)
        cdf = np.cumsum(probs)
        for i, tok in enumerate(toks):
            u = uniform_for(100 + ci, i)
            assert probs[tok] > 0, (ci, i, tok)
            lo, hi = cdf[tok] - probs[tok], cdf[tok]
            assert lo - 2e-5 <= u <= hi + 2e-5, (ci, i, tok, u, lo, hi)
        if params.top_k == 1:
            assert set(toks) <= {7, 11}
    # greedy with a penalty: the first maximum after the penalty
    rows = [SampleRow(SamplingParams(repetition_penalty=3.0), context, 0), SampleRow(SamplingParams(), None, 0)]
    toks = sampler.sample(base.repeat(2, 1).cuda().contiguous(), rows)
    assert toks == [greedy_pick(base[0].numpy(), context, 3.0), 7]
    assert toks[0] == 11
    # greedy rows beside sampled ones take the sampling kernel too (one launch, nothing for the host to merge): the
    # first of the tied maxima, whatever the row's seed; the sampled rows draw what they draw alone
    sampled = SamplingParams(temperature=0.8, top_k=30, top_p=0.9)
    rows = [SampleRow(SamplingParams(), None, i, seed=i) if i % 3 else SampleRow(sampled, None, i, seed=40) for i in range(12)]
    assert sampler.can_sample_async(rows)
    alone = sampler.sample(base.repeat(4, 1).cuda().contiguous(), [r for r in rows if not r.params.greedy])
    for toks in (sampler.sample(base.repeat(12, 1).cuda().contiguous(), rows),
                 sampler.sample_async(base.repeat(12, 1).cuda().contiguous(), rows).wait()):
        assert [t for t, r in zip(toks, rows) if r.params.greedy] == [7] * 8
        assert [t for t, r in zip(toks, rows) if not r.params.greedy] == alone
    # a penalty with one more id per row on the device (the token of a step in flight): penalised once, whether the
    # row's own list holds it already (row 0), not (row 1), or the row has no penalty (row 2)
    K = load_kernels()
    l3 = base.repeat(3, 1).cuda().contiguous()
    K.repetition_penalty(l3, torch.tensor([7, 3, 3], dtype=torch.int32, device="cuda"), torch.tensor([0, 2, 3, 3], dtype=torch.int32, device="cuda"),
                         torch.tensor([2.0, 4.0, 1.0], device="cuda"), torch.tensor([3, 7, 7], dtype=torch.int32, device="cuda"))
    want3 = base.repeat(3, 1)
    for r, ids, p in ((0, [7, 3], 2.0), (1, [3, 7], 4.0)):
        for i in ids:
            want3[r, i] = want3[r, i] / p if want3[r, i] > 0 else want3[r, i] * p
    assert torch.equal(l3.cpu(), want3)
    shifted = base.clone()
    shifted[0, 11] += 1e-3          # no tie: the one maximum
    assert sampler.sample(shifted.repeat(2, 1).cuda().contiguous(), rows[:2]) [1] == 11


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_graphs_padding_wants_and_buckets(model_dirs, dtype):
    """Pure decode steps are replayed from captured graphs: three live requests in a bucket of four
    (one padding row), contexts that cross a bucket edge (256), rows that want nothing, and the same
    without graphs must agree with the plain implementation."""
    from nanoinfer_b200.engine import StepEntry
    d, page = model_dirs["B"]
    plain = PlainModel(d)
    g = torch.Generator().manual_seed(9)
    seqs = [torch.randint(0, 503, (n,), generator=g).tolist() for n in (300, 290, 40)]
    want = [plain.logits(s) for s in seqs]
    for graphs in (True, False):
        eng = engine_for(d, page, dtype, num_pages=128, cuda_graphs=graphs)
        assert (eng._graphs is not None) == graphs
        rcs = [eng.open(i) for i in range(3)]
        starts = [240, 250, 5]
        eng.step([StepEntry(rc, s[:n], []) for rc, s, n in zip(rcs, seqs, starts)])
        got = [[] for _ in seqs]
        for step in range(35):
            entries, rows = [], []
            for i, (rc, s) in enumerate(zip(rcs, seqs)):
                pos = starts[i] + step
                wants = [0] if (step + i) % 3 else []
                entries.append(StepEntry(rc, [s[pos]], wants))
                if wants:
                    rows.append((i, pos))
            logits = eng.step(entries)
            for (i, pos), row in zip(rows, logits):
                got[i].append((pos, row.clone()))
        if graphs:
            assert len(eng._graphs.captured) >= 2 and eng.graph_launches > 0
        for i in range(3):
            for pos, row in got[i]:
                assert_close(row, want[i][pos], tdt(dtype), f"graphs={graphs} request {i} position {pos}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "W"])
def test_decode_graphs_rows_change_hands(model_dirs, name, dtype):
    """A captured graph's input rows are refreshed in place. A request ends and the others move up a
    row, a new request takes the first row, the batch shrinks so that a row becomes padding and grows
    again, and (model W) a window frees pages in the middle of it: every row must still show its own
    request's pages."""
    from nanoinfer_b200.engine import StepEntry
    d, page = model_dirs[name]
    plain = PlainModel(d)
    g = torch.Generator().manual_seed(4)
    n = min(plain.cfg["max_pos"], 120)
    seqs = {k: torch.randint(0, plain.cfg["vocab"], (n,), generator=g).tolist() for k in "abcd"}
    want = {k: plain.logits(s) for k, s in seqs.items()}
    eng = engine_for(d, page, dtype, num_pages=64)
    fed, rcs = {}, {}

    def prompt(k, count):
        rcs[k] = eng.open(k)
        eng.step([StepEntry(rcs[k], seqs[k][:count], [])])
        fed[k] = count

    def decode(order, steps):
        for _ in range(steps):
            logits = eng.step([StepEntry(rcs[k], [seqs[k][fed[k]]], [0]) for k in order])
            for k, row in zip(order, logits):
                assert_close(row, want[k][fed[k]], tdt(dtype), f"{name} request {k} position {fed[k]}")
                fed[k] += 1

    prompt("a", 30); prompt("b", 7); prompt("c", 19)
    decode("abc", 20)
    eng.close(rcs.pop("a"))
    decode("bc", 6)                 # b and c move up; the third row is padding of another bucket
    prompt("d", 3)
    decode("dbc", 20)               # d takes the first row, pages that a held are used again
    decode("c", 5)
    decode("cbd", 10)
    assert eng.graph_launches > 0
    for rc in rcs.values():
        eng.close(rc)
    eng.cache.check()


REAL_WIDTHS = {
    # name: layers, hidden, heads, kv heads, head dim, intermediate, vocabulary, tied head
    "0.5b": (2, 896, 14, 2, 64, 4864, 151936, True),
    "1.5b": (1, 1536, 12, 2, 128, 8960, 30011, True),       # the family's widths with a smaller, odd vocabulary
    "7b": (1, 3584, 28, 4, 128, 18944, 30011, False),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", sorted(REAL_WIDTHS))
def test_real_layer_widths(tmp_path, dtype, shape):
    """Layers with the widths of the 0.5B, 1.5B and 7B models (theta 1e6): a prompt in one step, then cut
    into portions and single tokens, so that the prefill and the decode kernels both run at these sizes."""
    from nanoinfer_b200.engine import StepEntry
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    layers, hidden, heads, kv_heads, hd, inter, vocab, tied = REAL_WIDTHS[shape]
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers, "hidden_size": hidden,
           "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": hd, "intermediate_size": inter,
           "vocab_size": vocab, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": tied,
           "max_position_embeddings": 4096}
    d = str(tmp_path / "m")
    write_random_model(config_from_json_dict(cfg), d, seed=11)
    plain = PlainModel(d, torch.float32 if dtype == "bfloat16" else torch.float64)
    ids = torch.randint(0, vocab, (150,), generator=torch.Generator().manual_seed(12)).tolist()
    want = plain.logits(ids)[[0, 63, 64, 100, 149]]
    eng = engine_for(d, 16, dtype, num_pages=32)
    rc = eng.open("whole")
    got = eng.step([StepEntry(rc, ids, [0, 63, 64, 100, 149])])
    assert_close(got, want, tdt(dtype), "real widths, whole")
    eng.close(rc)
    rc = eng.open("cut")
    rows = [eng.step([StepEntry(rc, ids[:64], [0, 63])]), eng.step([StepEntry(rc, ids[64:100], [0])])]
    rows.append(eng.step([StepEntry(rc, [ids[100]], [0])]).clone())
    for t in ids[101:149]:
        eng.step([StepEntry(rc, [t], [])])
    rows.append(eng.step([StepEntry(rc, [ids[149]], [0])]).clone())
    assert_close(torch.cat(rows), want, tdt(dtype), "real widths, cut")
    eng.close(rc)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_portions_of_a_recurring_shape_replay_a_captured_graph(model_dirs, dtype):
    """A step of prompt portions whose shape has been seen before is captured once and replayed from then on: the
    first step of a shape runs eagerly, the second captures, the third only replays. Different requests, ids,
    pages and wanted rows each time (those are data the graph reads from its input buffer); every row against the
    plain implementation; a step of another shape in between runs eagerly and disturbs nothing."""
    from nanoinfer_b200.engine import StepEntry
    d, page = model_dirs["C"]
    plain = PlainModel(d)
    eng = engine_for(d, page, dtype, num_pages=200, max_batch=4)
    assert eng._portion_graphs is not None
    eng._portion_graphs.min_tokens, eng._portion_graphs.sightings = 64, 2
    g = torch.Generator().manual_seed(31)
    vocab = plain.cfg["vocab"]
    shapes = [(70, 30), (70, 30), (33,), (70, 30), (70, 30)]
    wants = [([0, 69], [29]), ([5, 17], [0]), ([32],), ([68, 69], [1]), ([1, 2], [3])]
    for turn, (shape, want) in enumerate(zip(shapes, wants)):
        prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in shape]
        reqs = [eng.open(f"t{turn}r{i}") for i in range(len(shape))]
        replayed_before = eng.graph_launches
        got = eng.step([StepEntry(rc, p, w) for rc, p, w in zip(reqs, prompts, want)])
        assert (eng.graph_launches > replayed_before) == (turn in (1, 3, 4)), "which steps ran from the graph"
        ref = torch.cat([plain.logits(p)[list(w)] for p, w in zip(prompts, want)])
        assert_close(got, ref, tdt(dtype), f"portion step {turn}")
        # and the cache it left: one more token for each request, decoded from the pages
        nxt = [int(torch.randint(0, vocab, (1,), generator=g)) for _ in shape]
        got = eng.step([StepEntry(rc, [t], [0]) for rc, t in zip(reqs, nxt)])
        ref = torch.stack([plain.logits(p + [t])[-1] for p, t in zip(prompts, nxt)])
        assert_close(got, ref, tdt(dtype), f"token after portion step {turn}")
        for rc in reqs:
            eng.close(rc)
        if turn == 0:
            assert not eng._portion_graphs.captured
        if turn in (1, 3, 4):
            assert len(eng._portion_graphs.captured) == 1
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_steps_of_a_recurring_shape_replay_a_captured_graph(model_dirs, dtype):
    """Decoded tokens beside a prompt portion, the shape a long prompt fed under the token budget repeats while
    other requests decode: captured the second time, replayed from then on, with the decoding requests' contexts
    growing across a page edge meanwhile (the graph reads lengths and block tables from its input buffer). Named
    portion first on purpose: the step lays the decoded tokens out first and returns the logits in the caller's order."""
    from nanoinfer_b200.engine import StepEntry
    d, page = model_dirs["C"]
    plain = PlainModel(d)
    eng = engine_for(d, page, dtype, num_pages=200, max_batch=4)
    eng._portion_graphs.min_tokens, eng._portion_graphs.sightings = 64, 2
    g = torch.Generator().manual_seed(37)
    vocab = plain.cfg["vocab"]
    decoding = {k: torch.randint(0, vocab, (n,), generator=g).tolist() for k, n in (("x", 60), ("y", 27))}
    reqs = {k: eng.open(k) for k in decoding}
    fed = {"x": 44, "y": 11}
    for k, rc in reqs.items():
        eng.step([StepEntry(rc, decoding[k][:fed[k]], [])])
    for turn in range(5):
        prompt = torch.randint(0, vocab, (90,), generator=g).tolist()
        new = eng.open(f"p{turn}")
        entries = [StepEntry(new, prompt, [0, 89])] + [StepEntry(reqs[k], [decoding[k][fed[k]]], [0]) for k in reqs]
        before = eng.graph_launches
        got = eng.step(entries)
        assert (eng.graph_launches > before) == (turn >= 1), "which steps ran from the graph"
        ref = torch.stack([plain.logits(prompt)[0], plain.logits(prompt)[89]] +
                          [plain.logits(decoding[k][:fed[k] + 1])[-1] for k in reqs])
        assert_close(got, ref, tdt(dtype), f"mixed step {turn}")
        for k in reqs:
            fed[k] += 1
        eng.close(new)
    assert len(eng._portion_graphs.captured) == 1
    for rc in reqs.values():
        eng.close(rc)
    eng.cache.check()
