"""Logits at the shapes that the benchmark times, against the plain implementation: prompts of 2,048 and
4,096 tokens in ONE step at the layer widths of the 0.5B and 1.5B models (the tcgen05 prefill attention
walks 16 and 32 key blocks, the two-SM GEMM runs inside the assembled step), 8 and 64 live requests
decoding at a context of about 4,000 tokens through the captured graphs and across the 4,096 edge of the
context buckets, and a step in which a decoding request comes AFTER a prompt portion. One layer and a
small, odd vocabulary keep the plain side (the same formulas in float64, computed by torch on the GPU)
short; the widths, head counts, head sizes and page size are the benchmark's."""
import pytest
import torch

from gpu_util import assert_close
from plain_qwen2 import PlainModel

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]

WIDTHS = {
    # name: hidden, heads, kv heads, head dim, intermediate, vocabulary, tied head
    "0.5b": (896, 14, 2, 64, 4864, 3011, True),
    "1.5b": (1536, 12, 2, 128, 8960, 2003, True),
}


def tdt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def make_model(tmp_path, shape, layers=1, max_pos=8192):
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    hidden, heads, kv_heads, hd, inter, vocab, tied = WIDTHS[shape]
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers, "hidden_size": hidden,
           "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": hd, "intermediate_size": inter,
           "vocab_size": vocab, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": tied,
           "max_position_embeddings": max_pos}
    d = str(tmp_path / f"m_{shape}")
    write_random_model(config_from_json_dict(cfg), d, seed=21)
    return d, vocab


def engine_for(model_dir, dtype, num_pages, max_batch):
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine
    return Engine(model_dir, EngineConfig(dtype=dtype, page_size=16, num_pages=num_pages, max_batch=max_batch))


def random_ids(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,tokens", [("0.5b", 2048), ("0.5b", 4096), ("1.5b", 2048), ("1.5b", 4096)])
def test_long_prompt_in_one_step(tmp_path, dtype, shape, tokens):
    """A whole prompt of the benchmark's length as one portion; rows at the first tile's edges, in the middle and
    at the end. Then the same prompt with its second half as a portion that starts inside the context."""
    from nanoinfer_b200.engine import StepEntry
    d, vocab = make_model(tmp_path, shape)
    plain = PlainModel(d, torch.float64, device="cuda")
    ids = random_ids(vocab, tokens, 22)
    rows = [0, 1, 127, 128, 129, 1023, 1024, 2047, tokens - 2, tokens - 1]
    want = plain.logits(ids)[rows]
    eng = engine_for(d, dtype, num_pages=tokens // 16 + 4, max_batch=2)
    rc = eng.open("whole")
    got = eng.step([StepEntry(rc, ids, rows)])
    eng.check_device()
    assert_close(got, want, tdt(dtype), f"{shape}: {tokens} tokens in one step")
    eng.close(rc)
    half = tokens // 2
    rc = eng.open("halves")
    first = eng.step([StepEntry(rc, ids[:half], [r for r in rows if r < half])])
    second = eng.step([StepEntry(rc, ids[half:], [r - half for r in rows if r >= half])])
    eng.check_device()
    assert_close(torch.cat([first, second]), want, tdt(dtype), f"{shape}: {tokens} tokens in two portions")
    eng.close(rc)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,batch", [("0.5b", 8), ("0.5b", 64), ("1.5b", 8)])
def test_decode_batches_at_context_4096_through_the_graphs(tmp_path, dtype, shape, batch):
    """``batch`` live requests of different lengths near 4,000 tokens, their prompts fed in interleaved portions
    (so that their pages interleave in the pool), then 40 decode steps of all of them as one batch: the
    longest request crosses position 4,096, where the captured graph of the next context bucket takes over.
    Every row of every step is compared."""
    from nanoinfer_b200.engine import StepEntry
    d, vocab = make_model(tmp_path, shape)
    plain = PlainModel(d, torch.float64, device="cuda")
    steps = 40
    lens = [4076 - 61 * i for i in range(batch)] if batch <= 8 else [4076 - 17 * i for i in range(batch)]
    seqs = [random_ids(vocab, n + steps, 100 + i) for i, n in enumerate(lens)]
    want = [plain.logits(s)[n - 1:] for s, n in zip(seqs, lens)]       # rows n-1 .. n+steps-1
    pages = sum(-(-(n + steps) // 16) for n in lens) + 8
    eng = engine_for(d, dtype, num_pages=pages, max_batch=batch)
    rcs = [eng.open(f"r{i}") for i in range(batch)]
    fed = [0] * batch
    portion = 1024
    got = [[] for _ in range(batch)]
    while any(f < n for f, n in zip(fed, lens)):
        entries, who = [], []
        budget = 8192
        for i in range(batch):
            n = min(portion + 64 * (i % 3), lens[i] - fed[i], budget)
            if n <= 0:
                continue
            last = fed[i] + n == lens[i]
            entries.append(StepEntry(rcs[i], seqs[i][fed[i]:fed[i] + n], [n - 1] if last else []))
            who.append((i, last))
            fed[i] += n
            budget -= n
        logits = eng.step(entries)
        row = 0
        for i, last in who:
            if last:
                got[i].append(logits[row].clone())
                row += 1
    for t in range(steps):
        entries = [StepEntry(rcs[i], [seqs[i][lens[i] + t]], [0]) for i in range(batch)]
        logits = eng.step(entries)
        for i in range(batch):
            got[i].append(logits[i].clone())
    eng.check_device()
    assert eng.graph_launches > 0
    assert max(rc.length for rc in rcs) > 4096
    for i in range(batch):
        assert_close(torch.stack(got[i]), want[i], tdt(dtype), f"{shape}: request {i} of {batch} (length {lens[i]})")
    for rc in rcs:
        eng.close(rc)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ["0.5b", "1.5b"])
def test_a_decoding_request_behind_a_prompt_portion(tmp_path, dtype, shape):
    """Entry order of a step: a prompt portion first, single tokens of two decoding requests after it, and a
    second portion last. Whatever kernel the rows behind the first portion take, their logits are the same."""
    from nanoinfer_b200.engine import StepEntry
    d, vocab = make_model(tmp_path, shape)
    plain = PlainModel(d, torch.float64, device="cuda")
    a, b, c, e = (random_ids(vocab, n, 200 + n) for n in (700, 1301, 520, 333))
    want = {k: plain.logits(v) for k, v in (("a", a), ("b", b), ("c", c), ("e", e))}
    eng = engine_for(d, dtype, num_pages=256, max_batch=4)
    rc = {k: eng.open(k) for k in "abce"}
    eng.step([StepEntry(rc["b"], b[:1300], []), StepEntry(rc["c"], c[:519], [])])
    eng.step([StepEntry(rc["a"], a[:400], [])])
    got = eng.step([StepEntry(rc["a"], a[400:], [0, 299]), StepEntry(rc["b"], b[1300:], [0]),
                    StepEntry(rc["c"], c[519:], [0]), StepEntry(rc["e"], e, [0, 332])])
    eng.check_device()
    ref = torch.stack([want["a"][400], want["a"][699], want["b"][1300], want["c"][519], want["e"][0], want["e"][332]])
    assert_close(got, ref, tdt(dtype), f"{shape}: decode rows behind a prompt portion")
    for r in rc.values():
        eng.close(r)
    eng.cache.check()
