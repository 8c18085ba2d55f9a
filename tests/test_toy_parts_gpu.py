"""Generality of the parts, shown with toy parts that live in this test only: a mixer with fixed-size
state of its own (a running mean of its inputs) is registered, built and stepped beside attention
layers in one model, without a change to the framework's files; the run order names a layer twice and
lets a layer read another layer's cache. Compared with a plain computation of whole sequences."""
from dataclasses import dataclass

import pytest
import torch

from gpu_util import assert_close
from plain_qwen2 import apply_rope, causal_attention_fast, linear, read_weights, rms_norm, rope_tables, swiglu

pytestmark = pytest.mark.gpu


def _register():
    from nanoinfer_b200.config.model_config import ModelConfig
    from nanoinfer_b200.parts.attention import GroupedQueryAttention
    from nanoinfer_b200.parts.base import Mixer, StateNeed
    from nanoinfer_b200.parts.embedding import LinearHead, TokenEmbedding
    from nanoinfer_b200.parts.feedforward import SwiGLU
    from nanoinfer_b200.parts.norm import RMSNorm
    from nanoinfer_b200.parts.position import RotaryEncoding
    from nanoinfer_b200.parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, TensorSpec
    from nanoinfer_b200.registry import register_architecture, register_part

    class RunningMeanMixer(Mixer):
        """out_t = W . mean(h_0..h_t): state per request = [sum of inputs | count]."""

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.hidden = int(spec.params["hidden"])
            self.w = rt.matrix(tensors["w"])

        def state_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)

        def forward(self, h, residual32, ctx, cache):
            start = 0
            for q_len, slot in zip(ctx.host.q_lens, ctx.host.slots):
                st = cache.state[slot]
                rows = h[start:start + q_len].float()
                sums = st[:self.hidden] + rows.cumsum(0)
                counts = st[self.hidden] + torch.arange(1, q_len + 1, device=h.device, dtype=torch.float32)
                mean = (sums / counts[:, None]).to(self.rt.dtype)
                out = torch.zeros(q_len, self.hidden, dtype=torch.float32, device=h.device)
                self.ops.linear(mean.contiguous(), self.w, None, out, "f32")
                residual32[start:start + q_len] += out
                st[:self.hidden] = sums[-1]
                st[self.hidden] = counts[-1]
                start += q_len

    register_part("toy_running_mean", RunningMeanMixer)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        intermediate_size: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_dim: int = 0
        eps: float = 1e-6

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyForCausalLM", model_type="toy", vocab_size=d["vocab_size"],
                       hidden_size=d["hidden_size"], num_hidden_layers=3, max_position_embeddings=d["max_pos"],
                       tie_word_embeddings=False, eos_token_id=-1, intermediate_size=d["intermediate_size"],
                       heads=d["heads"], kv_heads=d["kv_heads"], head_dim=d["head_dim"], eps=d["eps"])

        def to_json_dict(self):
            return {"architectures": ["ToyForCausalLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "max_pos": self.max_position_embeddings, "intermediate_size": self.intermediate_size,
                    "heads": self.heads, "kv_heads": self.kv_heads, "head_dim": self.head_dim, "eps": self.eps}

    def toy_plan(c):
        h = c.hidden_size

        def layer(i, mixer):
            return LayerSpec("pre_norm", {
                "mixer_norm": RMSNorm.spec(h, c.eps, f"l{i}.n1"), "mixer": mixer,
                "ffn_norm": RMSNorm.spec(h, c.eps, f"l{i}.n2"), "ffn": SwiGLU.spec(f"l{i}.mlp", h, c.intermediate_size)})
        attn = lambda i: GroupedQueryAttention.spec(f"l{i}.attn", h, c.heads, c.kv_heads, c.head_dim, True, "rot")
        toy = PartSpec("toy_running_mean", {"hidden": h}, {"w": TensorSpec("l0.toy.w", (h, h))})
        return ModelPlan(
            architecture=c.architecture, hidden_size=h, vocab_size=c.vocab_size,
            max_position_embeddings=c.max_position_embeddings,
            embedding=TokenEmbedding.spec("embed", c.vocab_size, h),
            positions={"rot": RotaryEncoding.spec(c.head_dim, 10000.0, c.max_position_embeddings)},
            layers=[layer(0, toy), layer(1, attn(1)), layer(2, attn(2))],
            # toy, attention, the toy layer AGAIN (state of its own), attention 1 again (cache of its own),
            # attention 2 reading the cache of entry 1 (it writes none)
            schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1),
                      ScheduleEntry(2, reads_cache_of=1)],
            final_norm=RMSNorm.spec(h, c.eps, "norm"), lm_head=LinearHead.spec("head", c.vocab_size, h))

    register_architecture("ToyForCausalLM", ToyConfig, toy_plan)
    return ToyConfig


TOY = {"architectures": ["ToyForCausalLM"], "vocab_size": 97, "hidden_size": 48, "max_pos": 128,
       "intermediate_size": 72, "heads": 3, "kv_heads": 1, "head_dim": 16, "eps": 2e-6}


def plain_toy(w, ids):
    """Whole sequence, float64."""
    c = TOY
    T = len(ids)
    x = w["embed"][torch.tensor(ids)]
    pos = torch.arange(T)
    cos, sin = rope_tables(pos, c["head_dim"], 10000.0)

    def qkv(i, h):
        g = lambda n: w[f"l{i}.attn.{n}"]
        q = linear(h, g("q_proj.weight"), g("q_proj.bias")).view(T, c["heads"], c["head_dim"])
        k = linear(h, g("k_proj.weight"), g("k_proj.bias")).view(T, c["kv_heads"], c["head_dim"])
        v = linear(h, g("v_proj.weight"), g("v_proj.bias")).view(T, c["kv_heads"], c["head_dim"])
        return apply_rope(q, cos, sin), apply_rope(k, cos, sin), v

    def ffn(i, x):
        h = rms_norm(x, w[f"l{i}.n2"], c["eps"])
        return x + swiglu(h, w[f"l{i}.mlp.gate_proj.weight"], w[f"l{i}.mlp.up_proj.weight"], w[f"l{i}.mlp.down_proj.weight"])

    def toy(x):
        h = rms_norm(x, w["l0.n1"], c["eps"])
        mean = h.cumsum(0) / torch.arange(1, T + 1, dtype=h.dtype)[:, None]
        return ffn(0, x + linear(mean, w["l0.toy.w"]))

    def attn(i, x, kv=None):
        h = rms_norm(x, w[f"l{i}.n1"], c["eps"])
        q, k, v = qkv(i, h)
        if kv is not None:
            k, v = kv
        a = causal_attention_fast(q, k, v)
        return ffn(i, x + linear(a.reshape(T, -1), w[f"l{i}.attn.o_proj.weight"])), (k, v)

    x = toy(x)
    x, kv1 = attn(1, x)
    x = toy(x)
    x, _ = attn(1, x)
    x, _ = attn(2, x, kv=kv1)
    return linear(rms_norm(x, w["norm"], c["eps"]), w["head"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_runs_beside_attention(tmp_path, dtype):
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine, StepEntry
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    _register()
    d = str(tmp_path / "toy")
    write_random_model(config_from_json_dict(TOY), d, seed=3)
    w = read_weights(d)
    eng = Engine(d, EngineConfig(dtype=dtype, page_size=8, num_pages=40, max_batch=3))
    needs = eng.model.cache_needs()
    assert [n[0] is not None for n in needs] == [False, True, False, True, False]
    assert [n[1] is not None for n in needs] == [True, False, True, False, False] and needs[4][2] == 1
    g = torch.Generator().manual_seed(4)
    seqs = {k: torch.randint(0, 97, (n,), generator=g).tolist() for k, n in (("a", 37), ("b", 20), ("c", 51))}
    want = {k: plain_toy(w, v) for k, v in seqs.items()}
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16

    # whole, each alone
    for k, ids in seqs.items():
        rc = eng.open(k)
        assert_close(eng.step([StepEntry(rc, ids, list(range(len(ids))))]), want[k], tdt, f"toy whole {k}")
        eng.close(rc)
    # mixed: portions of changing size beside single tokens, three live; slots are used again
    live = {k: eng.open(k) for k in seqs}
    fed = {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    sizes = {"a": [5, 1, 9, 2], "b": [1, 1, 7], "c": [13, 2, 1]}
    turn = 0
    while live:
        entries, keys = [], []
        for k, rc in live.items():
            n = min(sizes[k][turn % len(sizes[k])], len(seqs[k]) - fed[k])
            entries.append(StepEntry(rc, seqs[k][fed[k]:fed[k] + n], list(range(n))))
            keys.append((k, n))
        logits = eng.step(entries)
        row = 0
        for k, n in keys:
            got[k].append(logits[row:row + n].clone())
            row += n
            fed[k] += n
        for k in [k for k in live if fed[k] == len(seqs[k])]:
            eng.close(live.pop(k))
        turn += 1
    for k in seqs:
        assert_close(torch.cat(got[k]), want[k], tdt, f"toy mixed {k}")
    # a slot handed out again starts from zero state
    rc = eng.open("again")
    assert_close(eng.step([StepEntry(rc, seqs["b"], [len(seqs["b"]) - 1])]), want["b"][-1:], tdt, "toy slot reuse")
    eng.close(rc)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_that_keeps_keys_alone_and_unequal_keys_and_values(tmp_path, dtype):
    """What a mixer keeps per token is a list of paged tensors: a toy mixer that keeps 32-bit keys alone in one
    layer and keys beside wider values (in the compute dtype) in another is registered, built and stepped on the
    device, whole and mixed in portions, with no change to the framework's files."""
    import toy_memory_mixer as toy
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    toy.register()
    d = str(tmp_path / "toy_memory")
    write_random_model(config_from_json_dict(toy.TOY), d, seed=17)
    eng = Engine(d, EngineConfig(dtype=dtype, page_size=4, num_pages=22, max_batch=3))
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    pages = eng.storage.pages
    assert pages[0]["keys"].dtype == torch.float32 and pages[1]["values"].dtype == tdt and "values" not in pages[2]
    assert tuple(pages[1]["values"].shape) == (22, 2, 4, 20) and tuple(pages[1]["keys"].shape) == (22, 2, 4, 12)
    toy.run_through_the_engine(eng, read_weights(d), lambda got, ref, what: assert_close(got, ref, tdt, what))


# ------------------------------------------------------------------ a mixer with state whose steps are captured in graphs
TOY_GRAPH = {"architectures": ["ToyGraphForCausalLM"], "vocab_size": 71, "hidden_size": 32, "max_pos": 160,
             "intermediate_size": 48, "eps": 1e-5}


def _register_graph_safe_toy():
    from nanoinfer_b200.config.model_config import ModelConfig
    from nanoinfer_b200.parts.base import Mixer, StateNeed, as_tensor
    from nanoinfer_b200.parts.embedding import LinearHead, TokenEmbedding
    from nanoinfer_b200.parts.feedforward import SwiGLU
    from nanoinfer_b200.parts.norm import RMSNorm
    from nanoinfer_b200.parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, TensorSpec
    from nanoinfer_b200.registry import register_architecture, register_part

    class RunningMeanOnDevice(Mixer):
        """out_t = W . mean(h_0..h_t), state per request = [sum of inputs | count], computed with device-side index
        arithmetic only (nothing of the batch is read on the host), so its launches are the same for every batch
        and a decode step with it may be captured. A padding row of a captured step carries the spare state slot."""

        graph_safe = True

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.hidden = int(spec.params["hidden"])
            self.w = rt.matrix(tensors["w"])

        def state_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)

        def forward(self, h, residual32, ctx, cache):
            h = as_tensor(h).float()
            req = ctx.req_index.long()
            slots = ctx.state_slots.long()
            start = ctx.q_start.long()
            csum = torch.cat([torch.zeros_like(h[:1]), h.cumsum(0)])            # csum[i] = sum of rows < i
            before = csum[start[:-1]]                                          # per request: rows before its first
            own = csum[1:] - before[req]                                       # inclusive sum within the request's rows
            nth = torch.arange(1, h.shape[0] + 1, device=h.device) - start[:-1][req]
            st = cache.state[slots]                                            # [R, hidden + 1]
            mean = (st[req, :self.hidden] + own) / (st[req, self.hidden] + nth)[:, None]
            out = torch.empty(h.shape[0], self.hidden, dtype=torch.float32, device=h.device)
            self.ops.linear(mean.to(self.rt.dtype).contiguous(), self.w, None, out, "f32")
            residual32 += out
            totals = csum[start[1:]] - before
            counts = (start[1:] - start[:-1]).float()
            cache.state.index_add_(0, slots, torch.cat([totals, counts[:, None]], dim=1))

    register_part("toy_running_mean_on_device", RunningMeanOnDevice)

    @dataclass(frozen=True)
    class ToyGraphConfig(ModelConfig):
        intermediate_size: int = 0
        eps: float = 1e-6

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyGraphForCausalLM", model_type="toy_graph", vocab_size=d["vocab_size"],
                       hidden_size=d["hidden_size"], num_hidden_layers=2, max_position_embeddings=d["max_pos"],
                       tie_word_embeddings=False, eos_token_id=-1, intermediate_size=d["intermediate_size"], eps=d["eps"])

        def to_json_dict(self):
            return {"architectures": ["ToyGraphForCausalLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "max_pos": self.max_position_embeddings, "intermediate_size": self.intermediate_size, "eps": self.eps}

    def plan(c):
        h = c.hidden_size

        def layer(i):
            return LayerSpec("pre_norm", {
                "mixer_norm": RMSNorm.spec(h, c.eps, f"l{i}.n1"),
                "mixer": PartSpec("toy_running_mean_on_device", {"hidden": h}, {"w": TensorSpec(f"l{i}.toy.w", (h, h))}),
                "ffn_norm": RMSNorm.spec(h, c.eps, f"l{i}.n2"), "ffn": SwiGLU.spec(f"l{i}.mlp", h, c.intermediate_size)})
        return ModelPlan(architecture=c.architecture, hidden_size=h, vocab_size=c.vocab_size,
                         max_position_embeddings=c.max_position_embeddings, embedding=TokenEmbedding.spec("embed", c.vocab_size, h),
                         positions={}, layers=[layer(0), layer(1)], schedule=[ScheduleEntry(0), ScheduleEntry(1)],
                         final_norm=RMSNorm.spec(h, c.eps, "norm"), lm_head=LinearHead.spec("head", c.vocab_size, h))

    register_architecture("ToyGraphForCausalLM", ToyGraphConfig, plan)


def plain_toy_graph(w, ids):
    c = TOY_GRAPH
    T = len(ids)
    x = w["embed"][torch.tensor(ids)]
    for i in range(2):
        h = rms_norm(x, w[f"l{i}.n1"], c["eps"])
        mean = h.cumsum(0) / torch.arange(1, T + 1, dtype=h.dtype)[:, None]
        x = x + linear(mean, w[f"l{i}.toy.w"])
        h = rms_norm(x, w[f"l{i}.n2"], c["eps"])
        x = x + swiglu(h, w[f"l{i}.mlp.gate_proj.weight"], w[f"l{i}.mlp.up_proj.weight"], w[f"l{i}.mlp.down_proj.weight"])
    return linear(rms_norm(x, w["norm"], c["eps"]), w["head"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_decodes_through_captured_graphs(tmp_path, dtype):
    """A mixer with state of its own that declares itself graph safe: its decode steps are captured and replayed.
    Three live requests decode in a bucket of four, so every replay has a padding row; that row carries the spare
    state slot, and the live requests' states (sums and counts) stay exactly theirs: every decoded position of every
    request equals the plain whole-sequence computation, also for a request that takes over a finished one's slot."""
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine, StepEntry
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    _register_graph_safe_toy()
    d = str(tmp_path / "toy_graph")
    write_random_model(config_from_json_dict(TOY_GRAPH), d, seed=5)
    w = read_weights(d)
    eng = Engine(d, EngineConfig(dtype=dtype, page_size=8, num_pages=8, max_batch=4))
    assert eng._graphs is not None, "the model is graph safe: decode steps are captured"
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(6)
    seqs = {k: torch.randint(0, 71, (n,), generator=g).tolist() for k, n in (("a", 40), ("b", 33), ("c", 52), ("d", 45))}
    want = {k: plain_toy_graph(w, v) for k, v in seqs.items()}
    prompt = {"a": 9, "b": 17, "c": 3, "d": 20}
    live = {k: eng.open(k) for k in ("a", "b", "c")}
    got = {k: [] for k in seqs}
    for k, rc in live.items():          # prompts, eagerly
        got[k].append(eng.step([StepEntry(rc, seqs[k][:prompt[k]], list(range(prompt[k])))]).clone())
    fed = dict(prompt)
    replays_before = eng.graph_launches
    while live:
        entries = [StepEntry(rc, [seqs[k][fed[k]]], [0]) for k, rc in live.items()]
        logits = eng.step(entries)
        for row, k in enumerate(list(live)):
            got[k].append(logits[row:row + 1].clone())
            fed[k] += 1
        for k in [k for k in live if fed[k] == len(seqs[k])]:
            eng.close(live.pop(k))
            if k == "b":                # "d" takes over the slot that "b" gave back: its state starts from zero
                live["d"] = eng.open("d")
                got["d"].append(eng.step([StepEntry(live["d"], seqs["d"][:prompt["d"]], list(range(prompt["d"])))]).clone())
                fed["d"] = prompt["d"]
    assert eng.graph_launches > replays_before and eng._graphs.captured, "decode steps ran from captured graphs"
    for k in seqs:
        assert_close(torch.cat(got[k]), want[k], tdt, f"graph-safe toy mixer, request {k}")
