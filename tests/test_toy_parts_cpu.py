"""Generality of the parts beyond what the built-in architecture uses, shown with toy parts that live in
this test only and run on the host backend (tests/torch_ops.py), so no GPU is needed:

* a position encoding of another kind (a learned table added to the embedding; the attention bound to it
  rotates nothing),
* a feed-forward with routing (a 32-bit router picks two of several small experts per token and weighs
  them by a softmax over the two),
* another norm (mean-subtracting, with gain and bias),
* another arrangement of a block (mixer and feed-forward both read ONE norm of the block's input),
* different mixers and feed-forwards in different layers, one of them with a window (a cache group of
  its own), and a run order that names a layer twice.

Everything is registered from here; no file of the framework changes. The engine steps the model whole,
in portions and mixed with other requests, and is compared with a plain whole-sequence computation.
"""
from dataclasses import dataclass

import torch

from plain_qwen2 import causal_attention_fast, linear, read_weights, rms_norm, swiglu
from torch_ops import TorchOps

TOY = {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": 89, "hidden_size": 40, "max_pos": 96,
       "intermediate_size": 56, "heads": 4, "kv_heads": 2, "head_dim": 16, "eps": 3e-6,
       "experts": 5, "expert_inner": 24, "window": 6}


def _register():
    from nanoinfer_b200.config.model_config import ModelConfig
    from nanoinfer_b200.parts.attention import GroupedQueryAttention
    from nanoinfer_b200.parts.base import FeedForward, Norm, PositionEncoding
    from nanoinfer_b200.parts.embedding import LinearHead, TokenEmbedding
    from nanoinfer_b200.parts.feedforward import SwiGLU
    from nanoinfer_b200.parts.norm import RMSNorm
    from nanoinfer_b200.parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, TensorSpec
    from nanoinfer_b200.registry import register_architecture, register_arrangement, register_part

    class LearnedPosition(PositionEncoding):
        """x[t] += table[position of t]; mixers bound to it get no rotation (``rotary()`` is None)."""

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.table = rt.vector32(tensors["table"])

        def add_to_embedding(self, x32, ctx):
            x32 += self.table[ctx.positions.long()]

    class CenteredNorm(Norm):
        """(x - mean) / sqrt(var + eps) * gain + bias, in 32-bit or wider."""

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.eps = float(spec.params["eps"])
            self.gain, self.bias = rt.vector32(tensors["gain"]), rt.vector32(tensors["bias"])

        def forward(self, x32, rows=None):
            x = (x32 if rows is None else x32[rows.long()]).double()
            x = x - x.mean(-1, keepdim=True)
            y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.gain.double() + self.bias.double()
            return y.to(self.rt.dtype)

    class TwoOfManyExperts(FeedForward):
        """Router logits in 32-bit; the two best experts of a token, weighed by a softmax over their two
        logits; an expert is ``relu(h Win^T)^2 Wout^T``. Tokens are gathered per expert, so the launches
        depend on the routing (the part is not marked graph_safe)."""

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            p = spec.params
            self.hidden, self.inner, self.experts = int(p["hidden"]), int(p["inner"]), int(p["experts"])
            self.router = rt.matrix(tensors["router"])
            self.w_in = [rt.matrix(w) for w in tensors["w_in"].chunk(self.experts, dim=0)]
            self.w_out = [rt.matrix(w) for w in tensors["w_out"].chunk(self.experts, dim=0)]

        def forward(self, h, residual32, ctx):
            m = h.shape[0]
            logits = torch.empty((m, self.experts), dtype=torch.float32, device=h.device)
            self.ops.linear(h, self.router, None, logits, "f32")
            top, which = logits.topk(2, dim=-1)
            weight = torch.softmax(top, dim=-1)
            for e in range(self.experts):
                rows, slot = (which == e).nonzero(as_tuple=True)
                if rows.numel() == 0:
                    continue
                mid = torch.empty((rows.numel(), self.inner), dtype=torch.float32, device=h.device)
                self.ops.linear(h[rows].contiguous(), self.w_in[e], None, mid, "f32")
                mid = (torch.relu(mid) ** 2).to(self.rt.dtype)
                out = torch.empty((rows.numel(), self.hidden), dtype=torch.float32, device=h.device)
                self.ops.linear(mid, self.w_out[e], None, out, "f32")
                residual32.index_add_(0, rows, out * weight[rows, slot][:, None])

    class SharedNormBlock:
        """x += mixer(n) + feed_forward(n) with n = norm(x) computed once."""

        def __init__(self, parts):
            self.norm, self.mixer, self.ffn = parts["norm"], parts["mixer"], parts["ffn"]

        def forward(self, x32, ctx, cache):
            n = self.norm.forward(x32)
            self.mixer.forward(n, x32, ctx, cache)
            self.ffn.forward(n, x32, ctx)

    register_part("toy_learned_position", LearnedPosition)
    register_part("toy_centered_norm", CenteredNorm)
    register_part("toy_two_of_many", TwoOfManyExperts)
    register_arrangement("toy_shared_norm", SharedNormBlock)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        intermediate_size: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_dim: int = 0
        eps: float = 1e-6
        experts: int = 0
        expert_inner: int = 0
        window: int = 0

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyRoutedForCausalLM", model_type="toy_routed", vocab_size=d["vocab_size"],
                       hidden_size=d["hidden_size"], num_hidden_layers=2, max_position_embeddings=d["max_pos"],
                       tie_word_embeddings=False, eos_token_id=-1, intermediate_size=d["intermediate_size"],
                       heads=d["heads"], kv_heads=d["kv_heads"], head_dim=d["head_dim"], eps=d["eps"],
                       experts=d["experts"], expert_inner=d["expert_inner"], window=d["window"])

        def to_json_dict(self):
            return {"architectures": ["ToyRoutedForCausalLM"], "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "max_pos": self.max_position_embeddings,
                    "intermediate_size": self.intermediate_size, "heads": self.heads, "kv_heads": self.kv_heads,
                    "head_dim": self.head_dim, "eps": self.eps, "experts": self.experts,
                    "expert_inner": self.expert_inner, "window": self.window}

    def centered(name, h, eps):
        return PartSpec("toy_centered_norm", {"eps": eps}, {"gain": TensorSpec(f"{name}.g", (h,), "gain"),
                                                            "bias": TensorSpec(f"{name}.b", (h,), "bias")})

    def plan(c):
        h = c.hidden_size
        dense = LayerSpec("pre_norm", {
            "mixer_norm": RMSNorm.spec(h, c.eps, "l0.n1"),
            "mixer": GroupedQueryAttention.spec("l0.attn", h, c.heads, c.kv_heads, c.head_dim, False, "learned"),
            "ffn_norm": RMSNorm.spec(h, c.eps, "l0.n2"), "ffn": SwiGLU.spec("l0.mlp", h, c.intermediate_size)})
        routed = LayerSpec("toy_shared_norm", {
            "norm": centered("l1.n", h, c.eps),
            "mixer": GroupedQueryAttention.spec("l1.attn", h, c.heads, c.heads, c.head_dim, True, "learned",
                                                window=c.window, scale=0.3),
            "ffn": PartSpec("toy_two_of_many", {"hidden": h, "inner": c.expert_inner, "experts": c.experts}, {
                "router": TensorSpec("l1.moe.router", (c.experts, h)),
                "w_in": TensorSpec("l1.moe.w_in", (c.experts * c.expert_inner, h)),
                "w_out": TensorSpec("l1.moe.w_out", (c.experts * h, c.expert_inner))})})
        return ModelPlan(
            architecture=c.architecture, hidden_size=h, vocab_size=c.vocab_size,
            max_position_embeddings=c.max_position_embeddings,
            embedding=TokenEmbedding.spec("embed", c.vocab_size, h),
            positions={"learned": PartSpec("toy_learned_position", {}, {
                "table": TensorSpec("pos.table", (c.max_position_embeddings, h), "embedding")})},
            layers=[dense, routed],
            schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1)],     # the routed layer runs twice
            final_norm=centered("norm", h, c.eps), lm_head=LinearHead.spec("head", c.vocab_size, h))

    register_architecture("ToyRoutedForCausalLM", ToyConfig, plan)


def plain_toy(w, ids, used=None):
    """Whole sequence in float64, one function per part. ``used`` collects the experts that were chosen."""
    c = TOY
    T, hd = len(ids), c["head_dim"]

    def centered(x, name):
        x = x - x.mean(-1, keepdim=True)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + c["eps"]) * w[f"{name}.g"] + w[f"{name}.b"]

    def attention(h, prefix, heads, kv_heads, bias, window, scale):
        b = (lambda n: w[f"{prefix}.{n}_proj.bias"]) if bias else (lambda n: None)
        q = linear(h, w[f"{prefix}.q_proj.weight"], b("q")).view(T, heads, hd)
        k = linear(h, w[f"{prefix}.k_proj.weight"], b("k")).view(T, kv_heads, hd)
        v = linear(h, w[f"{prefix}.v_proj.weight"], b("v")).view(T, kv_heads, hd)
        a = causal_attention_fast(q, k, v, window=window, scale=scale)
        return linear(a.reshape(T, -1), w[f"{prefix}.o_proj.weight"])

    def experts(h):
        logits = linear(h, w["l1.moe.router"])
        top, which = logits.topk(2, dim=-1)
        weight = torch.softmax(top, dim=-1)
        w_in = w["l1.moe.w_in"].chunk(c["experts"], dim=0)
        w_out = w["l1.moe.w_out"].chunk(c["experts"], dim=0)
        out = torch.zeros_like(h)
        for t in range(T):
            for s in range(2):
                e = int(which[t, s])
                if used is not None:
                    used.add(e)
                out[t] += weight[t, s] * linear(torch.relu(linear(h[t], w_in[e])) ** 2, w_out[e])
        return out

    def dense(x):
        x = x + attention(rms_norm(x, w["l0.n1"], c["eps"]), "l0.attn", c["heads"], c["kv_heads"], False, 0, None)
        return x + swiglu(rms_norm(x, w["l0.n2"], c["eps"]), w["l0.mlp.gate_proj.weight"],
                          w["l0.mlp.up_proj.weight"], w["l0.mlp.down_proj.weight"])

    def routed(x):
        n = centered(x, "l1.n")
        return x + attention(n, "l1.attn", c["heads"], c["heads"], True, c["window"], 0.3) + experts(n)

    x = w["embed"][torch.tensor(ids)] + w["pos.table"][:T]
    x = routed(routed(dense(x)))
    return linear(centered(x, "norm"), w["head"])


def test_toy_parts_are_registered_built_and_stepped(tmp_path):
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine, StepEntry
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    _register()
    d = str(tmp_path / "toy_routed")
    write_random_model(config_from_json_dict(TOY), d, seed=11)
    w = read_weights(d)
    page = 4
    eng = Engine(d, EngineConfig(dtype="float32", page_size=page, num_pages=60, max_batch=3, device="cpu"),
                 ops=TorchOps())
    # three caches (one per schedule entry) in two groups: all keys; a window of them
    needs = eng.model.cache_needs()
    assert [n[0].window for n in needs] == [0, TOY["window"], TOY["window"]]
    assert len(eng.cache.groups) == 2
    g = torch.Generator().manual_seed(12)
    seqs = {k: torch.randint(0, TOY["vocab_size"], (n,), generator=g).tolist()
            for k, n in (("a", 41), ("b", 18), ("c", 29))}
    used = set()
    want = {k: plain_toy(w, v, used) for k, v in seqs.items()}
    assert used == set(range(TOY["experts"]))          # the routing is not degenerate: every expert gets tokens

    def close_enough(got, ref, what):
        assert (got.double().cpu() - ref).abs().max().item() < 1e-4, what

    for k, ids in seqs.items():                         # whole
        rc = eng.open(k)
        close_enough(eng.step([StepEntry(rc, ids, list(range(len(ids))))]), want[k], f"whole {k}")
        eng.close(rc)
    live = {k: eng.open(k) for k in seqs}                # mixed, in portions down to one token
    fed = {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    sizes = {"a": [7, 1, 2, 11], "b": [1, 3, 1], "c": [2, 13, 1]}
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
        eng.cache.check()
        turn += 1
    for k in seqs:
        close_enough(torch.cat(got[k]), want[k], f"mixed {k}")
    # the window's group gave pages back while the requests ran, the other group only at their end
    assert all(eng.cache.num_free(gi) == eng.cache.num_pages for gi in range(len(eng.cache.groups)))


def test_toy_model_generates_through_the_scheduler(tmp_path):
    """The same toy model behind the user-level entry point: greedy generation under a small token budget
    equals repeated whole-sequence evaluation of the plain computation."""
    from nanoinfer_b200 import Model
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    _register()
    d = str(tmp_path / "toy_routed")
    write_random_model(config_from_json_dict(TOY), d, seed=11)
    w = read_weights(d)
    model = Model(d, EngineConfig(dtype="float32", page_size=4, num_pages=40, max_batch=2, max_tokens_per_step=5,
                                  device="cpu"), ops=TorchOps())
    g = torch.Generator().manual_seed(13)
    prompt = torch.randint(0, TOY["vocab_size"], (17,), generator=g).tolist()
    ids, expect = list(prompt), []
    for _ in range(6):
        expect.append(int(plain_toy(w, ids)[-1].argmax()))
        ids.append(expect[-1])
    assert model.generate(prompt, max_tokens=6) == expect
    assert model.engine.cache.num_free(0) == 40


def test_toy_mixer_that_keeps_keys_alone_and_unequal_keys_and_values(tmp_path):
    """What a mixer keeps per token is a list of paged tensors: a toy mixer that keeps 32-bit keys alone in one
    layer and keys beside wider values in another (tests/toy_memory_mixer.py) is registered, built and stepped,
    whole and mixed in portions, with no change to the framework's files."""
    import toy_memory_mixer as toy
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    toy.register()
    d = str(tmp_path / "toy_memory")
    write_random_model(config_from_json_dict(toy.TOY), d, seed=17)
    eng = Engine(d, EngineConfig(dtype="float32", page_size=4, num_pages=22, max_batch=3, device="cpu"), ops=TorchOps())
    assert eng.storage.bytes_per_token() == 2 * (2 * 12 * 4) + (2 * 12 * 4 + 2 * 20 * 4)

    def close_enough(got, ref, what):
        assert (got.double().cpu() - ref).abs().max().item() < 1e-4, what
    toy.run_through_the_engine(eng, read_weights(d), close_enough)
