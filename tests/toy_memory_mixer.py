"""A toy mixer that keeps OTHER things per token than attention's pair of equal keys and values, defined for the
tests only: in one layer it keeps keys alone (32-bit, whatever the compute dtype; the values are the keys), in the
next keys and values of different widths and dtypes. Its cache need is a list of paged tensors; the storage, the
page manager and the step function run it without knowing what the tensors mean, and no file of the framework
changes. The mixer does its own arithmetic with torch (it is a toy); its projections go through the kernel library.

``register()`` registers the parts and the architecture; ``plain(w, ids)`` is the whole-sequence float64 statement."""
from dataclasses import dataclass

import torch

from plain_qwen2 import linear, rms_norm, swiglu

TOY = {"architectures": ["ToyMemoryForCausalLM"], "vocab_size": 83, "hidden_size": 32, "max_pos": 96,
       "intermediate_size": 48, "heads": 2, "key_width": 12, "value_width": 20, "eps": 1e-5}


def register():
    from nanoinfer_b200.config.model_config import ModelConfig
    from nanoinfer_b200.parts.base import CacheNeed, Mixer, PagedTensor, as_tensor
    from nanoinfer_b200.parts.embedding import LinearHead, TokenEmbedding
    from nanoinfer_b200.parts.feedforward import SwiGLU
    from nanoinfer_b200.parts.norm import RMSNorm
    from nanoinfer_b200.parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, TensorSpec
    from nanoinfer_b200.registry import register_architecture, register_part

    class MemoryMixer(Mixer):
        """scores = q . k / sqrt(key_width) over the request's positions so far, softmax, weighted sum of the
        values (of the keys themselves when ``value_width`` is 0), output projection, added to the residual stream.
        params: hidden, heads, key_width, value_width. Keys are cached in 32-bit, values in the compute dtype."""

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            p = spec.params
            self.hidden, self.heads, self.kw, self.vw = int(p["hidden"]), int(p["heads"]), int(p["key_width"]), int(p["value_width"])
            self.w_q, self.w_k, self.w_o = rt.matrix(tensors["q"]), rt.matrix(tensors["k"]), rt.matrix(tensors["o"])
            self.w_v = rt.matrix(tensors["v"]) if self.vw else None

        def cache_need(self):
            kept = [PagedTensor("keys", self.heads, self.kw, torch.float32)]
            if self.vw:
                kept.append(PagedTensor("values", self.heads, self.vw))
            return CacheNeed(tuple(kept))

        def _project(self, h, w):
            out = torch.empty((h.shape[0], w.shape[0]), dtype=torch.float32, device=h.device)
            self.ops.linear(h, w, None, out, "f32")
            return out

        def forward(self, h, residual32, ctx, cache):
            h = as_tensor(h).contiguous()
            q = self._project(h, self.w_q).view(-1, self.heads, self.kw)
            k = self._project(h, self.w_k).view(-1, self.heads, self.kw)
            v = self._project(h, self.w_v).view(-1, self.heads, self.vw) if self.vw else None
            keys, values = cache.pages["keys"], cache.pages.get("values")
            assert keys.dtype == torch.float32 and (values is None or values.dtype == self.rt.dtype)
            assert set(cache.pages) == ({"keys", "values"} if self.vw else {"keys"})
            mixed = torch.empty((h.shape[0], self.heads * (self.vw or self.kw)), dtype=self.rt.dtype, device=h.device)
            start = 0
            for r, (q_len, held) in enumerate(zip(ctx.host.q_lens, ctx.host.ctx_lens)):
                table = cache.block_table[r].long()
                pos = torch.arange(held - q_len, held, device=h.device)
                keys[table[pos // cache.page_size], :, pos % cache.page_size] = k[start:start + q_len]
                if v is not None:
                    values[table[pos // cache.page_size], :, pos % cache.page_size] = v[start:start + q_len].to(values.dtype)
                every = torch.arange(held, device=h.device)
                all_k = keys[table[every // cache.page_size], :, every % cache.page_size].double()      # [held, heads, kw]
                all_v = all_k if v is None else values[table[every // cache.page_size], :, every % cache.page_size].double()
                s = torch.einsum("thd,shd->hts", q[start:start + q_len].double(), all_k) / self.kw ** 0.5
                s = s.masked_fill(every[None, None, :] > pos[None, :, None], float("-inf"))
                o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), all_v)
                mixed[start:start + q_len] = o.reshape(q_len, -1).to(mixed.dtype)
                start += q_len
            self.ops.linear(mixed, self.w_o, None, residual32, "add")

    register_part("toy_memory", MemoryMixer)

    @dataclass(frozen=True)
    class ToyMemoryConfig(ModelConfig):
        intermediate_size: int = 0
        heads: int = 0
        key_width: int = 0
        value_width: int = 0
        eps: float = 1e-6

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyMemoryForCausalLM", model_type="toy_memory", vocab_size=d["vocab_size"],
                       hidden_size=d["hidden_size"], num_hidden_layers=2, max_position_embeddings=d["max_pos"],
                       tie_word_embeddings=False, eos_token_id=-1, intermediate_size=d["intermediate_size"],
                       heads=d["heads"], key_width=d["key_width"], value_width=d["value_width"], eps=d["eps"])

        def to_json_dict(self):
            return {"architectures": ["ToyMemoryForCausalLM"], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "max_pos": self.max_position_embeddings, "intermediate_size": self.intermediate_size, "heads": self.heads,
                    "key_width": self.key_width, "value_width": self.value_width, "eps": self.eps}

    def plan(c):
        h = c.hidden_size

        def mixer(i, vw):
            t = {"q": TensorSpec(f"l{i}.mem.q", (c.heads * c.key_width, h)), "k": TensorSpec(f"l{i}.mem.k", (c.heads * c.key_width, h)),
                 "o": TensorSpec(f"l{i}.mem.o", (h, c.heads * (vw or c.key_width)))}
            if vw:
                t["v"] = TensorSpec(f"l{i}.mem.v", (c.heads * vw, h))
            return PartSpec("toy_memory", {"hidden": h, "heads": c.heads, "key_width": c.key_width, "value_width": vw}, t)

        def layer(i, vw):
            return LayerSpec("pre_norm", {
                "mixer_norm": RMSNorm.spec(h, c.eps, f"l{i}.n1"), "mixer": mixer(i, vw),
                "ffn_norm": RMSNorm.spec(h, c.eps, f"l{i}.n2"), "ffn": SwiGLU.spec(f"l{i}.mlp", h, c.intermediate_size)})
        return ModelPlan(
            architecture=c.architecture, hidden_size=h, vocab_size=c.vocab_size, max_position_embeddings=c.max_position_embeddings,
            embedding=TokenEmbedding.spec("embed", c.vocab_size, h), positions={},
            layers=[layer(0, 0), layer(1, c.value_width)], schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)],
            final_norm=RMSNorm.spec(h, c.eps, "norm"), lm_head=LinearHead.spec("head", c.vocab_size, h))

    register_architecture("ToyMemoryForCausalLM", ToyMemoryConfig, plan)


def plain(w, ids):
    """Whole sequence, float64, no cache."""
    c = TOY
    T = len(ids)
    x = w["embed"][torch.tensor(ids)]
    causal = torch.ones(T, T).tril().bool()

    def layer(i, x, vw):
        h = rms_norm(x, w[f"l{i}.n1"], c["eps"])
        q = linear(h, w[f"l{i}.mem.q"]).view(T, c["heads"], c["key_width"])
        k = linear(h, w[f"l{i}.mem.k"]).view(T, c["heads"], c["key_width"])
        v = linear(h, w[f"l{i}.mem.v"]).view(T, c["heads"], vw) if vw else k
        s = torch.einsum("thd,shd->hts", q, k) / c["key_width"] ** 0.5
        o = torch.einsum("hts,shd->thd", torch.softmax(s.masked_fill(~causal, float("-inf")), -1), v)
        x = x + linear(o.reshape(T, -1), w[f"l{i}.mem.o"])
        h = rms_norm(x, w[f"l{i}.n2"], c["eps"])
        return x + swiglu(h, w[f"l{i}.mlp.gate_proj.weight"], w[f"l{i}.mlp.up_proj.weight"], w[f"l{i}.mlp.down_proj.weight"])

    x = layer(0, layer(1, layer(0, x, 0), c["value_width"]), 0)
    return linear(rms_norm(x, w["norm"], c["eps"]), w["head"])


def run_through_the_engine(eng, w, close_enough):
    """Whole, then three requests mixed in portions with so few pages that they are used again."""
    from nanoinfer_b200.engine import StepEntry
    # three caches (one per schedule entry) in two groups: keys alone; keys and wider values
    needs = [n[0] for n in eng.model.cache_needs()]
    assert [[t.name for t in n.tensors] for n in needs] == [["keys"], ["keys", "values"], ["keys"]]
    assert len(eng.cache.groups) == 2
    g = torch.Generator().manual_seed(21)
    seqs = {k: torch.randint(0, TOY["vocab_size"], (n,), generator=g).tolist() for k, n in (("a", 33), ("b", 14), ("c", 26))}
    want = {k: plain(w, v) for k, v in seqs.items()}
    for k, ids in seqs.items():
        rc = eng.open(k)
        close_enough(eng.step([StepEntry(rc, ids, list(range(len(ids))))]), want[k], f"whole {k}")
        eng.close(rc)
    live = {k: eng.open(k) for k in seqs}
    fed, got = {k: 0 for k in seqs}, {k: [] for k in seqs}
    sizes = {"a": [6, 1, 2, 9], "b": [1, 4, 1], "c": [2, 11, 1]}
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
    assert all(eng.cache.num_free(gi) == eng.cache.num_pages for gi in range(len(eng.cache.groups)))
