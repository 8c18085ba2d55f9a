"""``Qwen2ForCausalLM``: the Qwen2 / Qwen2.5 dense decoder as a plan over the shared parts.

Tensor names are the checkpoint's own (nanoinfer/weights.py:79-97 lists them):
``model.embed_tokens.weight``, ``model.layers.{i}.input_layernorm.weight``,
``model.layers.{i}.self_attn.{q,k,v,o}_proj.weight`` (+ ``.bias`` for q, k, v),
``model.layers.{i}.post_attention_layernorm.weight``, ``model.layers.{i}.mlp.{gate,up,down}_proj.weight``,
``model.norm.weight``, ``lm_head.weight`` (absent when the head is tied to the embedding).

Layer order, from cpp/src/model.cpp:361-406: for each layer pre-norm, attention, add, pre-norm,
SwiGLU, add; then the final norm and the head. With ``use_sliding_window`` layers with index
>= ``max_window_layers`` see only the last ``sliding_window`` keys; they form a cache group of
their own.
"""
from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..parts.attention import GroupedQueryAttention
from ..parts.embedding import LinearHead, TokenEmbedding
from ..parts.feedforward import SwiGLU
from ..parts.norm import RMSNorm
from ..parts.position import RotaryEncoding
from ..parts.spec import LayerSpec, ModelPlan, ScheduleEntry
from ..registry import register_architecture


def qwen2_plan(cfg: Qwen2Config) -> ModelPlan:
    h = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        window = cfg.sliding_window if (cfg.sliding_window and i >= cfg.max_window_layers) else 0
        layers.append(LayerSpec("pre_norm", {
            "mixer_norm": RMSNorm.spec(h, cfg.rms_norm_eps, f"{p}.input_layernorm.weight"),
            "mixer": GroupedQueryAttention.spec(
                f"{p}.self_attn", h, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                cfg.attention_bias, position="rotary", window=window),
            "ffn_norm": RMSNorm.spec(h, cfg.rms_norm_eps, f"{p}.post_attention_layernorm.weight"),
            "ffn": SwiGLU.spec(f"{p}.mlp", h, cfg.intermediate_size),
        }))
    embed_name = "model.embed_tokens.weight"
    head_name = embed_name if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=TokenEmbedding.spec(embed_name, cfg.vocab_size, h),
        positions={"rotary": RotaryEncoding.spec(cfg.head_dim, cfg.rope_theta, cfg.max_position_embeddings)},
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=RMSNorm.spec(h, cfg.rms_norm_eps, "model.norm.weight"),
        lm_head=LinearHead.spec(head_name, cfg.vocab_size, h),
        eos_token_id=cfg.eos_token_id,
        ignored_tensors=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_plan)
