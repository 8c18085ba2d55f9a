"""A plain, slow implementation of the Qwen2 decoder for whole sequences: no cache, no batching,
one function for each part, float64 by default. It shares no code with ``nanoinfer_b200``; it
reads ``config.json`` and ``model.safetensors`` by itself. Every function cites the lines of the
reference (AustinJiangg/nanoinfer) whose formula it restates.

Checked once against the reference's own Python model on tiny random models: see
``tests/golden/make_golden.py`` and ``tests/test_plain_vs_golden.py``.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# ----------------------------------------------------------------------------- reading a folder
def read_config(model_dir: str) -> dict:
    """The keys and defaults of nanoinfer/config.py:100-163, from config.json itself."""
    with open(os.path.join(model_dir, "config.json")) as f:
        d = json.load(f)
    heads = d["num_attention_heads"]
    theta = d.get("rope_theta")
    if theta is None:  # nanoinfer/config.py:13-29
        for k in ("rope_parameters", "rope_scaling"):
            if isinstance(d.get(k), dict) and d[k].get("rope_theta") is not None:
                theta = d[k]["rope_theta"]
                break
    ab = d.get("attention_bias")
    window = d.get("sliding_window") or 0
    if not d.get("use_sliding_window", False):  # nanoinfer/config.py:112-116
        window = 0
    return {
        "vocab": d["vocab_size"], "hidden": d["hidden_size"], "inter": d["intermediate_size"],
        "layers": d["num_hidden_layers"], "heads": heads,
        "kv_heads": d.get("num_key_value_heads") or heads,
        "head_dim": d.get("head_dim") or d["hidden_size"] // heads,
        "eps": d.get("rms_norm_eps", 1e-6), "theta": float(theta if theta is not None else 10000.0),
        "max_pos": d.get("max_position_embeddings", 4096),
        "tied": bool(d.get("tie_word_embeddings", False)),
        "bias": bool(ab) if ab is not None else d.get("model_type", "qwen2") == "qwen2",
        "window": int(window), "max_window_layers": int(d.get("max_window_layers") or 0),
    }


_NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "F64": np.float64, "I32": np.int32, "I64": np.int64}


def read_weights(model_dir: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    """Every tensor of model.safetensors as ``dtype`` (8-byte header length, JSON header, raw data)."""
    path = os.path.join(model_dir, "model.safetensors")
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, end = e["data_offsets"]
        arr = np.frombuffer(data[b:end], dtype=_NP[e["dtype"]]).reshape(e["shape"])
        if e["dtype"] == "BF16":
            t = torch.from_numpy((arr.astype(np.uint32) << 16).view(np.float32).copy())
        else:
            t = torch.from_numpy(arr.copy())
        out[name] = t.to(dtype)
    return out


# ----------------------------------------------------------------------------- the parts
def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x * 1/sqrt(mean(x^2) + eps) * gain   (cpp/src/ops.cpp:286-289; nanoinfer/layers.py:35-38)."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T + b with W [out, in]   (cpp/src/ops.cpp:42-69)."""
    y = x @ w.t()
    return y if b is None else y + b


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    """cos, sin [T, head_dim]: inv_freq_i = theta^(-2i/head_dim), angle = position * inv_freq_i, each
    frequency repeated in both halves, angles in float64   (cpp/src/ops.cpp:121-144)."""
    half = head_dim // 2
    inv_freq = 1.0 / (float(theta) ** (torch.arange(0, half, dtype=torch.float64, device=positions.device) * 2.0 / head_dim))
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, heads, head_dim]: out = x*cos + rotate_half(x)*sin, rotate_half = [-x2, x1]
    (cpp/src/ops.cpp:146-168; nanoinfer/layers.py:100-119)."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos[:, None, :].to(x.dtype) + rot * sin[:, None, :].to(x.dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0,
                     scale: Optional[float] = None) -> torch.Tensor:
    """q [T, heads, d], k, v [T, kv_heads, d] of ONE whole sequence (positions 0..T-1).
    Query head h uses kv head h // (heads/kv_heads) (cpp/src/paged.cpp:171; cpp/src/ops.cpp:193-204).
    scores = (q.k) * 1/sqrt(d), scale after the dot; query i sees keys 0..i; softmax with the max
    subtracted; out = sum p_j v_j   (cpp/src/ops.cpp:206-270). With a window w, query i sees keys j
    with i - w < j <= i."""
    T, heads, d = q.shape
    n_rep = heads // k.shape[1]
    scale = 1.0 / math.sqrt(float(d)) if scale is None else scale
    out = torch.empty_like(q)
    for h in range(heads):
        kh, vh = k[:, h // n_rep, :], v[:, h // n_rep, :]
        for i in range(T):
            lo = max(0, i - window + 1) if window else 0
            s = (kh[lo:i + 1] @ q[i, h]) * scale
            e = torch.exp(s - s.max())
            out[i, h] = (e / e.sum()) @ vh[lo:i + 1]
    return out


def causal_attention_fast(q, k, v, window: int = 0, scale: Optional[float] = None):
    """Same as ``causal_attention`` with a mask instead of loops (for long test sequences)."""
    T, heads, d = q.shape
    n_rep = heads // k.shape[1]
    scale = 1.0 / math.sqrt(float(d)) if scale is None else scale
    kk = k.repeat_interleave(n_rep, dim=1)   # out head j*n_rep + r <- kv head j
    vv = v.repeat_interleave(n_rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i = torch.arange(T, device=q.device)[:, None]
    j = torch.arange(T, device=q.device)[None, :]
    visible = j <= i
    if window:
        visible &= j > i - window
    s = s.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, vv)


def swiglu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + exp(-g))
    (cpp/src/model.cpp:217-223; cpp/src/ops.cpp:86-93)."""
    g = linear(x, wg)
    return linear(g / (1.0 + torch.exp(-g)) * linear(x, wu), wd)


def attention_part(x, w, prefix: str, cfg: dict, window: int, positions: torch.Tensor,
                   fast: bool = True) -> torch.Tensor:
    """Projections with bias, rotation of q and k, attention, output projection without bias
    (cpp/src/model.cpp:366-395)."""
    T = x.shape[0]
    g = lambda n: w.get(f"{prefix}.{n}")
    q = linear(x, g("q_proj.weight"), g("q_proj.bias")).view(T, cfg["heads"], cfg["head_dim"])
    k = linear(x, g("k_proj.weight"), g("k_proj.bias")).view(T, cfg["kv_heads"], cfg["head_dim"])
    v = linear(x, g("v_proj.weight"), g("v_proj.bias")).view(T, cfg["kv_heads"], cfg["head_dim"])
    cos, sin = rope_tables(positions, cfg["head_dim"], cfg["theta"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    a = (causal_attention_fast if fast else causal_attention)(q, k, v, window)
    return linear(a.reshape(T, -1), g("o_proj.weight"))


def block(x, w, i: int, cfg: dict, positions, fast: bool = True) -> torch.Tensor:
    """x = x + attn(norm(x)); x = x + ffn(norm(x))   (cpp/src/model.cpp:364-400)."""
    p = f"model.layers.{i}"
    window = cfg["window"] if (cfg["window"] and i >= cfg["max_window_layers"]) else 0
    h = rms_norm(x, w[f"{p}.input_layernorm.weight"], cfg["eps"])
    x = x + attention_part(h, w, f"{p}.self_attn", cfg, window, positions, fast)
    h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["eps"])
    return x + swiglu(h, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                      w[f"{p}.mlp.down_proj.weight"])


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], fast: bool = True) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence: embedding, blocks, final norm, head (tied: the
    embedding table)   (cpp/src/model.cpp:347-410; nanoinfer/model.py:33-89)."""
    table = w["model.embed_tokens.weight"]
    x = table[torch.tensor(ids, dtype=torch.long, device=table.device)]
    positions = torch.arange(len(ids), device=table.device)
    for i in range(cfg["layers"]):
        x = block(x, w, i, cfg, positions, fast)
    x = rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = table if cfg["tied"] else w["lm_head.weight"]
    return linear(x, head)


class PlainModel:
    """A folder's model, for whole sequences."""

    def __init__(self, model_dir: str, dtype=torch.float64, device="cpu"):
        """``device``: where torch computes (long test sequences may run the same plain formulas on a GPU)."""
        self.cfg = read_config(model_dir)
        self.w = {k: v.to(device) for k, v in read_weights(model_dir, dtype).items()}

    def logits(self, ids: List[int], fast: bool = True) -> torch.Tensor:
        return forward_logits(self.cfg, self.w, list(ids), fast)

    def greedy(self, prompt: List[int], n: int, eos: int = -1) -> List[int]:
        """Full recompute each step; EOS is not emitted (nanoinfer/generate.py:72-83)."""
        ids, out = list(prompt), []
        for _ in range(n):
            nxt = int(torch.argmax(self.logits(ids)[-1]))
            if eos >= 0 and nxt == eos:
                break
            out.append(nxt)
            ids.append(nxt)
        return out


# ----------------------------------------------------------------------------- sampling
def repetition_penalty(logits: np.ndarray, context: List[int], penalty: float) -> np.ndarray:
    """Seen tokens: s > 0 ? s / p : s * p   (nanoinfer/sampling.py:58-81)."""
    out = np.array(logits, dtype=np.float64, copy=True)
    if penalty == 1.0:
        return out
    seen = np.unique(np.asarray(context, dtype=np.int64))
    seen = seen[(seen >= 0) & (seen < out.shape[0])]
    s = out[seen]
    out[seen] = np.where(s > 0, s / penalty, s * penalty)
    return out


def top_k_filter(logits: np.ndarray, k: int) -> np.ndarray:
    """Below the k-th largest -> -inf; ties at the k-th value stay (nanoinfer/sampling.py:93-104)."""
    if not k or k <= 0:
        return logits
    k = min(k, logits.shape[0])
    kth = np.partition(logits, -k)[-k]
    return np.where(logits < kth, -np.inf, logits)


def top_p_filter(logits: np.ndarray, p: float) -> np.ndarray:
    """Sort descending, softmax, drop a token iff the probability of those BEFORE it exceeds p; the
    first stays (nanoinfer/sampling.py:107-123; cpp/python/ni/scheduler.py:115-119)."""
    if p is None or p >= 1.0:
        return logits
    order = np.argsort(-logits, kind="stable")
    srt = logits[order]
    e = np.exp(srt - srt.max())
    probs = e / e.sum()
    before = np.cumsum(probs) - probs
    out = logits.copy()
    out[order[before > p]] = -np.inf
    return out


def sampling_distribution(logits, context, temperature, top_k=0, top_p=1.0, penalty=1.0) -> np.ndarray:
    """Probabilities after penalty -> temperature -> top-k -> top-p -> softmax (nanoinfer/sampling.py:126-151)."""
    x = repetition_penalty(np.asarray(logits), context, penalty)
    x = x / temperature
    x = top_k_filter(x, top_k)
    x = top_p_filter(x, top_p)
    e = np.exp(x - x.max())
    return e / e.sum()


def greedy_pick(logits, context, penalty=1.0) -> int:
    """First index of the maximum after the penalty (nanoinfer/sampling.py:139-142)."""
    return int(np.argmax(repetition_penalty(np.asarray(logits), context, penalty)))
