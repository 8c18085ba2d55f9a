#!/usr/bin/env python3
"""Headline benchmark: decode throughput of the Qwen2.5-0.5B shape (random weights, bfloat16) at a
batch of 8 and a context of 4,096 tokens on ONE B200, with prefill of 2,048 tokens, the decode
roofline and batch 1 / 64 points on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 0.5b|1.5b|7b]

A "step" is one decode step of the whole batch. ``value`` is decoded tokens per second over K steps
timed with CUDA events on the launching stream; ``e2e`` is the same through the Python entry point
(the scheduler with lookahead, as ``Model.generate`` and the serve command run it: host token ids in,
sampled ids out, every step; each step's inputs go up from pinned memory and each step's tokens come
back, the latter while the next step already runs). Inputs larger than L2: every step
reads all weights (~1 GB) and the live requests' cache, several times the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the benchmark model: the Qwen2.5-0.5B shape, the reference's headline configuration.
MODEL = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 24, "hidden_size": 896,
    "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 4864,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "use_sliding_window": False, "hidden_act": "silu",
    "torch_dtype": "bfloat16",
}
# the other sizes of the family that the baseline names; --shape selects one (the default run is the 0.5B shape)
SHAPES = {
    "0.5b": {},
    "1.5b": {"num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
             "head_dim": 128, "intermediate_size": 8960},
    "7b": {"num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
           "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064, "tie_word_embeddings": False},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            found = 0
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                v = d.get(k)
                if isinstance(v, dict):             # {"value": ...} is read as well as a bare number
                    v = v.get("value")
                if isinstance(v, str):
                    v = float(v)
                if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                    out[k] = float(v)
                    found += 1
            if found:
                out["source"] = "measured" if found == 3 else "measured (partly fallback)"
                return out
        except (OSError, ValueError, AttributeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(layers: int) -> dict:
    """Matrix parameters, bytes a decode step has to read, FLOPs of a prefill, from the sizes."""
    m = MODEL
    h, inter, v = m["hidden_size"], m["intermediate_size"], m["vocab_size"]
    nq, nkv, hd = m["num_attention_heads"], m["num_key_value_heads"], m["head_dim"]
    per_layer = (nq + 2 * nkv) * hd * h + h * nq * hd + 3 * h * inter
    return {
        "kinds": {"qkv": (nq + 2 * nkv) * hd * h, "o_proj": h * nq * hd, "gate_up": 2 * h * inter, "down": h * inter,
                  "lm_head": v * h},
        "attention_flops": lambda t: 4.0 * nq * hd * t * (t + 1) / 2.0,           # one layer, a prompt of t tokens
        "kv_bytes_per_token_layer": 2 * nkv * hd * 2,
        "per_layer_params": per_layer,
        "weight_bytes": 2 * (layers * per_layer + v * h),           # every matrix once, head included
        "kv_bytes_per_token": 2 * layers * nkv * hd * 2,
        "prefill_flops": lambda t: 2.0 * t * layers * per_layer + 2.0 * v * h
        + layers * 4.0 * nq * hd * t * (t + 1) / 2.0,
    }


def _kind_of(kernel: str, what: str, state: dict) -> str:
    """Which part of a layer a launch is, from its kernel and its place in the layer's order: norm, q/k/v,
    (rotation), attention, output projection, norm, gate/up, down."""
    w = what.lower()
    if "attention" in kernel or "attention" in w:
        state["after_attention"] = True
        return "attention"
    if "rmsnorm" in kernel or "rmsnorm" in w:
        return "rmsnorm"
    if "rope" in kernel or "rope" in w:
        return "rope_store"
    if "embed" in kernel or "embed" in w:
        return "embed"
    if "argmax" in kernel or "argmax" in w:
        return "argmax"
    if "gemm" in kernel or "linear" in w or "q/k/v" in w:
        tag = state.get("tag")
        if tag == "swiglu":
            state["after_gate_up"] = True
            return "gate_up"
        if tag == "f32":
            return "lm_head"
        if tag in ("qkv", "store"):
            return "qkv"
        if state.pop("after_attention", False):
            return "o_proj"
        state.pop("after_gate_up", None)
        return "down"
    return kernel or what


def _rows_from_notes(notes):
    """{kind: [microseconds]} and the step's length from the kernels' timer notes: a kernel's share runs from the
    moment its wait for the earlier kernels ended to the moment the next kernel's did."""
    epi = {0: "store", 1: "add", 2: "f32", 3: "swiglu", 4: "qkv"}
    starts = [(t, k, tag) for t, k, tag, phase in notes if phase == 1]
    ends = [t for t, _, _, phase in notes if phase == 2]
    if len(starts) < 2 or not ends:
        return {}, 0.0
    state, rows = {}, {}
    for i, (t, kernel, tag) in enumerate(starts):
        state["tag"] = epi.get(tag) if kernel.startswith("gemm") else None
        kind = _kind_of(kernel, "", state)
        t_next = starts[i + 1][0] if i + 1 < len(starts) else max(ends)
        rows.setdefault(kind, []).append((t_next - t) / 1e3)
    return rows, (max(ends) - starts[0][0]) / 1e3


def decode_breakdown(engine, ops, reqs, rng, vocab, batch, mean_ctx, nums, pk) -> dict:
    """Where the time of ONE decode step goes, from the kernels' own notes of the GPU timer (they keep the overlap
    of dependent launches inside the captured graph): a kernel's share is the time from the moment its wait for the
    earlier kernels ended to the moment the next kernel's did. Bytes: the weights of its product once, or the
    cached keys and values of the live requests; the fraction is of the measured copy bandwidth."""
    import torch
    from nanoinfer_b200.engine import StepEntry
    base = [rc.length for rc in reqs]
    ops.timeline_start()
    engine.reset_graphs()

    def one():
        engine.step([StepEntry(rc, [int(rng.integers(0, vocab))], [0]) for rc in reqs], borrow_logits=True)
    for _ in range(4):
        one()
    ops.timeline_clear()
    one()
    notes = ops.timeline()
    ops.timeline_stop()
    engine.reset_graphs()
    for rc, n in zip(reqs, base):
        engine.truncate(rc, n)
    rows, step_us = _rows_from_notes(notes)
    if not rows:
        return {}
    bytes_of = {k: 2.0 * v for k, v in nums["kinds"].items()}
    bytes_of["attention"] = batch * mean_ctx * nums["kv_bytes_per_token_layer"]
    out = {"step_us": round(step_us, 1)}
    for kind, us in rows.items():
        mean = sum(us) / len(us)
        row = {"n": len(us), "us": round(mean, 2), "share": round(sum(us) / step_us, 3)}
        if kind in bytes_of:
            gbs = bytes_of[kind] / (mean * 1e-6) / 1e9
            row.update({"mb": round(bytes_of[kind] / 1e6, 2), "gbs": round(gbs, 0), "frac": round(gbs / pk["hbm_gbs"], 3)})
        out[kind] = row
    return out


def prefill_breakdown(engine, ops, rng, vocab, t_pre, nums, pk) -> dict:
    """Where the time of one prompt portion goes, from the kernels' own notes of the GPU timer as in
    ``decode_breakdown`` (the third step of the shape: a replay of its captured graph, so the kernels overlap as
    they do in production and the host is not in the way). FLOPs of a product: 2 x tokens x weights; of the
    attention: 4 x heads x head size x t(t+1)/2; the fraction is of the measured cuBLAS burst throughput."""
    import numpy as np
    import torch
    from nanoinfer_b200.engine import StepEntry
    ops.timeline_start()
    engine.reset_graphs()
    rc = engine.open("breakdown")
    ids = rng.integers(0, vocab, t_pre).astype(np.int32)
    for i in range(3):
        if i == 2:
            ops.timeline_clear()
        engine.step([StepEntry(rc, ids, [t_pre - 1])])
        torch.cuda.synchronize()
        engine.truncate(rc, 0)
    notes = ops.timeline()
    ops.timeline_stop()
    engine.reset_graphs()
    engine.close(rc)
    rows, total = _rows_from_notes(notes)
    if not rows:
        return {}
    flops_of = {k: 2.0 * t_pre * v for k, v in nums["kinds"].items()}
    flops_of["lm_head"] = 2.0 * nums["kinds"]["lm_head"]          # one wanted row
    flops_of["attention"] = nums["attention_flops"](t_pre)
    out = {"step_us": round(total, 1)}
    for kind, us in rows.items():
        mean = sum(us) / len(us)
        row = {"n": len(us), "us": round(mean, 2), "share": round(sum(us) / total, 3)}
        if kind in flops_of and kind != "lm_head":
            tf = flops_of[kind] / (mean * 1e-6) / 1e12
            row.update({"gflop": round(flops_of[kind] / 1e9, 2), "tflops": round(tf, 0), "frac": round(tf / pk["bf16_tflops"], 3)})
        out[kind] = row
    return out


def run_ours(args) -> dict:
    import numpy as np
    import torch
    from nanoinfer_b200 import Request, Scheduler, load_model
    from nanoinfer_b200.engine import StepEntry
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model

    pk = peaks()
    layers = args.layers or MODEL["num_hidden_layers"]
    cfg_json = dict(MODEL, num_hidden_layers=layers)
    nums = model_numbers(layers)
    ctx, batch, steps, warmup = args.context, args.batch, args.steps, max(3, args.warmup)
    rng = np.random.default_rng(0)
    vocab = MODEL["vocab_size"]

    tmp = tempfile.mkdtemp(prefix="nanoinfer_b200_bench_")
    t0 = time.time()
    write_random_model(config_from_json_dict(cfg_json), tmp, seed=0)
    max_batch = max(batch, 64)
    page = 16
    num_pages = max_batch * (-(-ctx // page) + 1) + 8
    try:
        model = load_model(tmp, dtype="bfloat16", page_size=page, num_pages=num_pages, max_batch=max_batch,
                           max_tokens_per_step=4096, cuda_graphs=not args.no_graphs)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)      # the weights are on the device now; the folder can be gigabytes
    engine, ops = model.engine, model.engine.rt.ops
    print(f"[bench] model ready in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    if args.only == "serve":
        return serve_workload(model, args, rng, vocab, layers)

    def fill(n_req: int, length: int):
        """n_req live requests holding ``length`` random tokens each."""
        reqs = [engine.open(f"b{n_req}_{i}") for i in range(n_req)]
        for rc in reqs:
            done = 0
            while done < length:
                n = min(2048, length - done)
                engine.step([StepEntry(rc, rng.integers(0, vocab, n).tolist(), [])])
                done += n
        return reqs

    def decode_timed(reqs, n_warm: int, n_steps: int, min_seconds: float = 0.5, max_repeats: int = 40):
        """Device time of n_steps decode steps (one token for every request, greedy pick on the device), measured
        again and again FROM THE SAME CONTEXT (the requests forget the n_steps positions in between) until
        min_seconds have been timed. Returns (median ms per step, launches of one region, ms per step of every
        repeat)."""
        out = torch.empty(len(reqs), dtype=torch.int32, device=engine.device)
        toks = [rng.integers(0, vocab, len(reqs)).tolist() for _ in range(n_warm + n_steps)]

        def one(i):
            logits = engine.step([StepEntry(rc, [toks[i][j]], [0]) for j, rc in enumerate(reqs)], borrow_logits=True)
            ops.argmax(logits, out)
        for i in range(n_warm):
            one(i)
        torch.cuda.synchronize()
        base = [rc.length for rc in reqs]
        per_step, launches, total = [], 0, 0.0
        while total < min_seconds * 1e3 and len(per_step) < max_repeats:
            l0 = ops.launches + engine.graph_launches
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(n_warm, n_warm + n_steps):
                one(i)
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end)
            launches = ops.launches + engine.graph_launches - l0
            per_step.append(ms / n_steps)
            total += ms
            for rc, n in zip(reqs, base):
                engine.truncate(rc, n)
        return statistics.median(per_step), launches, per_step

    def close_all(reqs):
        for rc in reqs:
            engine.close(rc)

    # ---- prefill of 2,048 tokens ----------------------------------------------------------
    t_pre = args.prefill_tokens
    pre_ms = []
    for i in range((3 + 7) if args.only != "decode" else 0):
        rc = engine.open(f"p{i}")
        ids = rng.integers(0, vocab, t_pre).astype(np.int32)        # host memory, as a tokenizer's array would be
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step([StepEntry(rc, ids, [t_pre - 1])])
        e.record()
        torch.cuda.synchronize()
        if i >= 3:
            pre_ms.append(s.elapsed_time(e))
        engine.close(rc)
    prefill = None
    if pre_ms:
        pre = statistics.median(pre_ms)
        prefill = {"value": round(t_pre / (pre / 1e3), 1), "tokens": t_pre, "ms": round(pre, 3),
                   "frac": round(nums["prefill_flops"](t_pre) / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "peak": f"{pk['bf16_tflops']:.0f} TFLOP/s, cuBLAS bf16 burst, {pk['source']}"}
    prefill_kernels = None
    if pre_ms and args.breakdown:
        prefill_kernels = prefill_breakdown(engine, ops, rng, vocab, t_pre, nums, pk)

    if args.only == "prefill":
        out = {"impl": "ours", "only": "prefill", "prefill": prefill,
               "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": layers}}
        if prefill_kernels:
            out["kernels"] = {"prefill": prefill_kernels}
        return out

    # The clocks are sampled from before the warm-up to the end of the timed regions.
    sampler = ClockSampler()
    sampler.__enter__()
    # ---- decode points at batch 1 and 64 --------------------------------------------------
    points = {}
    for b in ((1, 64) if args.only == "all" else ()):
        n_w, n_s = 4, min(steps, 32)
        reqs = fill(b, ctx - n_w - n_s - 1)
        ms, _, _ = decode_timed(reqs, n_w, n_s, min_seconds=0.15)
        points[f"decode_b{b}"] = round(b / (ms / 1e3), 1)
        close_all(reqs)

    # ---- the headline: batch 8 (default), device-timed -------------------------------------
    reqs = fill(batch, ctx - warmup - steps - 1)
    ms_step, launches, repeats = decode_timed(reqs, warmup, steps)
    sampler.__exit__()
    clocks = sampler.summary()
    mean_ctx = ctx - steps / 2.0
    step_bytes = nums["weight_bytes"] + batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    kernels = None
    if args.breakdown:
        kernels = {"decode": decode_breakdown(engine, ops, reqs, rng, vocab, batch, mean_ctx, nums, pk)}
        if prefill_kernels is not None:
            kernels["prefill"] = prefill_kernels
    close_all(reqs)
    if args.only == "decode":
        out = {"impl": "ours", "only": "decode", "value": round(batch / (ms_step / 1e3), 1), "ms_per_step": round(ms_step, 4),
               "gpu_launches": launches, "repeats": len(repeats), "clocks": clocks,
               "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                            "frac": round(achieved / pk["hbm_gbs"], 4)},
               "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": layers, "global_batch": batch, "seq_len": ctx}}
        if kernels:
            out["kernels"] = kernels
        return out

    # ---- end to end through the Python entry point (scheduler) -----------------------------
    sched = Scheduler(model, max_batch=batch, max_tokens_per_step=4096, lookahead=True)
    # Requests admitted first decode while the later prompts are still being prefilled (about one step per
    # prompt), so they are ahead by up to `batch` tokens when timing starts; nobody may finish, and nobody may
    # leave the context (and with it the captured graph's bucket), before the timed steps end.
    prompt_len = ctx - warmup - steps - 2 * batch - 8
    for i in range(batch):
        sched.add(Request(f"e{i}", rng.integers(0, vocab, prompt_len).tolist(), max_tokens=ctx))
    while any(s.pending > 1 for s in sched.running) or sched.waiting:
        sched.step()
    for _ in range(warmup):
        sched.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(steps):
        n_tok += len(sched.step().entries)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = engine.last_h2d_bytes
    for rid in [s.req.request_id for s in sched.running]:
        sched.cancel(rid)
    e2e = {"value": round(n_tok / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": 4 * batch, "ms_per_step": round(dt / steps * 1e3, 4)}

    value = batch / (ms_step / 1e3)
    extra = {"kernels": kernels} if kernels else {}
    return {
        **extra,
        "metric": f"decode tok/s at batch {batch} (Qwen2.5-{args.shape.upper()} shape, context {ctx})", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and random token ids", "impl": "ours",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": layers, "layers_full": MODEL["num_hidden_layers"],
                   "hidden": MODEL["hidden_size"], "heads": MODEL["num_attention_heads"],
                   "kv_heads": MODEL["num_key_value_heads"], "head_dim": MODEL["head_dim"],
                   "intermediate": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"], "tied_head": MODEL["tie_word_embeddings"],
                   "global_batch": batch, "seq_len": ctx, "page_size": page, "prefill_tokens": t_pre,
                   "parallelism": "single-gpu", "l2": f"inputs larger than L2 (weights {nums['weight_bytes'] / 1e9:.1f} GB per step)",
                   "peaks": pk["source"], "timed_regions": len(repeats)},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }


def serve_workload(model, args, rng, vocab: int, layers: int) -> dict:
    """A mixed continuous batch through the scheduler: 64 requests with prompts of 128 to 2,048 random ids
    and 256 decoded tokens each, all queued at once; prompts are cut under a budget of 2,048 tokens a step
    and run beside the decoding requests. Wall-clock time from the first step to the last token, host ids in
    and sampled ids out; the first run warms up (it captures the decode graphs), the second is timed."""
    import torch
    from nanoinfer_b200 import Request, Scheduler
    n_req, new_tokens, budget = 64, 256, 2048
    lens = rng.integers(128, 2049, n_req)

    def run():
        sched = Scheduler(model, max_batch=n_req, max_tokens_per_step=budget, lookahead=True)
        for i, n in enumerate(lens):
            sched.add(Request(f"r{i}", rng.integers(0, vocab, int(n)).tolist(), max_tokens=new_tokens))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        t_prompts, steps_prompts = None, 0
        while sched.has_work():
            plan = sched.step()
            if t_prompts is None and not sched.waiting and all(e.count == 1 for e in plan.entries):
                torch.cuda.synchronize()            # every prompt is in the cache: the rest is decoding
                t_prompts, steps_prompts = time.perf_counter() - t0, sched.steps
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        generated = sum(len(v) for v in sched.finished.values())
        return dt, generated, sched.steps, t_prompts, steps_prompts, sched.preemptions

    run()
    dt, generated, steps, t_prompts, steps_prompts, preemptions = run()
    return {"impl": "ours", "only": "serve", "metric": "generated tok/s of a continuous batch (64 requests, prompts 128-2048, 256 new tokens each)",
            "value": round(generated / dt, 1), "unit": "tokens/s", "ms_total": round(dt * 1e3, 1), "steps": steps,
            "total_tokens_per_s": round((generated + int(lens.sum())) / dt, 1),
            "prompt_phase_ms": round(t_prompts * 1e3, 1), "prompt_phase_steps": steps_prompts,
            "decode_ms_per_step": round((dt - t_prompts) * 1e3 / max(1, steps - steps_prompts), 4),
            "preemptions": preemptions,
            "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": layers, "requests": n_req,
                       "prompt_tokens": int(lens.sum()), "new_tokens": new_tokens, "max_tokens_per_step": budget,
                       "page_size": 16}}


def run_reference(args) -> dict:
    """The unmodified reference (its Python model, installed under baseline/_ref) on the same workload:
    random weights of the same shape, batch 8 decode at context 4096 through ``Model.forward`` with its
    ``KVCache`` and ``sample_next_token``, the calls its own generate loop makes (nanoinfer/generate.py:72-83)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "nanoinfer")):
        return {"impl": "reference", "unavailable": "baseline/_ref/nanoinfer is not installed (pip install --no-deps --target baseline/_ref <reference>)"}
    sys.path.insert(0, ref_dir)
    try:
        import torch
        from nanoinfer.config import ModelConfig
        from nanoinfer.model import Model
        from nanoinfer.sampling import SamplingParams, sample_next_token
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"cannot import the reference: {type(e).__name__}: {e}"}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    m = MODEL
    layers = args.layers or m["num_hidden_layers"]
    ctx, batch, steps, warmup = args.context, args.batch, args.steps, max(3, args.warmup)
    cfg = ModelConfig(vocab_size=m["vocab_size"], hidden_size=m["hidden_size"], intermediate_size=m["intermediate_size"],
                      num_layers=layers, num_attention_heads=m["num_attention_heads"],
                      num_kv_heads=m["num_key_value_heads"], head_dim=m["head_dim"], rms_norm_eps=m["rms_norm_eps"],
                      rope_theta=m["rope_theta"], max_position_embeddings=m["max_position_embeddings"],
                      tie_word_embeddings=True)
    torch.manual_seed(0)
    model = Model(cfg).to(device="cuda", dtype=torch.bfloat16).eval()
    model.lm_head.weight = model.embed_tokens.weight
    cache = model.init_cache(batch, ctx)
    g = torch.Generator(device="cpu").manual_seed(0)
    filled, target = 0, ctx - warmup - steps - 1
    with torch.no_grad():
        while filled < target:
            n = min(512, target - filled)
            model(torch.randint(0, m["vocab_size"], (batch, n), generator=g).cuda(), cache=cache)
            filled += n
        params = SamplingParams()
        pinned = torch.empty((batch, 1), dtype=torch.long).pin_memory()

        def one():
            pinned.copy_(torch.randint(0, m["vocab_size"], (batch, 1), generator=g))
            cur = pinned.to("cuda", non_blocking=True)
            logits = model(cur, cache=cache)[:, -1, :]
            return [sample_next_token(logits[b], params) for b in range(batch)]
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler() as cs:
            t0 = time.perf_counter()
            s.record()
            for _ in range(steps):
                one()
            e.record()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        ms = s.elapsed_time(e) / steps
    return {
        "metric": "decode tok/s at batch 8 (Qwen2.5-0.5B shape, context 4096)", "value": round(batch / (ms / 1e3), 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights and random token ids", "impl": "reference",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": layers, "layers_full": m["num_hidden_layers"],
                   "hidden": m["hidden_size"], "heads": m["num_attention_heads"], "kv_heads": m["num_key_value_heads"],
                   "head_dim": m["head_dim"], "intermediate": m["intermediate_size"], "vocab": m["vocab_size"],
                   "tied_head": m["tie_word_embeddings"], "global_batch": batch, "seq_len": ctx, "page_size": 16,
                   "prefill_tokens": args.prefill_tokens, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights 1.0 GB per step)", "peaks": peaks()["source"], "timed_regions": 1},
        "engine": "reference Python model (torch, CUDA)",
        "clocks": cs.summary(),
        "e2e": {"value": round(batch * steps / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": 8 * batch,
                "d2h_bytes_per_step": 8 * batch},
        "gpu_launches": 0,
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0 = all)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profilers that filter by kernel name)")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode", "serve"],
                    help="measure one part only (for profiling small cases); the JSON line then lacks the rest. "
                         "'serve' runs the continuous-batching workload (64 requests through the scheduler) instead")
    ap.add_argument("--breakdown", action="store_true",
                    help="add a 'kernels' block: where the time of a decode step and of a prompt portion goes, kernel kind by "
                         "kind, with bytes or FLOPs and the fraction of the measured peak")
    ap.add_argument("--shape", default="0.5b", choices=sorted(SHAPES), help="layer sizes: the family's 0.5B (default), 1.5B or 7B")
    args = ap.parse_args()
    MODEL.update(SHAPES[args.shape])
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"unavailable": f"this engine runs on one GPU; --gpus {args.gpus} is not supported",
                              "n_gpus": args.gpus}))
        return 2
    if args.steps + args.warmup + 2 >= args.context:
        print(json.dumps({"unavailable": "steps + warmup must be smaller than the context"}))
        return 2
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
