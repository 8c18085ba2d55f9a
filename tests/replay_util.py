"""Building traces for bin/trace_run, running it as a user would (a subprocess fed line by line),
and collecting the logits it writes."""
import json
import os
import subprocess
import sys
from typing import Dict, List, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Trace:
    """Steps, and for every wanted row which (request, position) it is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.rows: List[List[Tuple[str, int]]] = []
        self.fed: Dict[str, int] = {}
        self.live_tokens: Dict[str, int] = {}
        self.max_tokens = 0

    def step(self, portions: List[Tuple[str, List[int], List[int]]], end: List[str] = ()):
        """portions: (request id, tokens, wanted places among them)."""
        entries, rows = [], []
        for rid, toks, want in portions:
            base = self.fed.get(rid, 0)
            entries.append({"id": rid, "tokens": list(map(int, toks)), "want": list(map(int, want))})
            rows += [(rid, base + w) for w in want]
            self.fed[rid] = base + len(toks)
            self.live_tokens[rid] = self.fed[rid]
        held = sum(-(-n // 64) * 64 for n in self.live_tokens.values())
        self.max_tokens = max(self.max_tokens, held)
        for rid in end:
            self.live_tokens.pop(rid, None)
        self.steps.append({"step": len(self.steps), "entries": entries, "end": list(end)})
        self.rows.append(rows)


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int = None,
              page_size: int = None, timeout: float = 900.0) -> Dict[Tuple[str, int], List[np.ndarray]]:
    """Runs bin/trace_run; feeds the next step only after ``done <step>``. Returns for each
    (request, position) the list of logit rows written for it (one per time it was wanted)."""
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens if max_tokens is not None else trace.max_tokens)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        for st in trace.steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {st['step']}", f"trace_run said {line!r} at step {st['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    out: Dict[Tuple[str, int], List[np.ndarray]] = {}
    for st, rows in zip(trace.steps, trace.rows):
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if not rows:
            assert not os.path.exists(path)
            continue
        arr = np.fromfile(path, dtype="<f4")
        assert arr.size % len(rows) == 0
        arr = arr.reshape(len(rows), -1)
        for key, row in zip(rows, arr):
            out.setdefault(key, []).append(row)
    return out


def add_whole(trace: Trace, rid: str, ids: List[int]):
    trace.step([(rid, ids, list(range(len(ids))))], end=[rid])


def add_decode_tail(trace: Trace, rid: str, ids: List[int], tail: int = 32):
    head = max(1, len(ids) - tail)
    trace.step([(rid, ids[:head], [head - 1])])
    for i in range(head, len(ids)):
        trace.step([(rid, [ids[i]], [0])], end=[rid] if i == len(ids) - 1 else [])
    if head == len(ids):
        trace.step([], end=[rid])


def add_portions(trace: Trace, rid: str, ids: List[int], sizes=(2, 3, 5, 7, 11, 13, 2, 17, 4)):
    pos, k = 0, 0
    while pos < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - pos)
        k += 1
        last = pos + n == len(ids)
        trace.step([(rid, ids[pos:pos + n], list(range(n)))], end=[rid] if last else [])
        pos += n


def add_mixed(trace: Trace, prompts: Dict[str, List[int]], max_live: int = 4, tail: int = 8,
              sizes=(13, 7, 2, 16, 5, 9)):
    """Up to ``max_live`` requests at a time: each is fed in portions (sizes rotate) and its last ``tail``
    tokens one by one, beside the others; a finished request's place is taken by the next one."""
    waiting = list(prompts)
    live: List[str] = []
    fed = {k: 0 for k in prompts}
    turn = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        portions, ending = [], []
        for j, rid in enumerate(live):
            ids = prompts[rid]
            left = len(ids) - fed[rid]
            if (turn + j) % 5 == 4 and left > 1:
                continue      # a request may be left out of a step and go on later
            n = 1 if left <= tail else min(sizes[(turn + j) % len(sizes)], left - tail)
            toks = ids[fed[rid]:fed[rid] + n]
            want = [n - 1] if n > 1 else [0]
            if n > 2 and (turn + j) % 2 == 0:
                want = [0, n - 1]
            portions.append((rid, toks, want))
            fed[rid] += n
            if fed[rid] == len(ids):
                ending.append(rid)
        if portions:
            trace.step(portions, end=ending)
        for rid in ending:
            live.remove(rid)
        turn += 1
