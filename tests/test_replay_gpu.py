"""Trace replay through bin/trace_run, as a user runs it, against the plain implementation: the same
requests whole; most of each in one step and the last 32 tokens one by one; in portions of changing
size down to two tokens; and mixed, up to four live requests, portions of some beside decoded tokens
of others, with so few pages that they are used again. In 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

from gpu_util import assert_close, bf16_slack
from plain_qwen2 import PlainModel
from replay_util import Trace, add_decode_tail, add_mixed, add_portions, add_whole, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 7, 33, 90, 200, 61], "B": [2, 9, 17, 64, 100, 150], "W": [3, 40, 77, 130, 58, 101],
           "C": [5, 70, 300, 129, 260, 33]}      # C: heads of 64, prompts beyond 256 tokens (the kernels of the large models)


def prompts_for(name, vocab):
    g = torch.Generator().manual_seed({"A": 11, "B": 22, "W": 33, "C": 44}[name])
    return {f"{name}{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W", "C"])
def test_replay_all_cuts(model_dirs, tmp_path, name, dtype):
    d, page = model_dirs[name]
    plain = PlainModel(d)
    prompts = prompts_for(name, plain.cfg["vocab"])
    want = {rid: plain.logits(ids) for rid, ids in prompts.items()}

    trace = Trace()
    tag = {}
    for mode, add in (("whole", add_whole), ("tail", add_decode_tail), ("portions", add_portions)):
        for rid, ids in prompts.items():
            tag[f"{mode}:{rid}"] = rid
            add(trace, f"{mode}:{rid}", ids)
    solo_max = trace.max_tokens
    mixed = {f"mixed:{rid}": ids for rid, ids in prompts.items()}
    for k in mixed:
        tag[k] = k.split(":", 1)[1]
    add_mixed(trace, mixed, max_live=4)
    total_mixed = sum(-(-len(v) // 64) * 64 for v in mixed.values())
    assert trace.max_tokens < total_mixed, "the pool must be smaller than all mixed requests together"

    got = run_trace(d, dtype, trace, str(tmp_path / "out"), page_size=page)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    seen = set()
    by_mode = {}
    decided = 0
    for (rid, pos), rows in got.items():
        ref = want[tag[rid]][pos]
        best2 = torch.topk(ref, 2).values
        clear = (best2[0] - best2[1]).item() > (bf16_slack(ref) if dtype == "bfloat16" else 1e-4)
        decided += clear
        for row in rows:
            assert_close(torch.from_numpy(row.copy()), ref, tdt, f"{rid}@{pos}")
            if clear:       # where the margin allows it, the greedy token is the plain implementation's
                assert int(row.argmax()) == int(ref.argmax()), f"{rid}@{pos}: another best token"
        seen.add((rid.split(":")[0], tag[rid], pos))
        by_mode.setdefault((tag[rid], pos), {})[rid.split(":")[0]] = rows[0]
    assert decided > len(got) // (8 if dtype == "bfloat16" else 2), "too few positions with a clear best token to mean anything"
    # every position of every request was checked whole and in portions
    for rid, ids in prompts.items():
        for pos in range(len(ids)):
            assert ("whole", rid, pos) in seen and ("portions", rid, pos) in seen
    if dtype == "float32":
        # 32-bit: every reduction's order depends on the position's own data only (ascending k per output in the
        # products, keys in absolute blocks of 32 in the attention, one warp per row in the norms), so the cut,
        # the batch and the pages change NO bit of a logit (the reference holds max|diff| = 0 for changes of
        # placement: its cpp/docs notes on batching, lines 52-54, and cpp/tests/run_batch.cpp:79-96)
        for (rid, pos), modes in by_mode.items():
            base = modes["whole"]
            for mode, row in modes.items():
                assert np.array_equal(row, base), \
                    f"{rid}@{pos}: {mode} differs from whole by {np.abs(row - base).max()}"
