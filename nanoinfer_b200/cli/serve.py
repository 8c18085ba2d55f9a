"""Several prompts at once through the continuous-batching scheduler; the reference's options
(cpp/tools/serve.py:31-89).

    python -m nanoinfer_b200.cli.serve --model-dir DIR --max-batch 2 --prompt "..." --prompt "..." --prompt "..."
"""
from __future__ import annotations

import argparse
import sys
import time

from .generate import add_model_args, add_sampling_args, resolve_model_dir
from .tokenizer import load_tokenizer


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="nanoinfer_b200 multi-prompt serving")
    p.add_argument("--prompt", action="append", required=True, dest="prompts",
                   help="repeat to enqueue several prompts")
    p.add_argument("--max-batch", type=int, default=4, help="concurrent sequences")
    add_model_args(p)
    add_sampling_args(p)
    args = p.parse_args(argv)

    from ..api import load_model
    from ..engine.scheduler import Request, Scheduler
    model_dir = resolve_model_dir(args)
    model = load_model(model_dir, dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages,
                       max_batch=args.max_batch, max_tokens_per_step=args.max_tokens_per_step)
    tok = load_tokenizer(model_dir, model.eos_token_id)
    sched = Scheduler(model, max_batch=args.max_batch, lookahead=True)
    prompts = {}
    for i, text in enumerate(args.prompts):
        rid = f"req{i}"
        prompts[rid] = text
        try:
            ids = tok.encode(text)
        except ValueError as e:
            raise SystemExit(str(e)) from None
        sched.add(Request(rid, ids, max_tokens=args.max_tokens, temperature=args.temperature,
                          top_k=args.top_k, top_p=args.top_p, repetition_penalty=args.repetition_penalty,
                          seed=args.seed, eos_id=model.eos_token_id))
    t0 = time.perf_counter()
    out = sched.run()
    dt = time.perf_counter() - t0
    n_tok = sum(len(v) for v in out.values())
    print(f"served {len(prompts)} prompts, max_batch={args.max_batch}, "
          f"cache=paged(block_size={args.page_size}, {args.num_pages} blocks): {sched.steps} steps, "
          f"peak_batch={sched.peak_batch}, preemptions={sched.preemptions}, "
          f"{n_tok} tokens in {dt:.2f}s ({n_tok / dt:.1f} tok/s)")
    st = sched.stats()
    actual, as_fp32 = model.weight_bytes()
    print(f"steps: {st['tokens_per_step']:.1f} tokens a step, at most {st['peak_step_tokens']}; "
          f"{st['prompt_steps']} with a prompt's portion at {100 * st['budget_use']:.0f}% of the budget of "
          f"{sched.max_tokens_per_step}; weights {actual / 2**20:.1f} MiB ({as_fp32 / 2**20:.1f} MiB in 32-bit)\n")
    for rid, text in prompts.items():
        print(f"Prompt: {text}")
        print(f"Completion: {tok.decode(out[rid])}\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
