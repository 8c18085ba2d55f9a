"""Single-prompt generation from the command line; the reference's options and meanings
(nanoinfer/generate.py:88-129, cpp/tools/generate.py:30-66).

    python -m nanoinfer_b200.cli.generate --model-dir DIR --prompt "The capital of France is" --max-tokens 20
    python -m nanoinfer_b200.cli.generate --random-weights tiny --prompt "5 17 3" --temperature 0.8 --top-p 0.95 --seed 1234
"""
from __future__ import annotations

import argparse
import sys
import tempfile

from .tokenizer import load_tokenizer


def add_model_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model-dir", "--weights-dir", "--model", dest="model_dir", default=None,
                   help="folder with config.json and model.safetensors (the reference's --model takes a hub id; "
                        "there is no network here, so this takes a local folder)")
    p.add_argument("--device", default="cuda", help="the reference's option; this engine runs on a CUDA device only")
    p.add_argument("--random-weights", metavar="CONFIG_JSON", default=None,
                   help="write a random-weights model folder from this config.json file and use it")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--block-size", "--page-size", dest="page_size", type=int, default=16,
                   help="tokens per cache page")
    p.add_argument("--num-blocks", "--num-pages", dest="num_pages", type=int, default=1024,
                   help="pages in the cache pool")
    p.add_argument("--max-tokens-per-step", type=int, default=2048, help="token budget of one step")


def add_sampling_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--max-tokens", type=int, default=32)
    p.add_argument("--temperature", type=float, default=0.0, help="0 (default) is greedy/deterministic")
    p.add_argument("--top-k", type=int, default=0, help="keep the k highest-logit tokens (0=off)")
    p.add_argument("--top-p", type=float, default=1.0, help="nucleus: keep cumprob >= p (1=off)")
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=0, help="seed of the sampler (and of --random-weights)")


def resolve_model_dir(args) -> str:
    import os
    if not str(getattr(args, "device", "cuda")).startswith("cuda"):
        raise SystemExit(f"--device {args.device}: this engine has no CPU path; give a CUDA device")
    if args.model_dir:
        if not os.path.isdir(args.model_dir):
            raise SystemExit(f"{args.model_dir} is not a folder; models are read from a local folder with "
                             f"config.json and model.safetensors (nothing is downloaded)")
        return args.model_dir
    if args.random_weights:
        import json
        from ..registry import config_from_json_dict
        from ..weights import write_random_model
        with open(args.random_weights) as f:
            cfg = config_from_json_dict(json.load(f))
        d = tempfile.mkdtemp(prefix="nanoinfer_b200_model_")
        write_random_model(cfg, d, seed=args.seed)
        print(f"wrote a random-weights model to {d}", file=sys.stderr)
        return d
    raise SystemExit("give --model-dir DIR or --random-weights CONFIG_JSON")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="nanoinfer_b200 text generation")
    p.add_argument("--prompt", required=True, help="text (with tokenizer.json in the model folder) or token ids")
    add_model_args(p)
    add_sampling_args(p)
    p.add_argument("--no-cache", dest="use_cache", action="store_false",
                   help="recompute the whole sequence for every token (slow; checks the cache: same output)")
    args = p.parse_args(argv)

    from ..api import generate, load_model
    from ..sampling.params import SamplingParams
    model_dir = resolve_model_dir(args)
    model = load_model(model_dir, dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages,
                       max_batch=1, max_tokens_per_step=args.max_tokens_per_step)
    tok = load_tokenizer(model_dir, model.eos_token_id)
    try:
        tok.encode(args.prompt)
    except ValueError as e:
        raise SystemExit(str(e)) from None
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            repetition_penalty=args.repetition_penalty, seed=args.seed)
    print(f"Prompt: {args.prompt}")
    print(f"Completion: {generate(model, tok, args.prompt, max_tokens=args.max_tokens, use_cache=args.use_cache, sampling=params)}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
