"""Offline command line.  The reference's only command line is its server
(ullm/entrypoints/api_server.py:127-184); its flags keep their names, defaults
and meanings here, and offline use, which the reference leaves to scripts
(bench.py), gets sub-commands:

    python -m ullm_b200 generate --model DIR --prompt-ids 1,2,3 --max-new-tokens 16
    python -m ullm_b200 random-model --out DIR --config config.json --seed 0
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _generate(args) -> int:
    from ..config import EngineConfig
    from ..sampling import SamplingParams
    from .llm import LLM

    cfg = EngineConfig.from_args(args)
    llm = LLM(cfg)
    prompts: list = []
    for s in args.prompt_ids or []:
        prompts.append([int(t) for t in s.replace(" ", "").split(",") if t])
    for s in args.prompt or []:
        prompts.append(s)
    if not prompts:
        print("give --prompt-ids 1,2,3 or --prompt TEXT", file=sys.stderr)
        return 2
    sp = SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
        max_new_tokens=args.max_new_tokens, max_tokens=args.max_tokens, ignore_eos=args.ignore_eos,
        seed=args.sampling_seed,
    )
    t0 = time.time()
    outs = llm.generate_batch(prompts, sp)
    dt = time.time() - t0
    llm.engine.shutdown()  # (ends a --profile run: its tables are printed and written here)
    for o in outs:
        print(json.dumps({"prompt_tokens": o.num_prompt_tokens, "token_ids": o.token_ids, "text": o.text,
                          "finish_reason": o.finish_reason.name if o.finish_reason else None}))
    n = sum(o.num_generated_tokens for o in outs)
    print(f"{n} tokens in {dt:.2f} s ({n / max(dt, 1e-9):.1f} tok/s); {json.dumps(llm.engine.stats())}",
          file=sys.stderr)
    return 0


def _random_model(args) -> int:
    from ..weights import write_random_model

    with open(args.config) as f:
        config = json.load(f)
    write_random_model(args.out, config, seed=args.seed, std=args.std, norm_std=args.norm_std, dtype=args.dtype)
    print(args.out)
    return 0


def main(argv=None) -> int:
    from ..config import EngineConfig

    ap = argparse.ArgumentParser(prog="ullm_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate from token ids or text")
    EngineConfig.add_cli_args(g)
    g.add_argument("--prompt-ids", action="append", help="comma-separated token ids (repeatable)")
    g.add_argument("--prompt", action="append", help="text (needs a tokenizer in the model folder; repeatable)")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--max-tokens", type=int, default=None, help="bound on prompt + generated tokens")
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--sampling-seed", type=int, default=None)
    g.set_defaults(fn=_generate)
    r = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    r.add_argument("--out", required=True)
    r.add_argument("--config", required=True, help="a config.json with the architecture's keys")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-std", type=float, default=0.0)
    r.add_argument("--dtype", default=None, help="bfloat16, float16 or float32 (default: the config's)")
    r.set_defaults(fn=_random_model)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
