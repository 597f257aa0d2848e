"""The command line, after the reference's ``xrt generate`` (crates/xrt-cli/src/main.rs:22-49, 82-127):
the same option names, defaults and meanings where the reference has them; ``--prompt-ids`` takes
token ids where the reference's ``--prompt`` takes text (there is no tokenizer here), and the
generated ids go to standard output, the statistics line to standard error.

    python -m xeno_rt_b200 generate (--model DIR | --random-config CONFIG.json [--seed-weights N])
        --prompt-ids 1,2,3 [--prompt-ids 4,5 ...] [--max-tokens 128] [--temperature 0.8] [--top-k 40] [--top-p 0.95]
        [--repetition-penalty 1.1] [--seed N] [--dtype bfloat16|float32] [--stop-ids 2,3] [--device cuda:0]

The reference's command takes its model from one of two sources, a file or a repository to fetch it
from (main.rs:28-34); the two sources here are a folder (``--model``: config.json and safetensors,
one file or shards) and a configuration alone (``--random-config``: weights drawn on the device from
``--seed-weights`` by the generator of weights/random_init.py, the same values that
``write_random_model`` writes for that seed).
"""
from __future__ import annotations

import argparse
import sys


def _ids(text: str) -> list:
    try:
        return [int(t) for t in text.replace(" ", "").split(",") if t != ""]
    except ValueError:
        raise argparse.ArgumentTypeError(f"{text!r} is not a comma-separated list of token ids") from None


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="xrt", description="xeno-rt_b200 command line")
    sub = parser.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate tokens for one or more prompts")
    source = g.add_mutually_exclusive_group(required=True)
    source.add_argument("--model", help="folder with config.json and model.safetensors (one file, or shards with "
                                        "model.safetensors.index.json)")
    source.add_argument("--random-config", metavar="JSON",
                        help="a config.json file; the weights are random, drawn from --seed-weights")
    g.add_argument("--seed-weights", type=int, default=0, help="seed of the random weights (with --random-config)")
    g.add_argument("--prompt-ids", required=True, action="append", type=_ids,
                   help="token ids of a prompt, comma-separated; repeat the option for a batch")
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.8)
    g.add_argument("--top-k", type=int, default=40)
    g.add_argument("--top-p", type=float, default=0.95)
    g.add_argument("--repetition-penalty", type=float, default=1.1)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--stop-ids", type=_ids, default=None,
                   help="ids that end a sequence (default: eos_token_id of config.json)")
    g.add_argument("--device", default="cuda:0")
    return parser


def run_generate(args) -> int:
    import json

    from .core import ConfigError
    from .engine import GenerateRequest, Model, Runtime

    if args.model is not None:
        runtime = Runtime.load(args.model, dtype=args.dtype, device=args.device)
    else:
        try:
            with open(args.random_config) as fh:
                raw = json.load(fh)
        except FileNotFoundError:
            raise ConfigError(f"{args.random_config}: no such file") from None
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{args.random_config}: not valid JSON ({exc})") from None
        runtime = Runtime(Model.random(raw, seed=args.seed_weights, dtype=args.dtype, device=args.device))
    session = runtime.new_session()
    requests = [GenerateRequest(prompt_ids=p, max_tokens=args.max_tokens, temperature=args.temperature,
                                top_k=args.top_k, top_p=args.top_p, repetition_penalty=args.repetition_penalty,
                                seed=(None if args.seed is None else args.seed + i),
                                stop_ids=(None if args.stop_ids is None else tuple(args.stop_ids)))
                for i, p in enumerate(args.prompt_ids)]
    results, stats = session.generate_batch(requests)
    for r in results:
        print(",".join(str(t) for t in r.tokens), flush=True)
    print("\n" + stats.line(), file=sys.stderr)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .core import XrtError
    try:
        if args.command == "generate":
            return run_generate(args)
    except XrtError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    return 2
