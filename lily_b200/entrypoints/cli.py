"""Command line.  Every ``ServerArgs`` field is a ``--flag`` as in lily/server_args.py:145-174 and
lily/entrypoints/launch.py:100-112; where the reference's ``lily-serve`` starts an HTTP server,
this engine (token in, token out, one process) offers sub-commands:

    python -m lily_b200 generate --model-path DIR --prompt-ids 1,2,3 [--prompt-ids ...] \
        [--max-new-tokens N --temperature T --top-k K --top-p P --min-p M --seed S --ignore-eos]
    python -m lily_b200 init-random --config config.json --out DIR --seed S [--store-dtype bfloat16]
    python -m lily_b200 architectures
"""

from __future__ import annotations

import argparse
import json
import logging
import sys
from typing import List, Optional

from lily_b200.config.server_args import ServerArgs


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv: Optional[List[str]] = None) -> int:
    parser = argparse.ArgumentParser("lily_b200")
    sub = parser.add_subparsers(dest="command", required=True)

    gen = sub.add_parser("generate", help="generate from token ids")
    ServerArgs.add_cli_args(gen)
    gen.add_argument("--prompt-ids", action="append", required=True, help="token ids, comma or space separated")
    gen.add_argument("--max-new-tokens", type=int, default=128)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--top-k", type=int, default=-1)
    gen.add_argument("--top-p", type=float, default=1.0)
    gen.add_argument("--min-p", type=float, default=0.0)
    gen.add_argument("--repetition-penalty", type=float, default=1.0)
    gen.add_argument("--frequency-penalty", type=float, default=0.0)
    gen.add_argument("--presence-penalty", type=float, default=0.0)
    gen.add_argument("--stop-token-ids", type=_ids, default=[], help="token ids, comma or space separated")
    gen.add_argument("--logprobs", action="store_true", help="the chosen tokens' log-probabilities")
    gen.add_argument("--top-logprobs", type=int, default=None, help="the k most probable tokens at every step")
    gen.add_argument("--seed", type=int, default=None)
    gen.add_argument("--ignore-eos", action="store_true")

    rnd = sub.add_parser("init-random", help="write a model folder with seeded random weights")
    rnd.add_argument("--config", required=True, help="a config.json of a supported architecture")
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--store-dtype", default=None, choices=["bfloat16", "float32"])
    rnd.add_argument("--std", type=float, default=0.02)
    rnd.add_argument("--gain-jitter", type=float, default=0.0)

    sub.add_parser("architectures", help="list the supported architectures")
    args = parser.parse_args(argv)

    if args.command == "architectures":
        from lily_b200.config.registry import supported_architectures
        print("\n".join(supported_architectures()))
        return 0
    if args.command == "init-random":
        from lily_b200.weights.random_init import write_random_model
        with open(args.config) as f:
            cfg = json.load(f)
        print(write_random_model(args.out, cfg, args.seed, args.store_dtype, args.std, args.gain_jitter))
        return 0

    server_args = ServerArgs.from_cli_args(args)
    if not server_args.model_path:
        parser.error("--model-path is required")
    logging.basicConfig(level=getattr(logging, server_args.log_level.upper(), logging.INFO),
                        format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    from lily_b200.engine.engine import Engine, EngineConfig
    from lily_b200.engine.runner import ModelRunner
    from lily_b200.sampling.params import SamplingParams

    engine = Engine(EngineConfig(server_args.model_path, dtype=server_args.dtype, device=server_args.device),
                    runner=ModelRunner.from_model_dir(server_args))
    engine.server_args = server_args
    params = SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
                            top_p=args.top_p, min_p=args.min_p, repetition_penalty=args.repetition_penalty,
                            frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty,
                            stop_token_ids=args.stop_token_ids, logprobs=args.logprobs, top_logprobs=args.top_logprobs,
                            seed=args.seed, ignore_eos=args.ignore_eos)
    for out in engine.generate([_ids(p) for p in args.prompt_ids], params):
        print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
