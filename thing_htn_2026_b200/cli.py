"""Command line.  Option names follow the reference's scripts where it has them:
``--model``, ``--seed`` and ``--shapes BxSxN`` (comma-separated batch x prompt length x
new tokens; prompts are seeded uniform-random ids) from tests/local_check.py:61-84, :191-194.

    python -m thing_htn_2026_b200 generate --model DIR --shapes 2x17x6 --seed 0
    python -m thing_htn_2026_b200 generate --model DIR --prompt-ids prompts.json --max-new-tokens 32 \\
        --temperature 0.7 --stop-token-ids 151645
    python -m thing_htn_2026_b200 random-model --config config.json --seed 0 --out DIR
    python -m thing_htn_2026_b200 replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Tuple


def parse_shapes(spec: str) -> List[Tuple[int, int, int]]:
    shapes = []
    for item in spec.split(","):
        item = item.strip()
        if not item:
            continue
        parts = item.lower().split("x")
        if len(parts) != 3:
            raise SystemExit(f"bad shape {item!r}: expected BxSxN")
        b, s, n = (int(v) for v in parts)
        if min(b, s, n) < 1:
            raise SystemExit(f"bad shape {item!r}: all of B, S, N must be >= 1")
        shapes.append((b, s, n))
    if not shapes:
        raise SystemExit("no shapes given")
    return shapes


def make_prompt(batch: int, length: int, vocab: int, seed: int) -> List[List[int]]:
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=g, dtype=torch.int64).tolist()


def _cmd_generate(args) -> int:
    from .engine.engine import Engine
    engine = Engine(args.model, dtype=args.dtype, device=args.device)
    vocab = engine.model.vocab_size
    stops = [int(t) for t in args.stop_token_ids.split(",")] if args.stop_token_ids else None
    jobs = []
    if args.prompt_ids:
        with open(args.prompt_ids) as handle:
            prompts = json.load(handle)
        jobs.append((prompts, args.max_new_tokens))
    else:
        for i, (b, s, n) in enumerate(parse_shapes(args.shapes)):
            jobs.append((make_prompt(b, s, vocab, args.seed + i), n))
    for prompts, n in jobs:
        started = time.perf_counter()
        done = engine.generate_all(prompts, n, temperature=args.temperature, seed=args.seed, stop_token_ids=stops)
        seconds = time.perf_counter() - started
        for i, c in enumerate(done):
            print(json.dumps({"sequence": i, "tokens": c.tokens, "finish_reason": c.finish_reason}))
        total = sum(len(c.tokens) for c in done)
        print(f"[generate] {len(prompts)} sequences, {total} tokens in {seconds:.3f} s", file=sys.stderr)
    return 0


def _cmd_random_model(args) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    with open(args.config) as handle:
        config = config_from_dict(json.load(handle))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    write_random_model(args.out, config, args.seed, dtype=dtype, matrix_std=args.matrix_std, gain_std=args.gain_std)
    print(args.out)
    return 0


def _cmd_replay(args, rest) -> int:
    from .engine.replay import main as replay_main
    return replay_main(rest)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        return _cmd_replay(None, argv[1:])
    parser = argparse.ArgumentParser(prog="thing_htn_2026_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="continue prompts and print the tokens")
    g.add_argument("--model", required=True, help="model folder (config.json + model.safetensors)")
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--shapes", default="1x5x4,2x17x6,3x64x4,1x130x9", help="comma-separated BxSxN")
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--prompt-ids", help="JSON file: list of token-id lists (overrides --shapes)")
    g.add_argument("--max-new-tokens", type=int, default=32)
    g.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    g.add_argument("--stop-token-ids", default="", help="comma-separated ids; none by default")
    g.set_defaults(run=_cmd_generate)

    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--matrix-std", type=float, default=0.02)
    r.add_argument("--gain-std", type=float, default=0.02)
    r.set_defaults(run=_cmd_random_model)

    sub.add_parser("replay", help="trace replay (same options as bin/trace_run)")
    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
