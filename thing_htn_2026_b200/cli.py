"""Command line.  Option names follow the reference's scripts where it has them:
``--model``, ``--seed`` and ``--shapes BxSxN`` (comma-separated batch x prompt length x
new tokens; prompts are seeded uniform-random ids) from tests/local_check.py:61-84, :191-194.

    python -m thing_htn_2026_b200 generate --model DIR --shapes 2x17x6 --seed 0
    python -m thing_htn_2026_b200 generate --model DIR --prompt-ids prompts.json --max-new-tokens 32 \\
        --temperature 0.7 --stop-token-ids 151645
    python -m thing_htn_2026_b200 generate --random-config tiny-b --seed 1 --prompt-lens 1,23 --max-new-tokens 12
    python -m thing_htn_2026_b200 random-model --random-config qwen3-4b --seed 0 --out DIR
    python -m thing_htn_2026_b200 bench --random-config qwen3-4b --shapes 8x512x64
    python -m thing_htn_2026_b200 replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl

A model is either a folder (``--model``) or a named configuration with random weights
(``--random-config``; ``--seed`` seeds both the weights and the prompts).
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


def parse_lens(spec: str) -> List[int]:
    try:
        lens = [int(item) for item in spec.split(",") if item.strip()]
    except ValueError:
        raise SystemExit(f"bad --prompt-lens {spec!r}: expected comma-separated lengths") from None
    if not lens or min(lens) < 1:
        raise SystemExit(f"bad --prompt-lens {spec!r}: every length must be >= 1")
    return lens


def make_prompt(batch: int, length: int, vocab: int, seed: int) -> List[List[int]]:
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=g, dtype=torch.int64).tolist()


def make_prompts_of(lens: List[int], vocab: int, seed: int) -> List[List[int]]:
    """One seeded uniform-random prompt per length."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g, dtype=torch.int64).tolist() for n in lens]


def _named_config(args):
    from .config import config_from_dict, named_config_json
    data = named_config_json(args.random_config)
    if getattr(args, "layers", 0):
        data["num_hidden_layers"] = args.layers
    return config_from_dict(data)


def _engine(args):
    from .engine.engine import Engine
    if bool(args.model) == bool(args.random_config):
        raise SystemExit("give exactly one of --model DIR and --random-config NAME")
    if args.model:
        return Engine(args.model, dtype=args.dtype, device=args.device)
    return Engine.from_config(_named_config(args), seed=args.seed, dtype=args.dtype, device=args.device)


def _jobs(args, vocab: int):
    """(prompts, new tokens) per generate call, from --prompt-ids, --prompt-lens or --shapes."""
    if args.prompt_ids:
        with open(args.prompt_ids) as handle:
            return [(json.load(handle), args.max_new_tokens)]
    if args.prompt_lens:
        return [(make_prompts_of(parse_lens(args.prompt_lens), vocab, args.seed), args.max_new_tokens)]
    return [(make_prompt(b, s, vocab, args.seed + i), n) for i, (b, s, n) in enumerate(parse_shapes(args.shapes))]


def _cmd_generate(args) -> int:
    engine = _engine(args)
    stops = [int(t) for t in args.stop_token_ids.split(",")] if args.stop_token_ids else None
    for prompts, n in _jobs(args, engine.model.vocab_size):
        started = time.perf_counter()
        done = engine.generate_all(prompts, n, temperature=args.temperature, seed=args.seed, stop_token_ids=stops)
        seconds = time.perf_counter() - started
        for i, c in enumerate(done):
            print(json.dumps({"sequence": i, "tokens": c.tokens, "finish_reason": c.finish_reason}))
        total = sum(len(c.tokens) for c in done)
        print(f"[generate] {len(prompts)} sequences, {total} tokens in {seconds:.3f} s", file=sys.stderr)
    return 0


def _cmd_bench(args) -> int:
    """Tokens per second of whole ``generate`` calls (the reference's definition: batch x new
    tokens / time of the call, prefill included; QWEN_ENGINE_CONTRACT.md:93-94), and of the
    decode steps alone, per shape.  One JSON line per shape."""
    engine = _engine(args)
    vocab = engine.model.vocab_size
    for i, (b, s, n) in enumerate(parse_shapes(args.shapes)):
        best = None
        for attempt in range(args.repeats + 1):                 # the first call captures the decode graphs
            prompts = make_prompt(b, s, vocab, args.seed + i + 1000 * attempt)
            started = time.perf_counter()
            first = None
            produced = 0
            for _ in engine.generate(prompts, n, temperature=args.temperature, seed=args.seed):
                first = first or time.perf_counter()
                produced += 1
            ended = time.perf_counter()
            if attempt and (best is None or ended - started < best[0]):
                best = (ended - started, first - started, produced)
        whole, ttft, produced = best
        print(json.dumps({"shape": f"{b}x{s}x{n}", "tok_per_s": b * produced / whole, "ttft_ms": 1e3 * ttft,
                          "decode_tok_per_s": b * (produced - 1) / (whole - ttft) if produced > 1 else None,
                          "dtype": args.dtype}))
    return 0


def _cmd_random_model(args) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    if bool(args.config) == bool(args.random_config):
        raise SystemExit("give exactly one of --config FILE and --random-config NAME")
    if args.config:
        with open(args.config) as handle:
            config = config_from_dict(json.load(handle))
    else:
        config = _named_config(args)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    write_random_model(args.out, config, args.seed, dtype=dtype, matrix_std=args.matrix_std, gain_std=args.gain_std,
                       device=args.device)
    print(args.out)
    return 0


def _cmd_replay(args, rest) -> int:
    from .engine.replay import main as replay_main
    return replay_main(rest)


def _model_options(p) -> None:
    from .config import named_configs
    p.add_argument("--model", help="model folder (config.json + model.safetensors)")
    p.add_argument("--random-config", metavar="NAME",
                   help="random weights of a named configuration: " + ", ".join(named_configs()))
    p.add_argument("--layers", type=int, default=0, help="with --random-config: fewer layers (0 = all)")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--dtype", default="bfloat16", type=_dtype_name, choices=["bfloat16", "float32"],
                   help="bfloat16 (bf16) or float32 (fp32)")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")


def _dtype_name(text: str) -> str:
    """``bf16`` and ``fp32`` are accepted for ``bfloat16`` and ``float32``."""
    return {"bf16": "bfloat16", "fp32": "float32"}.get(text.lower(), text.lower())


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        return _cmd_replay(None, argv[1:])
    parser = argparse.ArgumentParser(prog="thing_htn_2026_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="continue prompts and print the tokens")
    _model_options(g)
    g.add_argument("--shapes", default="1x5x4,2x17x6,3x64x4,1x130x9", help="comma-separated BxSxN")
    g.add_argument("--prompt-lens", default="", help="comma-separated prompt lengths of ONE batch of unequal "
                                                     "prompts (overrides --shapes; new tokens from --max-new-tokens)")
    g.add_argument("--prompt-ids", help="JSON file: list of token-id lists (overrides --shapes and --prompt-lens)")
    g.add_argument("--max-new-tokens", type=int, default=32)
    g.add_argument("--stop-token-ids", default="", help="comma-separated ids; none by default")
    g.set_defaults(run=_cmd_generate)

    b = sub.add_parser("bench", help="tokens per second of generate calls, one JSON line per shape")
    _model_options(b)
    b.add_argument("--shapes", default="1x512x32,4x2048x32,16x512x128",
                   help="comma-separated BxSxN (default: the reference's public workloads, AGENTS.md:56-60)")
    b.add_argument("--repeats", type=int, default=2, help="timed calls per shape (the best counts)")
    b.set_defaults(run=_cmd_bench)

    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", help="a config.json")
    r.add_argument("--random-config", metavar="NAME", help="a named configuration instead of --config")
    r.add_argument("--layers", type=int, default=0, help="with --random-config: fewer layers (0 = all)")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--device", default="cpu", help="where the values are drawn (cuda:0 draws a large model in seconds)")
    r.add_argument("--dtype", default="bfloat16", type=_dtype_name, choices=["bfloat16", "float32"])
    r.add_argument("--matrix-std", type=float, default=0.02)
    r.add_argument("--gain-std", type=float, default=0.02)
    r.set_defaults(run=_cmd_random_model)

    sub.add_parser("replay", help="trace replay (same options as bin/trace_run)")
    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
