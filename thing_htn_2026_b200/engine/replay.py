"""Trace replay: feeds given token ids through the model step by step and writes logits.
It samples nothing and owns no forward pass, cache or loader: it drives the same model,
step function, cache and kernels that generation uses.

Input, one JSON object a line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted it writes ``OUT/<step>.f32`` (little-endian
float32 ``[wanted, vocab]``, in the order of the entries and of ``want``); after every
step it prints ``done <step>``.  Requests named under ``end`` give back what they hold.

The reference has no such program; its nearest relative is the teacher-forced replay of
its test harness (tests/local_check.py:254-271).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import torch

from ..cache.sequence_cache import SequenceCache
from .loading import load_model, parse_dtype
from .step import StepEntry, StepRunner


class Replayer:
    def __init__(self, model_dir: str, dtype, max_tokens: int, out_dir: str, device: str = "cuda:0"):
        self.model = load_model(model_dir, dtype, device)
        self.cache = SequenceCache(self.model.cache_needs(), max_tokens=max_tokens, dtype=parse_dtype(dtype),
                                   device=device)
        self.runner = StepRunner(self.model, self.cache)
        self.out_dir = out_dir
        os.makedirs(out_dir, exist_ok=True)
        self.slot_of: Dict[str, int] = {}

    def run_step(self, record: dict) -> None:
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            name = str(item["id"])
            if name not in self.slot_of:
                (self.slot_of[name],) = self.cache.open(1)
            entries.append(StepEntry(self.slot_of[name], item["tokens"], item.get("want", ())))
        if entries:
            logits = self.runner.step(entries)
            if logits.shape[0]:
                data = logits.to("cpu").contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(self.out_dir, f".{step}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(self.out_dir, f"{step}.f32"))
        ended = [str(name) for name in record.get("end", [])]
        self.cache.close([self.slot_of.pop(name) for name in ended if name in self.slot_of])


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time, each rounded up to 64")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this library has no CPU path", file=sys.stderr)
        return 1
    with torch.inference_mode():
        replayer = Replayer(args.model, args.dtype, args.max_tokens, args.out, args.device)
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            replayer.run_step(record)
            print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
