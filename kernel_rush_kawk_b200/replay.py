"""Trace replay: feed given token ids through a model step by step, write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Each entry brings a request's next tokens and the places among them whose logits
are wanted; ``end`` lists requests that are finished after the step (their slot
and pages are given back). For a step that wants something, ``<out>/<step>.f32``
receives the logits as little-endian float32 ``[wanted, vocab]``, in the order
of the entries and of their ``want`` lists. After every step ``done <step>`` is
printed and flushed. Nothing is sampled. The program drives the library's own
engine: the model, step function, cache and kernels that generation uses.

The reference's nearest things are its teacher-forced self-check and the replay its
contract describes (engine/engine.py:522-560, QWEN_ENGINE_CONTRACT.md:105-123 of
willzeng274/kernel-rush-kawk); it has no such program.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np

from .cache.store import PAGE


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder that receives <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time, each request rounded up to a multiple of 64")
    p.add_argument("--no-graphs", action="store_true", help="run decode steps without CUDA graphs")
    return p


def run(args, stdin=None, stdout=None) -> int:
    from .engine import Engine, StepEntry

    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    pages = max(1, -(-args.max_tokens // PAGE))
    engine = Engine(args.model, dtype=args.dtype, max_tokens=pages * PAGE, max_slots=min(pages, 4096),
                    max_context=pages * PAGE, use_cuda_graphs=not args.no_graphs)
    slots: dict[str, int] = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for e in step.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.cache.alloc()
            entries.append(StepEntry(slots[rid], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        logits = engine.step(entries)
        if logits.shape[0] > 0:
            data = logits.detach().float().cpu().numpy().astype("<f4", copy=False)
            tmp = out_dir / f".{step['step']}.f32.tmp"
            data.tofile(tmp)
            tmp.replace(out_dir / f"{step['step']}.f32")
        engine.ops.check()
        for rid in step.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.cache.free(slots.pop(rid))
        print(f"done {step['step']}", file=stdout, flush=True)
    return 0


def main(argv=None) -> int:
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
