"""Command line of the library.

    python -m kernel_rush_kawk_b200.cli generate --model DIR --prompt-ids 1,2,3 --max-new-tokens 16
    python -m kernel_rush_kawk_b200.cli generate --random tiny_a --weights-seed 0 --prompt-ids 5,6 --prompt-ids 7
    python -m kernel_rush_kawk_b200.cli write-random --preset tiny_b --seed 1 --out DIR
    python -m kernel_rush_kawk_b200.cli replay --model DIR --dtype float32 --out DIR --max-tokens 4096 < trace.jsonl

The reference has no command line for generation (its entry is the ``Engine`` class,
engine/engine.py:472 of willzeng274/kernel-rush-kawk, driven by a platform binary);
the option names here are those of ``Engine.generate`` (``input_ids`` as prompt ids,
``max_new_tokens``). Its one run-time switch that applies here keeps its name and
meaning: the environment variable ``ENGINE_NO_GRAPHS`` (engine.py:487) turns CUDA
graphs off.
"""

from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="kernel_rush_kawk_b200")
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens for one batch of prompts")
    src = g.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and *.safetensors")
    src.add_argument("--random", metavar="PRESET", help="random weights for a named configuration")
    g.add_argument("--weights-seed", type=int, default=0)
    g.add_argument("--prompt-ids", action="append", type=_ids, default=[], metavar="IDS",
                   help="token ids of one prompt, comma separated; repeat for a batch")
    g.add_argument("--prompt-file", help="JSON file with a list of token id lists")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0, help="0 selects greedily")
    g.add_argument("--seed", type=int, default=0, help="seed of temperature sampling")
    g.add_argument("--stop-token-id", action="append", type=int, default=None,
                   help="repeatable; default: none, as in the reference (give config.json's eos id to stop there)")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--max-slots", type=int, default=64)
    g.add_argument("--max-context", type=int, default=None)
    g.add_argument("--max-batch", type=int, default=None, help="run the prompts as consecutive batches of this size")

    w = sub.add_parser("write-random", help="write a model folder with random weights")
    w.add_argument("--preset", required=True)
    w.add_argument("--seed", type=int, default=0)
    w.add_argument("--std", type=float, default=0.02)
    w.add_argument("--out", required=True)

    from .replay import build_parser as replay_parser
    sub.add_parser("replay", parents=[replay_parser()], add_help=False, help="trace replay (see bin/trace_run)")
    b = sub.add_parser("bench", help="the measurement script at the root of a source checkout (bench.py); "
                                     "arguments after `bench` are passed to it")
    return p


def main(argv=None) -> int:
    parser = build_parser()
    args, rest = parser.parse_known_args(argv)
    if rest and args.command != "bench":
        parser.error("unrecognized arguments: " + " ".join(rest))
    if args.command == "replay":
        from .replay import run
        return run(args)
    if args.command == "bench":
        import runpy
        from pathlib import Path
        script = Path(__file__).resolve().parent.parent / "bench.py"
        if not script.is_file():
            print(f"no bench.py beside the package ({script}): the measurement script ships with the source checkout",
                  file=sys.stderr)
            return 2
        sys.argv = [str(script)] + list(rest)
        runpy.run_path(str(script), run_name="__main__")
        return 0
    if args.command == "write-random":
        from . import write_model_folder
        from .config.registry import preset_config
        folder = write_model_folder(args.out, preset_config(args.preset), args.seed, args.std)
        print(folder)
        return 0
    from . import Engine
    prompts = list(args.prompt_ids)
    if args.prompt_file:
        prompts += [list(map(int, row)) for row in json.load(open(args.prompt_file))]
    if not prompts:
        print("no prompts given (--prompt-ids or --prompt-file)", file=sys.stderr)
        return 2
    options = dict(dtype=args.dtype, max_slots=args.max_slots, max_context=args.max_context)
    if args.model:
        engine = Engine(args.model, **options)
    else:
        engine = Engine.from_random(args.random, seed=args.weights_seed, **options)
    outs = engine.generate_all(prompts, args.max_new_tokens, temperature=args.temperature, seed=args.seed,
                               stop_token_ids=args.stop_token_id or (), max_batch=args.max_batch)
    for prompt, out in zip(prompts, outs):
        print(json.dumps({"prompt": prompt, "tokens": out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
