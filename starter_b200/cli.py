"""Command line: generate from token ids, write random weights, replay a trace.

The reference has no command line for generation: its engine is driven by a
harness that hands it token ids and never text (QWEN_ENGINE_CONTRACT.md:83-85,
tests/test_harness.py:16-33).  This one keeps that convention (prompts are
token ids) and names its options after the reference's arguments
(``model_path``, ``input_ids``, ``max_new_tokens``).

    python -m starter_b200 generate --model DIR --input-ids "1,2,3;4,5" --max-new-tokens 8
    python -m starter_b200 random-weights --config config.json --seed 0 --out DIR
    python -m starter_b200 replay --model DIR --dtype float32 --out DIR --max-tokens 4096 < steps.jsonl
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _parse_ids(text: str):
    return [[int(t) for t in seq.replace(" ", "").split(",") if t] for seq in text.split(";") if seq.strip()]


def _generate(args) -> int:
    from .engine.engine import Engine
    if args.input_file:
        prompts = json.loads(Path(args.input_file).read_text())
    elif args.input_ids:
        prompts = _parse_ids(args.input_ids)
    else:
        print("give --input-ids or --input-file", file=sys.stderr)
        return 2
    engine = Engine(args.model, dtype=args.dtype, max_batch=args.max_batch, max_context=args.max_context,
                    use_graphs=False if args.no_graphs else None, verbose=True)
    if args.stream and len(prompts) <= args.max_batch:
        for step in engine.generate(prompts, args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
                                    seed=args.seed, stop_token_ids=args.stop_token):
            print(json.dumps(step), flush=True)
    else:
        for out in engine.generate_all(prompts, args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
                                       seed=args.seed, stop_token_ids=args.stop_token):
            print(json.dumps(out), flush=True)
    return 0


def _random_weights(args) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_model_folder
    config = config_from_dict(json.loads(Path(args.config).read_text()))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    write_model_folder(config, args.seed, args.out, dtype=dtype, shards=args.shards)
    files = "model.safetensors" if args.shards <= 1 else f"{args.shards} model-*-of-*.safetensors shards"
    print(f"wrote {args.out}/config.json and {args.out}/{files}")
    return 0


def _replay(args) -> int:
    from .engine.replay import run
    return run(args)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="starter_b200", description=__doc__.split("\n\n")[0])
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="continue prompts given as token ids")
    g.add_argument("--model", required=True, help="model_path: folder with config.json and model.safetensors (or its shards)")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--input-ids", help='prompts as token ids, sequences separated by ";": "1,2,3;4,5"')
    g.add_argument("--input-file", help="JSON file with a list of token-id lists")
    g.add_argument("--max-new-tokens", type=int, required=True)
    g.add_argument("--temperature", type=float, default=0.0, help="0 selects greedily (the reference's behaviour)")
    g.add_argument("--top-k", type=int, default=0, help="0 keeps the whole vocabulary")
    g.add_argument("--seed", type=int, default=0, help="seed of the sampler")
    g.add_argument("--stop-token", type=int, action="append", default=[], help="token id that ends a sequence; repeatable")
    g.add_argument("--max-batch", type=int, default=64)
    g.add_argument("--max-context", type=int, default=4096)
    g.add_argument("--no-graphs", action="store_true", help="run every step eagerly (as ENGINE_NO_GRAPHS does)")
    g.add_argument("--stream", action="store_true", help="print one line per step instead of one per request")
    g.set_defaults(func=_generate)

    r = sub.add_parser("random-weights", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="a config.json")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--shards", type=int, default=1, help="split the tensors over this many safetensors files")
    r.set_defaults(func=_random_weights)

    t = sub.add_parser("replay", help="feed given token ids step by step and write logits (see bin/trace_run)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.set_defaults(func=_replay)
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .csrc.build import BuildError
    from .engine.generate import GenerationError
    from .engine.step import StepError
    from .weights import SafetensorsError, WeightsError
    try:
        return args.func(args)
    except (BuildError, GenerationError, StepError, WeightsError, SafetensorsError, FileNotFoundError) as exc:
        # what a user can act on comes as one message, not as a traceback
        print(f"starter_b200: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
