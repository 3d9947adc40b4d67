"""Command line in the manner of the reference's llama-cli (crates/llama-cli/src/main.rs:13-228).

    llama-cli inspect MODEL [--tensors]
    llama-cli generate -m MODEL -p IDS [-p IDS ...] [-c N] [--memory-mib N] [--float-weights-f32]
                       [-n N] [--temperature T] [--top-k K] [--top-p P] [--repeat-penalty R] [--seed S]
    llama-cli random --config CONFIG.json --out DIR [--seed S] [--std X]

Options keep the reference's names, defaults and meanings. Text is outside this
library (no tokenizer, no chat templates): a prompt is a list of token ids,
"1,2,3" or "@file" with whitespace-separated ids (the reference's dump_logits
takes prompts the same way, crates/llama-rs/examples/dump_logits.rs:1-33), and
what is printed is token ids. `chat` and `--chat` therefore do not exist here;
the reference's `bench` is bench.py at the repository root.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _parse_prompt(text: str) -> List[int]:
    if text.startswith("@"):
        with open(text[1:], "r", encoding="utf-8") as handle:
            text = handle.read()
    return [int(piece) for piece in text.replace(",", " ").split()]


def _model_args(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("-m", "--model", required=True, help="model folder (config.json + safetensors)")
    parser.add_argument("-c", "--context", type=int, default=0,
                        help="Context capacity (0 selects min(8192, model limit))")
    parser.add_argument("--memory-mib", type=int, default=None, help="refuse to load beyond this many MiB")
    parser.add_argument("--float-weights-f32", action="store_true",
                        help="widen every weight to float32 and run the true 32-bit path")


def _sample_args(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("-n", "--max-tokens", type=int, default=256)
    parser.add_argument("--temperature", type=float, default=0.8)
    parser.add_argument("--top-k", type=int, default=40)
    parser.add_argument("--top-p", type=float, default=0.95)
    parser.add_argument("--repeat-penalty", type=float, default=1.0)
    parser.add_argument("--seed", type=int, default=42)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="llama-cli", description="B200 inference for the Llama 3 dense decoder")
    commands = parser.add_subparsers(dest="command", required=True)
    inspect = commands.add_parser("inspect", help="Inspect a model folder without initializing the GPU")
    inspect.add_argument("model")
    inspect.add_argument("--tensors", action="store_true")
    generate = commands.add_parser("generate", help="Generate from prompts given as token ids")
    _model_args(generate)
    generate.add_argument("-p", "--prompt", action="append", required=True,
                          help='token ids "1,2,3" or @file; repeat for a batch of prompts')
    generate.add_argument("--stop-ids", default=None, help="stop token ids (default: the model's eos ids)")
    generate.add_argument("--max-batch", type=int, default=None, help="sequences decoded together")
    _sample_args(generate)
    random = commands.add_parser("random", help="Write a model folder with seeded random weights")
    random.add_argument("--config", required=True, help="a config.json")
    random.add_argument("--out", required=True)
    random.add_argument("--seed", type=int, default=0)
    random.add_argument("--std", type=float, default=0.02)
    random.add_argument("--norm-std", type=float, default=0.0, help="norm weights are N(1, this)")
    random.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    return parser


def run_inspect(model: str, tensors: bool) -> dict:
    """crates/llama-cli/src/inspect.rs:23-42: format, config, tensor count and bytes, tensor table."""
    from .config.base import read_config_json
    from .weights.safetensors_io import open_checkpoint
    entries = open_checkpoint(model)
    report = {
        "format": "safetensors",
        "config": read_config_json(model),
        "tensor_count": len(entries),
        "weight_bytes": sum(e.nbytes for e in entries.values()),
        "chat_template": False,
        "tensors": {name: {"dimensions": list(e.shape), "storage_bytes": e.nbytes,
                           "encoding": str(e.dtype).replace("torch.", "")}
                    for name, e in sorted(entries.items())} if tensors else None,
    }
    return report


def run_generate(args) -> int:
    from . import Engine, GenerationOptions, Sampling
    prompts = [_parse_prompt(p) for p in args.prompt]
    limit = args.memory_mib * 1024 * 1024 if args.memory_mib is not None else None
    engine = Engine(memory_limit=limit)
    model = engine.load(args.model, dtype="float32" if args.float_weights_f32 else "bfloat16")
    batch = args.max_batch or min(len(prompts), 64)
    session = model.session(context=args.context, max_batch=batch)
    estimate = model.memory(session.context, batch)
    print(f"{engine.device_name()}; {model.config.architecture}; context {session.context}; "
          f"reserved model/session {(estimate.weights + estimate.cache) / 1048576:.1f} MiB", file=sys.stderr)
    options = GenerationOptions(max_tokens=args.max_tokens, sampling=Sampling(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
        repeat_penalty=args.repeat_penalty, seed=args.seed))
    stops = None if args.stop_ids is None else _parse_prompt(args.stop_ids)

    def show(request: int, token: int) -> None:
        print(f"{request}\t{token}", flush=True)  # one line per token as it arrives
    results = session.generate(prompts, options, stop_token_ids=stops, on_token=show)
    for r in results:
        print(json.dumps({"event": "finished", "request": r.request, "reason": r.finish_reason,
                          "tokens": len(r.tokens), "ids": r.tokens}))
    return 0


def run_random(args) -> int:
    import torch
    from .engine.session import write_random_model
    with open(args.config, "r", encoding="utf-8") as handle:
        config = json.load(handle)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    path = write_random_model(args.out, config, seed=args.seed, std=args.std, norm_std=args.norm_std, dtype=dtype)
    print(path)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        if args.command == "inspect":
            print(json.dumps(run_inspect(args.model, args.tensors), indent=2))
            return 0
        if args.command == "generate":
            return run_generate(args)
        return run_random(args)
    except Exception as exc:  # the reference prints `error: ...` and exits 1 (main.rs:158-163)
        print(f"error: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
