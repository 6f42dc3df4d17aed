"""Command line in the manner of the reference's (src/main.rs:35-287): the verbs ``inspect``,
``run``, ``generate`` and ``bench`` with its option names, defaults and printed lines, plus
``init`` for the random-weights mode.  Prompts are token ids (comma or space separated, or
``@file``) since this engine has no tokenizer.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _ids(text):
    if text.startswith("@"):
        with open(text[1:], "r", encoding="utf-8") as f:
            text = f.read()
    parts = text.replace(",", " ").split()
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"error: token ids must be integers, got {text!r}")


def _add_engine_options(p):
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                   help="bfloat16: serving kernels; float32: everything in true 32-bit")
    p.add_argument("--device", default="cuda:0")


def build_parser():
    ap = argparse.ArgumentParser(prog="glint_b200", description="Gemma 2 inference on one B200")
    sub = ap.add_subparsers(dest="command", required=True)

    p = sub.add_parser("inspect", help="Inspect a SafeTensors model folder.")
    p.add_argument("-f", "--file", required=True, help="model folder (config.json + safetensors)")
    p.add_argument("--show-metadata", action="store_true", help="show the file's metadata pairs")
    p.add_argument("--show-tensors", action="store_true", help="show all tensor names, shapes and types")

    p = sub.add_parser("run", help="Generate from a model with a prompt of token ids.")
    p.add_argument("-f", "--file", required=True)
    p.add_argument("-p", "--prompt", required=True, help="token ids: '1,2,3' or @file")
    p.add_argument("-m", "--max-tokens", type=int, default=50)
    p.add_argument("--temperature", type=float, default=0.0, help="0.0 = greedy (default)")
    p.add_argument("--top-k", type=int, default=0, help="0 = disabled (default)")
    p.add_argument("--top-p", type=float, default=1.0, help="1.0 = disabled (default)")
    p.add_argument("--min-p", type=float, default=0.0, help="0.0 = disabled (default)")
    p.add_argument("--repeat-penalty", type=float, default=1.0, help="1.0 = disabled (default)")
    p.add_argument("--seed", type=int, default=None)
    _add_engine_options(p)

    p = sub.add_parser("generate", help="Generate tokens from raw token ids, greedily (for debugging).")
    p.add_argument("-f", "--file", required=True)
    p.add_argument("-t", "--tokens", required=True, help="prompt as comma-separated token ids")
    p.add_argument("-m", "--max-tokens", type=int, default=20)
    _add_engine_options(p)

    p = sub.add_parser("bench", help="Measure prefill, decode and serving throughput with roofline fractions.")
    p.add_argument("-f", "--file", default=None, help="model folder (the same as --shape <folder>)")
    p.add_argument("--shape", default=None, help="2b, 9b, 27b (random weights made on the device) or a model folder")
    p.add_argument("--mode", default="all", choices=["all", "prefill", "decode", "concurrency", "serve"],
                   help="concurrency: decode at the batch sizes 1, 2, 4 .. --max-concurrent")
    p.add_argument("--batch", default=None, help="decode batch sizes, e.g. 1,8,64 (default: 1, 2, 4 .. --max-concurrent)")
    p.add_argument("--prompt-len", type=int, default=512)
    p.add_argument("--decode-tokens", type=int, default=128)
    p.add_argument("--context", type=int, default=None, help="context limit of a named shape (default 8192)")
    p.add_argument("--layers", type=int, default=None, help="run fewer layers of a named shape")
    p.add_argument("--requests", type=int, default=64, help="requests of the serve workload")
    p.add_argument("--max-concurrent", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--output", default="table", choices=["table", "json"])
    _add_engine_options(p)

    p = sub.add_parser("init", help="Write a model folder with random weights from a config.json and a seed.")
    p.add_argument("-c", "--config", required=True, help="a config.json to take the sizes from")
    p.add_argument("-o", "--out", required=True, help="folder to write config.json and model.safetensors to")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--std", type=float, default=0.02)
    p.add_argument("--norm-std", type=float, default=0.1)
    p.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    return ap


def cmd_inspect(args):
    from .config import load_config, read_config_json
    from .weights import SafeTensorsModel
    files = SafeTensorsModel(args.file)
    config = load_config(args.file)
    total = sum(e.nbytes for e in files.entries.values())
    print(f"Model folder: {args.file}")
    print(f"Weight files: {len(files.files)}   Tensors: {len(files.entries)}   Bytes: {total:,}")
    print("Configuration:")
    for k, v in config.to_dict().items():
        print(f"  {k}: {v}")
    print("Model info:")
    for k, v in config.model_info().items():
        print(f"  {k}: {v}")
    if args.show_metadata:
        print("Metadata:")
        for f in files.files:
            for k, v in f.metadata.items():
                print(f"  {k}: {v}")
        for k, v in read_config_json(args.file).items():
            print(f"  config.{k}: {v}")
    if args.show_tensors:
        print("Tensors:")
        for name in sorted(files.entries):
            e = files.entries[name]
            print(f"  {name:60s} {e.dtype_name:5s} {list(e.shape)!s:20s} {e.nbytes:>12,} B")
    return 0


def cmd_run(args):
    from .engine.api import LLM
    prompt = _ids(args.prompt)
    llm = LLM(args.file, dtype=args.dtype, device=args.device, max_active=1)      # one prompt: a cache of four contexts
    print(f"Prompt: {prompt}")
    t0 = time.time()
    out = llm.generate(prompt, max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                       top_p=args.top_p, min_p=args.min_p, repeat_penalty=args.repeat_penalty, seed=args.seed)
    dt = time.time() - t0
    print(f"Output: {out}")
    print(f"({len(out)} tokens in {dt:.1f}s — {len(out) / max(dt, 1e-9):.1f} tok/s)")
    return 0


def cmd_generate(args):
    from .engine.api import LLM
    prompt = _ids(args.tokens)
    llm = LLM(args.file, dtype=args.dtype, device=args.device, max_active=1)      # one prompt: a cache of four contexts
    out = llm.generate(prompt, max_tokens=args.max_tokens, temperature=0.0)
    print(f"Generated token ids: {prompt + out}")
    return 0


def cmd_bench(args):
    from .bench import run_cli_bench
    result = run_cli_bench(args)
    if args.output == "json":
        print(json.dumps(result))
    else:
        for row in result["rows"]:
            print("  ".join(f"{k}={v}" for k, v in row.items()))
    return 0


def cmd_init(args):
    from .weights import write_random_model
    with open(args.config, "r", encoding="utf-8") as f:
        cfg = json.load(f)
    out = write_random_model(cfg, args.out, seed=args.seed, std=args.std, norm_std=args.norm_std,
                             store_dtype=args.store_dtype)
    print(f"wrote {out}/config.json and {out}/model.safetensors")
    return 0


def main(argv=None):
    args = build_parser().parse_args(argv)
    from .errors import GlintError
    try:
        return {"inspect": cmd_inspect, "run": cmd_run, "generate": cmd_generate, "bench": cmd_bench,
                "init": cmd_init}[args.command](args)
    except (GlintError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
