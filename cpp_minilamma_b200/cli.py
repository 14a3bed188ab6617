"""The `mini-llama` command line, in the reference's manner.

    mini-llama generate <model> [--backend cuda] [--device N] [--prompt|-p IDS]... [--n-predict|-n N]
                                [--seed N] [--temperature T] [--top-k K] [--dtype bfloat16|float32]
                                [--ignore-eos] [--verbose]
    mini-llama bench    <model> [--backend cuda] [-p IDS] [-n N] [--warmup N] [--seed N] [--dtype ...]
    mini-llama inspect  <model>
    mini-llama random   <folder> --config FILE [--seed N]       write a folder with random weights
    mini-llama --cuda-info [--device N]

Commands, option names, defaults (`-n` 4 for generate and 32 for bench, `--seed 1`,
`--warmup 2`, prompt "hello" replaced by token id 1) and the closing "trace summary" line
follow app/backend_cli.cc:59-188 and src/bench_strict.cc:30-93; a failure prints its
message to stderr, leaves stdout's result empty and returns 1 (capacity: 2, as
src/bench_strict.cc:273-279).  The library starts at token ids, so `--prompt` takes ids
("5 17 3" or "5,17,3"); give `-p` several times for a batch.  `--backend cpu`,
`--threads` and `--linear-mode` belong to the reference's CPU path: `cpu` is refused,
the other two are accepted and have no effect.  `--temperature` and `--top-k` expose the
sampler fields that the reference's CLI leaves at their defaults (include/sampler.h:7-15).
"""
from __future__ import annotations

import argparse
import itertools
import json
import sys
import time
from typing import List

_serial = itertools.count(1)


def trace_id() -> str:
    return f"{time.monotonic_ns()}-{next(_serial)}"


def parse_ids(text: str) -> List[int]:
    try:
        ids = [int(piece) for piece in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"Invalid --prompt value (token ids expected): {text}")
    if not ids:
        raise SystemExit("Prompt encoded to an empty sequence")
    return ids


def _common(sub, n_default):
    sub.add_argument("model")
    sub.add_argument("--backend", default="cuda")
    sub.add_argument("--device", type=int, default=0)
    sub.add_argument("--prompt", "-p", action="append", default=None)
    sub.add_argument("--n-predict", "-n", type=int, default=n_default)
    sub.add_argument("--seed", type=int, default=1)
    sub.add_argument("--temperature", type=float, default=0.0)
    sub.add_argument("--top-k", type=int, default=0)
    sub.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    sub.add_argument("--ignore-eos", action="store_true")
    sub.add_argument("--verbose", action="store_true")
    sub.add_argument("--threads", "-threads", type=int, default=0, help="no effect (CPU path of the reference)")
    sub.add_argument("--linear-mode", default="native", help="no effect (CPU path of the reference)")


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="mini-llama", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--cuda-info", action="store_true")
    parser.add_argument("--device", type=int, default=0, dest="info_device")
    subs = parser.add_subparsers(dest="command")
    _common(subs.add_parser("generate"), 4)
    bench = subs.add_parser("bench")
    _common(bench, 32)
    bench.add_argument("--warmup", type=int, default=2)
    subs.add_parser("inspect").add_argument("model")
    rnd = subs.add_parser("random")
    rnd.add_argument("model")
    rnd.add_argument("--config", required=True)
    rnd.add_argument("--seed", type=int, default=0)
    return parser


def cuda_info(device: int) -> None:
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("Backend setup failed: no CUDA device")
    props = torch.cuda.get_device_properties(device)
    print(f"cuda runtime: built\ncuda device count: {torch.cuda.device_count()}\ndevice name: {props.name}\n"
          f"compute capability: {props.major}.{props.minor}\ntotal memory: {props.total_memory}\n"
          f"runtime version: {torch.version.cuda}")


def inspect(folder: str) -> None:
    from . import build_model, load_config
    from .weights import ModelFiles
    config = load_config(folder)
    print(f"architecture: {config.architecture}")
    for key, value in config.to_dict().items():
        if key != "architectures":
            print(f"{key}: {json.dumps(value)}")
    model = build_model(config, "float32", "cpu", max_positions=1)
    print(f"parameters: {model.parameter_count()}")
    files = ModelFiles(folder)
    for name in sorted(files.entries):
        entry = files.entries[name]
        print(f"tensor {name} {list(entry.shape)} {str(entry.dtype).replace('torch.', '')}")


def _load(args, prompts):
    from . import load
    if args.backend not in ("cuda", "gpu"):
        raise RuntimeError(f"Backend setup failed: backend {args.backend!r} is not available; "
                           "this library has a CUDA path only (--backend cuda)")
    if args.n_predict < 0:
        raise RuntimeError(f"Invalid --n-predict value: {args.n_predict}")
    # like the reference (app/backend_cli.cc:149), allocate only the cache the request needs
    held = sum(-(-(len(p) + args.n_predict) // 64) * 64 for p in prompts)
    return load(args.model, dtype=args.dtype, device=f"cuda:{args.device}", max_tokens=max(held, 64),
                max_seqs=len(prompts))


def run_generate(args) -> None:
    prompts = [parse_ids(p) for p in (args.prompt or ["1"])]
    llm = _load(args, prompts)
    done = llm.generate_detailed(prompts, max_new_tokens=args.n_predict, temperature=args.temperature,
                                 top_k=args.top_k, seed=args.seed, ignore_eos=args.ignore_eos)
    for completion in done:
        print(" ".join(str(t) for t in completion.tokens))
        if args.verbose:
            print(f"finish reason: {completion.finish_reason}", file=sys.stderr)
    print(f"backend: cuda\ncuda device: {args.device}\ndtype: {args.dtype}")


def run_bench(args) -> None:
    import torch
    prompts = [parse_ids(p) for p in (args.prompt or ["1"])]
    began = time.perf_counter()
    llm = _load(args, prompts)
    load_ms = (time.perf_counter() - began) * 1e3
    options = dict(max_new_tokens=args.n_predict, temperature=args.temperature, top_k=args.top_k, seed=args.seed,
                   ignore_eos=True)  # a stop token is a normal token here (src/bench_strict.cc:159)
    for _ in range(max(args.warmup, 0)):
        llm.generate(prompts, **options)
    torch.cuda.synchronize()
    stats = {}
    llm.generate(prompts, stats=stats, **options)
    n = args.n_predict * len(prompts)
    prefill_ms, decode_ms = stats.get("prefill_s", 0.0) * 1e3, stats.get("decode_s", 0.0) * 1e3
    total = prefill_ms + decode_ms
    print(f"prompt tokens: {sum(len(p) for p in prompts)}\ngenerated tokens: {n}\n"
          f"prefill ms: {prefill_ms:.2f}\ndecode ms: {decode_ms:.2f}\ntotal ms: {total:.2f}")
    print("tokens/s (total): " + (f"{1000.0 * n / total:.2f}" if total > 0 else "unavailable"))
    decoded = n - len(prompts)
    print("tokens/s (decode): " + (f"{1000.0 * decoded / decode_ms:.2f}" if decoded > 0 and decode_ms > 0
                                   else "unavailable"))
    print(f"gpu memory used: {torch.cuda.max_memory_allocated() / 1e6:.2f} MB\nload ms: {load_ms:.3f}")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    tid = trace_id()
    try:
        args = build_parser().parse_args(argv)
        if args.cuda_info:
            cuda_info(args.info_device)
        elif args.command == "generate":
            run_generate(args)
        elif args.command == "bench":
            run_bench(args)
        elif args.command == "inspect":
            inspect(args.model)
        elif args.command == "random":
            from . import config_from_dict, write_random_model
            write_random_model(config_from_dict(json.load(open(args.config))), args.model, args.seed)
            print(f"wrote {args.model}")
        else:
            raise RuntimeError("Expected generate, bench, inspect, random or --cuda-info")
        print(f"trace summary: trace_id={tid} status=ok")
        return 0
    except SystemExit as exc:
        if exc.code in (0, None):
            return 0
        print(exc.code if isinstance(exc.code, str) else "invalid arguments", file=sys.stderr)
        print(f"trace summary: trace_id={tid} status=error", file=sys.stderr)
        return 1
    except Exception as exc:  # every failure: message on stderr, exit code 1 (capacity: 2)
        from .cache import CacheFull
        from .engine import GenerationError
        print(str(exc), file=sys.stderr)
        print(f"trace summary: trace_id={tid} status=error", file=sys.stderr)
        return 2 if isinstance(exc, (CacheFull, GenerationError)) else 1


if __name__ == "__main__":
    sys.exit(main())
