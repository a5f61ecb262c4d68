"""Command line: `python -m pulsarlm_b200 <command>`.

Commands and options follow the reference's CLI where it has them
(pulsarlm/src/pulsarlm/cli/__init__.py:179-340; its option names use
underscores): `chat MODEL --system --temperature --top_p --top_k --dtype
--kv_cache_gib --prefill_tokens_per_step --device`. Added for an engine without
a model catalogue: `generate` (token ids in, token ids out), `bench` (tokens a
second of a batch of random prompts), `models random` (write a random model
folder) and `replay` (trace replay). Wherever a model folder is taken,
`--random_weights SEED --config FILE` stands for one: the model FILE (a
config.json) describes, with weights drawn from SEED on the device.
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def _engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("model", nargs="?", default=None,
                   help="model folder (config.json, model.safetensors[, tokenizer.json])")
    p.add_argument("--random_weights", "--random-weights", type=int, default=None, metavar="SEED",
                   help="instead of a model folder: random weights drawn from this seed (needs --config)")
    p.add_argument("--config", default=None, help="with --random_weights: the config.json that gives the sizes")
    p.add_argument("--device", default="cuda:0", help="CUDA device to run on")
    p.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"], help="weight and KV dtype")
    p.add_argument("--kv_cache_gib", type=float, default=4.0, help="size of the KV cache pool in GiB")
    p.add_argument("--prefill_tokens_per_step", type=int, default=256,
                   help="most prompt tokens forwarded in one step")
    p.add_argument("--page_size", type=int, default=16, help="tokens per KV cache page")


def _sampling_options(p: argparse.ArgumentParser, temperature: float) -> None:
    p.add_argument("--temperature", type=float, default=temperature,
                   help="sampling temperature; 0 takes the argmax")
    p.add_argument("--top_p", type=float, default=1.0, help="nucleus mass; 1 keeps every token")
    p.add_argument("--top_k", type=int, default=0, help="keep the k most probable tokens; 0 keeps all")
    p.add_argument("--seed", type=int, default=None, help="sampling seed; default: a fresh one per request")
    p.add_argument("--max_tokens", type=int, default=None, help="most tokens generated per reply")


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="pulsarlm_b200", description="Single-GPU inference engine for B200.")
    sub = parser.add_subparsers(dest="command", required=True)

    chat = sub.add_parser("chat", help="chat with a model in the terminal")
    _engine_options(chat)
    _sampling_options(chat, temperature=1.0)
    chat.add_argument("--system", default=os.environ.get("PULSARLM_SYSTEM_PROMPT"),
                      help="a system message opening the conversation")

    gen = sub.add_parser("generate", help="generate from token ids or text")
    _engine_options(gen)
    _sampling_options(gen, temperature=0.0)
    gen.add_argument("--prompt_ids", action="append", default=[],
                     help="comma-separated token ids; repeat for several prompts")
    gen.add_argument("--prompt", action="append", default=[], help="text prompt (needs tokenizer.json)")
    gen.add_argument("--ignore_eos", action="store_true", help="do not stop at eos_token_id")

    bench = sub.add_parser("bench", help="tokens a second of a batch of random prompts")
    _engine_options(bench)
    bench.add_argument("--batch", type=int, default=8, help="requests submitted at once")
    bench.add_argument("--prompt_len", type=int, default=512, help="tokens of every prompt")
    bench.add_argument("--new_tokens", type=int, default=128, help="tokens generated per request")
    bench.add_argument("--seed", type=int, default=0, help="seed of the prompts")

    models = sub.add_parser("models", help="model folders")
    msub = models.add_subparsers(dest="models_command", required=True)
    rnd = msub.add_parser("random", help="write a model folder with random weights")
    rnd.add_argument("out", help="folder to create")
    rnd.add_argument("--config", required=True, help="a config.json to take sizes from")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"])
    rnd.add_argument("--std", type=float, default=0.02)
    msub.add_parser("list", help="list registered architectures")

    replay = sub.add_parser("replay", help="trace replay; same options as bin/trace_run", add_help=False)
    replay.add_argument("rest", nargs=argparse.REMAINDER)
    return parser


def _load_tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


class UsageError(ValueError):
    pass


def _model_argument(args):
    """The model folder, or the configuration to draw random weights for."""
    if args.random_weights is not None:
        if args.model is not None or args.config is None:
            raise UsageError("--random_weights SEED takes --config FILE and no model folder")
        with open(args.config, "r", encoding="utf-8") as f:
            return json.load(f), args.random_weights
    if args.model is None:
        raise UsageError("give a model folder, or --random_weights SEED --config FILE")
    if args.config is not None:
        raise UsageError("--config goes with --random_weights")
    return args.model, None


def _make_engine(args, **more):
    from .engine.engine import Engine

    model, seed = _model_argument(args)
    return Engine(model, dtype=args.dtype, device=args.device, kv_cache_gib=args.kv_cache_gib,
                  page_size=args.page_size, prefill_tokens_per_step=args.prefill_tokens_per_step, seed=seed, **more)


def run_bench(args) -> int:
    """Submits `batch` prompts of `prompt_len` random token ids, generates `new_tokens`
    for each (stop tokens ignored) and prints one JSON line: tokens a second over the
    whole run, and of the prompt phase and the decode phase apart (host clock around
    device synchronisations; a warm-up pass runs first)."""
    import time

    import torch

    from .sampling.params import SamplingParams

    engine = _make_engine(args, max_requests=max(1, args.batch))
    gen = torch.Generator().manual_seed(args.seed)
    prompts = [torch.randint(0, engine.vocab_size, (args.prompt_len,), generator=gen).tolist()
               for _ in range(args.batch)]
    greedy = SamplingParams(temperature=0.0)
    record = {}
    for attempt in ("warm-up", "timed"):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        requests = [engine.submit(p, sampling=greedy, max_tokens=args.new_tokens, ignore_eos=True) for p in prompts]
        while any(not r.output and not r.finished for r in requests):
            engine.step()
        engine.sync()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        while engine.has_work():
            engine.step()
        engine.sync()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        generated = sum(len(r.output) for r in requests)
        record = {"batch": args.batch, "prompt_len": args.prompt_len, "new_tokens": args.new_tokens,
                  "dtype": args.dtype, "prompt_tok_s": args.batch * args.prompt_len / (t1 - t0),
                  "decode_tok_s": (generated - args.batch) / (t2 - t1) if t2 > t1 and generated > args.batch else None,
                  "tok_s": (args.batch * args.prompt_len + generated) / (t2 - t0), "seconds": t2 - t0,
                  "preemptions": engine.scheduler.preemptions}
    engine.runner.check_status()
    print(json.dumps(record))
    return 0


def _sampling(args):
    from .sampling.params import SamplingParams

    return SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, seed=args.seed)


def _chat_turn(tokenizer, role: str, text: str) -> list[int]:
    """Llama-3 style header framing when the tokenizer knows the header tokens,
    else the plain text."""
    framed = f"<|start_header_id|>{role}<|end_header_id|>\n\n{text}<|eot_id|>"
    if tokenizer.token_to_id("<|start_header_id|>") is not None:
        return tokenizer.encode(framed, add_special_tokens=False).ids
    return tokenizer.encode(text + "\n", add_special_tokens=False).ids


def run_chat(args) -> int:
    from .engine.engine import complete

    engine = _make_engine(args)
    tokenizer = _load_tokenizer(args.model) if args.model else None
    sampling = _sampling(args)
    history: list[int] = []
    if tokenizer is None:
        print("no tokenizer.json in the model folder: type token ids separated by spaces", file=sys.stderr)
    else:
        bos = tokenizer.token_to_id("<|begin_of_text|>")
        if bos is not None:
            history.append(bos)
        if args.system:
            history += _chat_turn(tokenizer, "system", args.system)
    extra_stops = set()
    if tokenizer is not None:
        for name in ("<|eot_id|>", "<|end_of_text|>", "<|endoftext|>"):
            if tokenizer.token_to_id(name) is not None:
                extra_stops.add(tokenizer.token_to_id(name))
    engine.scheduler.stop_ids = frozenset(engine.scheduler.stop_ids | extra_stops)
    while True:
        try:
            line = input(">>> ")
        except EOFError:
            print()
            return 0
        if not line.strip():
            continue
        if tokenizer is None:
            try:
                history += [int(t) for t in line.replace(",", " ").split()]
            except ValueError:
                print("token ids must be integers", file=sys.stderr)
                continue
        else:
            history += _chat_turn(tokenizer, "user", line)
            if tokenizer.token_to_id("<|start_header_id|>") is not None:
                history += tokenizer.encode("<|start_header_id|>assistant<|end_header_id|>\n\n",
                                            add_special_tokens=False).ids
        reply: list[int] = []
        shown = ""
        max_tokens = args.max_tokens if args.max_tokens is not None else (None if engine.scheduler.stop_ids else 256)
        try:
            for token in complete(engine, history, sampling=sampling, max_tokens=max_tokens):
                reply.append(token)
                if tokenizer is None:
                    print(token, end=" ", flush=True)
                else:
                    text = tokenizer.decode(reply, skip_special_tokens=True)
                    print(text[len(shown):], end="", flush=True)
                    shown = text
        except (ValueError, MemoryError) as error:
            print(f"\nerror: {error}", file=sys.stderr)
        print()
        history += reply


def run_generate(args) -> int:
    engine = _make_engine(args)
    tokenizer = _load_tokenizer(args.model) if args.model else None
    prompts = [[int(t) for t in ids.replace(",", " ").split()] for ids in args.prompt_ids]
    if args.prompt:
        if tokenizer is None:
            print("error: --prompt needs tokenizer.json in the model folder; use --prompt_ids", file=sys.stderr)
            return 1
        prompts += [tokenizer.encode(text).ids for text in args.prompt]
    if not prompts:
        print("error: give --prompt_ids or --prompt", file=sys.stderr)
        return 1
    max_tokens = args.max_tokens if args.max_tokens is not None else 16
    outputs = engine.generate(prompts, _sampling(args), max_tokens=max_tokens, ignore_eos=args.ignore_eos)
    for prompt, out in zip(prompts, outputs):
        record = {"prompt_ids": prompt, "output_ids": out}
        if tokenizer is not None:
            record["text"] = tokenizer.decode(out)
        print(json.dumps(record))
    return 0


def run_models(args) -> int:
    from . import models  # noqa: F401
    from .config.registry import registered_architectures

    if args.models_command == "list":
        for name in registered_architectures():
            print(name)
        return 0
    import torch

    from .weights.random_init import write_random_model

    with open(args.config, "r", encoding="utf-8") as f:
        text = json.load(f)
    dtype = torch.float32 if args.dtype == "float32" else torch.bfloat16
    write_random_model(args.out, text, args.seed, dtype, std=args.std)
    print(args.out)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .config.base import ConfigError
    from .weights.loader import WeightsError

    try:
        if args.command == "chat":
            return run_chat(args)
        if args.command == "generate":
            return run_generate(args)
        if args.command == "bench":
            return run_bench(args)
        if args.command == "models":
            return run_models(args)
        if args.command == "replay":
            from .engine.trace import run

            return run(args.rest)
    except (ConfigError, WeightsError, UsageError) as error:
        print(f"error: {error}", file=sys.stderr)
        return 1
    return 2
