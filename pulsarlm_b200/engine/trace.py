"""Trace replay: given token ids are fed through the model step by step and the
logits at the wanted places are written out. Nothing is sampled.

It drives the same model, step function, cache manager and kernels that
generation uses (ModelRunner.step); it has no forward pass, cache or loader of
its own.

Input, one JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: for each request its next tokens and the places among them whose
logits are wanted. All entries of a step run as one batch. `end`: requests that
are finished after this step; their pages and slot are given back. For a step
that wants something, `<out>/<step>.f32` holds the logits as little-endian
float32 [wanted, vocab], in the order of the entries and of `want`. After every
step a line `done <step>` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys


DEFAULT_PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 16


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", default=None, help="folder with config.json and model.safetensors")
    p.add_argument("--random-weights", "--random_weights", type=int, default=None, metavar="SEED",
                   help="instead of --model: random weights drawn from this seed for the model --config describes")
    p.add_argument("--config", default=None, help="with --random-weights: a config.json")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    p.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE, help="tokens per cache page")
    p.add_argument("--device", default="cuda:0")
    return p


def run(argv=None, stdin=None, stdout=None) -> int:
    args = build_parser().parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if (args.model is None) == (args.random_weights is None) or (args.random_weights is not None) != (
            args.config is not None):
        print("trace_run: give --model DIR, or --random-weights SEED with --config FILE", file=sys.stderr)
        return 2
    if args.max_tokens <= 0:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    if args.page_size <= 0 or 64 % args.page_size != 0:
        print("trace_run: --page-size must divide 64", file=sys.stderr)
        return 2

    import torch

    from ..cache.manager import CacheManager
    from ..kernels import ops
    from .loading import load_model, parse_dtype, random_model
    from .runner import ModelRunner, StepEntry

    ops.require_device()
    os.makedirs(args.out, exist_ok=True)
    dtype = parse_dtype(args.dtype)
    device = torch.device(args.device)
    torch.cuda.set_device(device)
    if args.random_weights is not None:
        with open(args.config, "r", encoding="utf-8") as f:
            model = random_model(json.load(f), args.random_weights, dtype, device)
    else:
        model = load_model(args.model, dtype, device)
    n_pages = -(-args.max_tokens // args.page_size)
    cache = CacheManager(model.cache_needs(), args.page_size, n_pages, MAX_LIVE_REQUESTS, dtype, device)
    runner = ModelRunner(model, cache)

    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in record.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                host = logits.to("cpu", torch.float32).contiguous().numpy()
                host.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
            runner.check_status()
        for request in record.get("end", []):
            runner.end(request)
        stdout.write(f"done {step}\n")
        stdout.flush()
    return 0


def main() -> None:
    sys.exit(run())
