"""Decode and prefill throughput of the engine at the Llama-3.1-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line. `value`: decoded tokens per second at batch 8, timed on the device
with CUDA events over K decode steps after W warm-up steps, each request holding
a 2,048-token prompt (real prefill through the engine) and decoding from there.
`e2e`: the same through the Python entry point (Engine.submit / Engine.step),
host token lists in and host token ids out every step. `prefill`: one 2,048-token
prompt in one step. `roofline`: bytes the decode step must read (every weight
once, the cache of the live requests) over its time, against the measured copy
bandwidth. `points`: decode at batch 1 and 64 at the same context, and at batch 1,
8 and 64 at the end of the configuration's context (the K timed steps end at 4,096
tokens); their caches are filled with random keys and values instead of being
prefilled: a decode step's time does not depend on the cache's contents. Each has
its own entry in `rooflines`. Two serving runs through Engine.submit / Engine.step
follow, each with its own model (`serving`): `mixed_1b`, 64 requests with prompts of
128 to 4,096 tokens on the Llama-3.2-1B shape, prompts cut into portions of 512
beside the decoding requests, 512 new tokens each (and the same with a third of the
pages, so that requests are preempted and recomputed); `serve_13b`, 32 requests of
1,024 prompt tokens and 512 new tokens on the Llama-2-13B shape. They report
all tokens per second (prompt and generated, over the whole run) and generated
tokens per second of the phase in which every request decodes, against the bytes
such a step must read. Weights are random (N(0, 0.02)) and drawn on the device;
token ids are uniform random. The weights (16 GB) and caches are far larger than L2
(126 MB), so no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 32,
    "hidden_size": 4096,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "intermediate_size": 14336,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 131072,
}
LLAMA32_1B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 16,
    "hidden_size": 2048,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 64,
    "intermediate_size": 8192,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 131072,
}
LLAMA2_13B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 40,
    "hidden_size": 5120,
    "num_attention_heads": 40,
    "num_key_value_heads": 40,
    "head_dim": 128,
    "intermediate_size": 13824,
    "vocab_size": 32000,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "max_position_embeddings": 4096,
}
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PAGE_SIZE = 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timed work runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int = 0):
        self.index = index
        self.samples: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self) -> dict:
        sm, sm_max, reasons = [], [], set()
        for row in self.samples:
            try:
                sm.append(float(row[0]))
                sm_max.append(float(row[1]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(self.NAMES, row[2:]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_config(layers: int) -> dict:
    cfg = dict(LLAMA31_8B)
    cfg["num_hidden_layers"] = layers
    return cfg


def weight_bytes(cfg: dict, width: int = 2) -> int:
    """Bytes of every weight a decode step reads once: all layer matrices and norms,
    the final norm and the lm_head (embedding rows are gathered, not streamed)."""
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * h + h * nh * hd + 3 * i * h + 2 * h
    return (cfg["num_hidden_layers"] * per_layer + cfg["vocab_size"] * h + h) * width


def kv_bytes_per_token(cfg: dict, width: int = 2) -> int:
    return cfg["num_hidden_layers"] * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * width


def prefill_flops(cfg: dict, tokens: int, logit_rows: int = 1) -> float:
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = 2.0 * tokens * ((nh + 2 * nkv) * hd * h + h * nh * hd + 3 * i * h)
    attention = 4.0 * nh * hd * tokens * (tokens + 1) / 2
    return cfg["num_hidden_layers"] * (per_layer + attention) + 2.0 * logit_rows * cfg["vocab_size"] * h


def fill_cache(engine, batch: int, length: int, tag: str) -> list:
    """Opens `batch` requests holding `length` tokens each without running a
    prefill; the pools are filled with small random numbers once."""
    ids = []
    for b in range(batch):
        rid = (tag, b)
        assert engine.cache.open(rid) is not None, "too few slots"
        assert engine.cache.reserve(rid, length), "too few pages"
        engine.cache.commit(rid, length)
        ids.append(rid)
    return ids


def time_decode(engine, ids: list, steps: int, warmup: int, vocab: int):
    """K graph-replayed decode steps on the device (CUDA events). Tokens fed are
    fixed (the step's time does not depend on them); positions advance."""
    import torch

    from pulsarlm_b200.engine.runner import StepEntry
    from pulsarlm_b200.sampling.params import SamplingParams

    params = [SamplingParams()] * len(ids)
    seeds = [0] * len(ids)
    entries = [StepEntry(r, [(7 * i + 3) % vocab], [0]) for i, r in enumerate(ids)]
    for _ in range(warmup):
        engine.runner.decode_step(entries, params, seeds, [0] * len(ids))
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before_steps = engine.runner.graph_steps
    start.record()
    for _ in range(steps):
        engine.runner.decode_step(entries, params, seeds, [0] * len(ids))
    end.record()
    torch.cuda.synchronize()
    engine.runner.check_status()
    graph = engine.runner.last_graph
    launches = graph.launches * (engine.runner.graph_steps - before_steps)
    return start.elapsed_time(end) / steps, launches


def describe(cfg: dict) -> str:
    return (f"{cfg['num_hidden_layers']} layers, hidden {cfg['hidden_size']}, heads {cfg['num_attention_heads']}/"
            f"{cfg['num_key_value_heads']}, head_dim {cfg['head_dim']}, intermediate {cfg['intermediate_size']}, "
            f"vocab {cfg['vocab_size']}, {'tied' if cfg['tie_word_embeddings'] else 'untied'} head")


def serve(engine, cfg: dict, prompts: list, max_new: int, pk: dict) -> dict:
    """Submits every prompt at once and steps the engine until all are done (host token
    lists in, host token ids out). Times the whole run, and within it the phase in
    which every request is decoding (from the step after the last prompt ends to the
    first request's end), whose steps are compared with the bytes they must read."""
    import torch

    from pulsarlm_b200 import SamplingParams

    greedy = SamplingParams(temperature=0.0)
    captures_before = engine.runner.graph_captures
    steps_before = engine.runner.steps
    preempted_before = engine.scheduler.preemptions
    torch.cuda.synchronize()
    t_start = time.perf_counter()
    requests = [engine.submit(p, sampling=greedy, max_tokens=max_new, ignore_eos=True) for p in prompts]
    weights = weight_bytes(cfg)
    per_token = kv_bytes_per_token(cfg)
    phase = None  # [seconds at start, tokens generated at start, steps, bytes]
    closed = None
    while engine.has_work():
        everyone_decodes = closed is None and all(r.output and not r.finished for r in requests)
        if everyone_decodes and phase is None:
            engine.sync()
            torch.cuda.synchronize()
            phase = [time.perf_counter(), sum(len(r.output) for r in requests), 0, 0.0]
        elif phase is not None and closed is None and not everyone_decodes:
            engine.sync()
            torch.cuda.synchronize()
            closed = (time.perf_counter(), sum(len(r.output) for r in requests))
        if phase is not None and closed is None:
            phase[2] += 1
            phase[3] += weights + per_token * sum(len(r.prompt) + len(r.output) for r in requests)
        engine.step()
    engine.sync()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t_start
    engine.runner.check_status()
    assert all(r.finish_reason == "length" and len(r.output) == max_new for r in requests), "a request fell short"
    prompt_tokens = sum(len(p) for p in prompts)
    generated = sum(len(r.output) for r in requests)
    out = {"requests": len(prompts), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
           "seconds": seconds, "tok_s": (prompt_tokens + generated) / seconds,
           "steps": engine.runner.steps - steps_before,
           "preemptions": engine.scheduler.preemptions - preempted_before,
           "graph_captures_in_run": engine.runner.graph_captures - captures_before}
    if phase is not None and closed is not None and phase[2] > 0:
        span = closed[0] - phase[0]
        bytes_per_step = phase[3] / phase[2]
        ms = span / phase[2] * 1e3
        out.update({"decode_tok_s": (closed[1] - phase[1]) / span, "decode_steps": phase[2], "decode_ms_per_step": ms,
                    "decode_bytes_per_step": bytes_per_step,
                    "decode_floor_ms": bytes_per_step / (pk["hbm_gbs"] * 1e9) * 1e3,
                    "decode_frac": bytes_per_step / (ms / 1e3) / 1e9 / pk["hbm_gbs"]})
    return out


def run_serving(name: str, cfg: dict, lengths: list, max_new: int, pk: dict, tight: bool) -> dict:
    """Builds the model, serves a warm-up pass over the same prompts (library set-up,
    the decode steps' captures), then the timed pass; with `tight`, once more with a third
    of the pages, so that the scheduler has to preempt and recompute."""
    import gc

    import torch

    from pulsarlm_b200 import Engine

    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    need_pages = sum(-(-(n + max_new + 2) // PAGE_SIZE) for n in lengths)
    engine = Engine(cfg, dtype="bfloat16", device="cuda:0", n_pages=need_pages + 64, page_size=PAGE_SIZE,
                    prefill_tokens_per_step=512, max_requests=len(lengths), seed=0)
    # The warm-up pass is the whole workload once: every shape of decode step that the timed
    # pass meets has then been captured, as in an engine that has been serving for a while.
    serve(engine, cfg, prompts, max_new, pk)
    result = serve(engine, cfg, prompts, max_new, pk)
    result["model"] = describe(cfg)
    result["prefill_tokens_per_step"] = 512
    if tight:
        small = Engine(engine.model, n_pages=max(need_pages // 3, -(-(max(lengths) + max_new + 2) // PAGE_SIZE) + 1),
                       page_size=PAGE_SIZE, prefill_tokens_per_step=512, max_requests=len(lengths))
        serve(small, cfg, prompts, min(128, max_new), pk)  # (warm-up: this engine's own captures)
        pressed = serve(small, cfg, prompts, min(128, max_new), pk)
        result["tight_pages"] = {k: pressed[k] for k in ("tok_s", "seconds", "steps", "preemptions",
                                                          "generated_tokens")}
        result["tight_pages"]["pages"] = small.cache.n_pages
        result["tight_pages"]["pages_for_everyone"] = need_pages
        del small
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return result


def run_ours(args) -> dict:
    import torch

    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.runner import StepEntry

    pk = peaks()
    cfg = model_config(args.layers)
    batch = args.batch
    torch.manual_seed(0)
    device = "cuda:0"
    max_batch = max(64, batch)
    phases = set(args.phases.split(","))
    per_request = CONTEXT_LEN + 64 if "ctx4096" in phases else PROMPT_LEN + 2 * (args.steps + args.warmup) + 128
    tokens_room = max_batch * per_request + 4 * PROMPT_LEN
    tokens_room = max(tokens_room, args.prefill_tokens + 4 * PROMPT_LEN)
    n_pages = -(-tokens_room // PAGE_SIZE)
    t0 = time.time()
    engine = Engine(cfg, dtype="bfloat16", device=device, n_pages=n_pages, page_size=PAGE_SIZE,
                    prefill_tokens_per_step=PROMPT_LEN, max_requests=max_batch + 2, seed=0)
    for g in engine.cache.groups:
        g.tensor.normal_(0.0, 0.5)
    vocab = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(1)
    setup_s = time.time() - t0

    prefill = e2e = None
    points: dict = {}
    rooflines: dict = {}
    serving: dict = {}

    def decode_point(name: str, b: int, first_context: int, steps: int) -> None:
        ids = fill_cache(engine, b, first_context, name)
        ms, _ = time_decode(engine, ids, steps, args.warmup, vocab)
        mid_context = first_context + args.warmup + steps / 2
        step_bytes = weight_bytes(cfg) + b * mid_context * kv_bytes_per_token(cfg)
        points[name] = b / (ms / 1e3)
        rooflines[name] = {"ms": ms, "context": mid_context, "bytes_per_step": step_bytes,
                           "achieved": step_bytes / (ms / 1e3) / 1e9,
                           "frac": step_bytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"]}
        for rid in ids:
            engine.cache.close(rid)

    ms_per_step, launches, achieved, step_bytes = None, 0, None, None
    clocks = ClockSampler()

    # ---- prefill: one 2,048-token prompt in one step, logits of the last token.
    if "prefill" in phases:
        n_prompt = args.prefill_tokens
        prompt = torch.randint(0, vocab, (n_prompt,), generator=gen).tolist()
        times = []
        for i in range(3 + 5):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.runner.step([StepEntry(("prefill", i), prompt, [n_prompt - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.runner.end(("prefill", i))
            if i >= 3:
                times.append(start.elapsed_time(end))
        prefill_ms = statistics.median(times)
        flops = prefill_flops(cfg, n_prompt)
        prefill = {"value": n_prompt / (prefill_ms / 1e3), "tokens": n_prompt, "ms": prefill_ms,
                   "frac": flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "unit": "tok/s",
                   "peak_tflops": pk["bf16_tflops"]}

    # ---- end to end through the public API: batch prompts in, tokens out per step.
    if "e2e" in phases:
        prompts = [torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist() for _ in range(batch)]
        sampling = SamplingParams(temperature=0.0)
        # Requests finish their prompts one step apart, so the first is `batch` tokens
        # ahead of the last: give all of them room to still be decoding at the end.
        total_new = args.warmup + args.steps + batch + 8
        requests = [engine.submit(p, sampling=sampling, max_tokens=total_new, ignore_eos=True) for p in prompts]
        while any(len(r.output) < 1 for r in requests):
            engine.step()  # prefill (untimed)
        for _ in range(args.warmup):
            engine.step()
        engine.sync()  # the engine pipelines decode steps one deep: nothing in flight at the start,
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        for _ in range(args.steps):
            engine.step()
        engine.sync()  # and every timed step's tokens read on the host at the end
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t_start
        assert all(not r.finished and len(r.output) >= args.warmup + args.steps + 1 for r in requests)
        graph = next(g for (n, _), g in engine.runner._graphs.items() if n == batch)
        e2e = {"value": batch * args.steps / e2e_s, "unit": "tok/s", "ms_per_step": e2e_s / args.steps * 1e3,
               "h2d_bytes_per_step": graph.layout.nbytes, "d2h_bytes_per_step": 4 * batch}
        for r in requests:
            r.cancel()
        engine.step()

    # ---- device-timed decode at the headline batch, same context.
    if "decode" in phases:
        ids = fill_cache(engine, batch, PROMPT_LEN + args.warmup, "main")
        with clocks:
            ms_per_step, launches = time_decode(engine, ids, args.steps, args.warmup, vocab)
        mid_context = PROMPT_LEN + 2 * args.warmup + args.steps / 2
        step_bytes = weight_bytes(cfg) + batch * mid_context * kv_bytes_per_token(cfg)
        achieved = step_bytes / (ms_per_step / 1e3) / 1e9
        for rid in ids:
            engine.cache.close(rid)

    # ---- other batch sizes.
    if "points" in phases:
        for b in (1, 64):
            decode_point(f"decode_b{b}", b, PROMPT_LEN, max(8, args.steps // 2))

        # a long prompt in the default portions: 8,192 tokens, 256 a step (tokens a second)
        long_prompt = torch.randint(0, vocab, (4 * PROMPT_LEN,), generator=gen).tolist()
        for attempt in ("warm", "timed"):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for at in range(0, len(long_prompt), 256):
                last = at + 256 >= len(long_prompt)
                engine.runner.step([StepEntry(("long", attempt), long_prompt[at:at + 256], [255] if last else [])])
            end.record()
            torch.cuda.synchronize()
            engine.runner.end(("long", attempt))
        points["prefill_8192_by_256"] = len(long_prompt) / (start.elapsed_time(end) / 1e3)
        # the same through the public entry point: milliseconds from submit to the first
        # token of a 2,048-token prompt, the scheduler cutting it into its default portions
        served = Engine(engine.model, n_pages=PROMPT_LEN // PAGE_SIZE + 8, page_size=PAGE_SIZE,
                        prefill_tokens_per_step=256, max_requests=2)
        first_prompt = torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist()
        for attempt in ("warm", "timed"):
            torch.cuda.synchronize()
            t_start = time.perf_counter()
            request = served.submit(first_prompt, sampling=SamplingParams(temperature=0.0), max_tokens=1,
                                    ignore_eos=True)
            while not request.finished:
                served.step()
            served.sync()
            points["first_token_ms_2048_by_256"] = (time.perf_counter() - t_start) * 1e3

    # ---- the end of the configuration's context: the timed steps end at 4,096 tokens.
    if "ctx4096" in phases:
        steps = max(8, args.steps // 2)
        for b in (1, 8, 64):
            decode_point(f"decode_b{b}_ctx4096", b, CONTEXT_LEN - steps - args.warmup, steps)

    # ---- serving runs on the other two shapes, each with its own model.
    if phases & {"mixed_1b", "serve_13b"}:
        import gc

        served = None
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        if "mixed_1b" in phases:
            lengths = torch.randint(128, 4097, (64,), generator=torch.Generator().manual_seed(3)).tolist()
            serving["mixed_1b"] = run_serving("mixed_1b", LLAMA32_1B, lengths, 512, pk, tight=True)
        if "serve_13b" in phases:
            serving["serve_13b"] = run_serving("serve_13b", LLAMA2_13B, [1024] * 32, 512, pk, tight=False)
        for name, run in serving.items():
            points[f"{name}_tok_s"] = run["tok_s"]
            if "decode_tok_s" in run:
                points[f"{name}_decode_tok_s"] = run["decode_tok_s"]
                rooflines[f"{name}_decode"] = {"ms": run["decode_ms_per_step"],
                                               "bytes_per_step": run["decode_bytes_per_step"],
                                               "achieved": run["decode_bytes_per_step"] / run["decode_ms_per_step"] / 1e6,
                                               "frac": run["decode_frac"]}

    clock_summary = clocks.summary()
    return {
        "metric": "decode tok/s at batch 8 (Llama-3.1-8B shape, 2,048-token prompts)",
        "value": batch / (ms_per_step / 1e3) if ms_per_step else None,
        "unit": "tok/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02) drawn on the device, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Llama-3.1-8B shape", "layers": cfg["num_hidden_layers"], "layers_full": 32,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "global_batch": batch, "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN,
            "decode_context_start": PROMPT_LEN + args.warmup, "page_size": PAGE_SIZE,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 16 GB)",
            "peaks": pk["source"],
            "mixed_1b_model": "Llama-3.2-1B shape: " + describe(LLAMA32_1B),
            "serve_13b_model": "Llama-2-13B shape: " + describe(LLAMA2_13B),
        },
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"] if achieved else None, "bytes_per_step": step_bytes},
        "points": points,
        "rooflines": rooflines,
        "serving": serving,
        "clocks": {"sm_mhz": clock_summary["sm_mhz"], "sm_max_mhz": clock_summary["sm_max_mhz"],
                   "reasons": clock_summary["reasons"]},
        "setup_s": setup_s,
    }


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=128)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--layers", type=int, default=32, help="fewer layers than the model's 32 (named in config)")
    p.add_argument("--prefill_tokens", type=int, default=PROMPT_LEN,
                   help="length of the prompt of the prefill phase (the contract's figure is the default's)")
    p.add_argument("--phases", default="prefill,e2e,decode,points,ctx4096,mixed_1b,serve_13b",
                   help="which measurements to run (a profiler run wants one): "
                        "prefill,e2e,decode,points,ctx4096,mixed_1b,serve_13b")
    args = p.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "cosmonomic/pulsarlm does not install offline here: its build needs hatchling, Python >= 3.13, "
                          "torch 2.15, xmake, CUDA 13.2 and gcc 15, none of which this image has"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    args.warmup = max(3, args.warmup)
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
