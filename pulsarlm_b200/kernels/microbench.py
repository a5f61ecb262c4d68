"""Device timings of single kernels at given sizes.

    python -m pulsarlm_b200.kernels.microbench gemm [--shapes T,N,K ...]
    python -m pulsarlm_b200.kernels.microbench attention_prefill [--tokens 2048 ...]
    python -m pulsarlm_b200.kernels.microbench attention_decode [--batch 8 --context 2048 ...]
    python -m pulsarlm_b200.kernels.microbench decode_timeline [--layers 8 --batch 8 --context 2048]
        [--shape 1b --batch 64 --context 128 4608]   (contexts spread evenly between the two)
    python -m pulsarlm_b200.kernels.microbench mixed_steps [--shape 1b --layers 16]

Each timing replays a CUDA graph of several launches (so host time does not
count) over inputs rotated through enough copies to exceed L2, after warm-up,
between CUDA events. Prints one line per case with achieved GB/s and TFLOP/s.
`gemm` times the tcgen05 kernels (skinny up to 64 tokens, pair above) beside the library
product torch.mm calls.
`decode_timeline` replays the engine's captured decode step of a Llama-3.1-8B-shaped
model (random weights, fewer layers) under the torch profiler's CUDA activity trace and
prints when each kernel of one layer starts and ends inside the graph: kernels overlap
(programmatic dependent launch), so the differences of the END times are what each costs.
`mixed_steps` runs the engine's eager steps under a serving load (prompt portions beside
single tokens) and prints a step's wall time beside the sum of its kernels' times.
"""

from __future__ import annotations

import argparse
import math

import torch

from . import ops

LLAMA8B_SHAPES = [(8, 6144, 4096), (8, 4096, 4096), (8, 28672, 4096), (8, 4096, 14336), (64, 6144, 4096),
                  (64, 28672, 4096), (2048, 6144, 4096), (2048, 4096, 4096), (2048, 28672, 4096), (2048, 4096, 14336)]


def graph_time_us(fn, reps: int = 10, iters: int = 10) -> float:
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / (iters * reps) * 1e3


def bench_gemm(shapes) -> None:
    for t, n, k in shapes:
        copies = max(2, min(10, int(600e6 // (n * k * 2)) + 1))
        weights = [(torch.randn(n, k, device="cuda") / 64).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(t, k, device="cuda").to(torch.bfloat16)
        out = torch.empty(t, n, device="cuda", dtype=torch.bfloat16)
        turn = [0]

        def own(kernel):
            def run():
                ops.gemm_bf16(x, weights[turn[0] % copies], out, kernel=kernel)
                turn[0] += 1
            return run

        def library():
            torch.mm(x, weights[turn[0] % copies].t(), out=out)
            turn[0] += 1

        gb, tf = n * k * 2 / 1e9, 2.0 * t * n * k / 1e12
        line = f"gemm t={t} n={n} k={k}:"
        if t <= ops.GEMM_GATED_IN_MAX_TOKENS:
            # the same product fed by a gate/up output: the SwiGLU kernel then the product, or the
            # activation made inside the product
            gate_up = torch.randn(t, 2 * k, device="cuda").to(torch.bfloat16)

            def two_kernels():
                ops.swiglu(gate_up, x)
                ops.gemm_bf16(x, weights[turn[0] % copies], out, kernel="skinny")
                turn[0] += 1

            def one_kernel():
                ops.gemm_bf16_gated_in(gate_up, weights[turn[0] % copies], out)
                turn[0] += 1

            line += f" | swiglu + skinny {graph_time_us(two_kernels):.1f} us | gated in {graph_time_us(one_kernel):.1f} us"
        for name in (["skinny"] if t <= ops.GEMM_SKINNY_MAX_TOKENS else []) + ["pair", "library"]:
            us = graph_time_us(library if name == "library" else own(name))
            line += f" | {name} {us:.1f} us ({gb / us * 1e6:.0f} GB/s, {tf / us * 1e6:.0f} TFLOP/s)"
        print(line, flush=True)


def bench_attention_prefill(tokens_list, n_heads, n_kv, head_dim, page, prior=0, force_splits=0,
                            cuda_cores=False) -> None:
    """A portion of `tokens` queries that follows `prior` keys already in the cache."""
    from ..parts.attention import prefill_splits

    for tokens in tokens_list:
        n_pages = (tokens + prior) // page + 4
        pool = (torch.randn(n_pages, 2, n_kv, page, head_dim, device="cuda") * 0.5).to(torch.bfloat16)
        kp, vp = pool[:, 0], pool[:, 1]
        table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(1, -1)
        qkv = torch.randn(tokens, (n_heads + 2 * n_kv) * head_dim, device="cuda").to(torch.bfloat16)
        q = qkv[:, : n_heads * head_dim].view(tokens, n_heads, head_dim)
        out = torch.empty(tokens, n_heads, head_dim, device="cuda", dtype=torch.bfloat16)
        def tile_list(rows):
            tiles = sorted(((r, min(rows, tokens - r), prior + r, 0) for r in range(0, tokens, rows)),
                           key=lambda t: -(t[1] + t[2]))
            return torch.tensor(tiles, dtype=torch.int32, device="cuda")

        tiles = tile_list(ops.attention_prefill_tile_rows())
        wide = (n_heads // n_kv) % 2 == 1  # one head per CTA: tiles of twice the rows
        wide_tiles = tile_list(ops.attention_prefill_tcgen05_tile_rows(n_heads // n_kv))
        scale = 1 / math.sqrt(head_dim)
        flops = 4.0 * n_heads * head_dim * (tokens * (tokens + 1) / 2 + tokens * prior)
        # the engine's choice: few tiles over many keys are split over the keys
        ctas = wide_tiles.shape[0] * n_heads if wide else tiles.shape[0] * n_heads // 2
        splits = force_splits or prefill_splits(ctas, tokens + prior, tokens, n_heads, head_dim, q.device)
        scratch = torch.empty(max(1, ops.attention_prefill_scratch_floats(tokens, n_heads, head_dim, splits)),
                              device="cuda")

        def tcgen05(q, kp, vp, table, tiles, *args):
            ops.attention_prefill_tcgen05(q, kp, vp, table, wide_tiles if wide else tiles, *args, None, splits,
                                          scratch, wide)

        def simt(q, kp, vp, table, tiles, out, page, window, scale):
            ops.attention_simt(q, kp, vp, table, positions, torch.zeros_like(positions), out, page, window, scale)

        positions = torch.arange(prior, prior + tokens, dtype=torch.int32, device="cuda")
        kernels = [("mma.sync", ops.attention_prefill)]
        if head_dim in (64, 128):
            kernels.insert(0, (f"tcgen05 splits={splits}", tcgen05))
        if cuda_cores:
            kernels.append(("CUDA cores", simt))
        for name, kernel in kernels:
            us = graph_time_us(lambda: kernel(q, kp, vp, table, tiles, out, page, None, scale), reps=4)
            print(f"attention_prefill {name} tokens={tokens} prior={prior} heads={n_heads}/{n_kv} head_dim={head_dim}: {us:.1f} us, "
                  f"{flops / us / 1e6:.0f} TFLOP/s (causal flops)", flush=True)


def bench_attention_decode(batches, contexts, n_heads, n_kv, head_dim, page, force_splits=0, shortest=0,
                           items_per_slot=0, cuda_cores=False) -> None:
    from ..parts import attention as attention_part
    from ..parts.attention import decode_splits

    for batch in batches:
        for context in contexts:
            pages_each = -(-context // page)
            n_pages = batch * pages_each
            pool_bytes = n_pages * 2 * n_kv * page * head_dim * 2
            copies = max(1, min(8, int(300e6 // pool_bytes)))  # rotate through more cache than the L2 holds
            pools = [(torch.randn(n_pages, 2, n_kv, page, head_dim, device="cuda") * 0.5).to(torch.bfloat16)
                     for _ in range(copies)]
            table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(batch, pages_each)
            q = torch.randn(batch, n_heads, head_dim, device="cuda").to(torch.bfloat16)
            out = torch.empty_like(q)
            # everyone at `context` keys, or lengths spread evenly from `shortest` up to it
            lengths = [context if not shortest else shortest + (context - shortest) * b // max(1, batch - 1)
                       for b in range(batch)]
            pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
            entry = torch.arange(batch, dtype=torch.int32, device="cuda")
            splits = force_splits or decode_splits(batch * n_kv, context, q.device, head_dim, n_heads // n_kv)
            scratch = torch.empty(max(1, ops.attention_decode_scratch_floats(batch, n_heads, head_dim, splits)),
                                  device="cuda")
            scale = 1 / math.sqrt(head_dim)
            turn = [0]

            if items_per_slot:  # the work list the engine makes for many or unequal requests
                ctas = attention_part.decode_item_ctas(q.device, head_dim, n_kv)
                host_items, host_slots = attention_part.decode_work_items(lengths, None, items_per_slot * ctas)
                items, slots = torch.from_numpy(host_items).cuda(), torch.from_numpy(host_slots).cuda()
                scratch = torch.empty(items.shape[0] * n_heads * (head_dim + 2), device="cuda")
                splits = f"work list of {int((host_items[:, 2] > 0).sum())} items"

            def run():
                pool = pools[turn[0] % copies]
                turn[0] += 1
                if items_per_slot:
                    ops.attention_decode_items(q, pool[:, 0], pool[:, 1], table, pos, entry, out, page, None, scale,
                                               items, slots, scratch)
                else:
                    ops.attention_decode(q, pool[:, 0], pool[:, 1], table, pos, entry, out, page, None, scale,
                                         splits, scratch)

            us = graph_time_us(run, reps=max(10, copies))
            gb = sum(lengths) * 2 * n_kv * head_dim * 2 / 1e9
            span = f"{shortest}..{context}" if shortest else f"{context}"
            other = ""
            if cuda_cores:  # the kernel that takes every shape, for comparison
                pool = pools[0]
                simt = graph_time_us(lambda: ops.attention_simt(q, pool[:, 0], pool[:, 1], table, pos, entry, out, page,
                                                                None, scale), reps=4)
                other = f"; CUDA-core kernel {simt:.1f} us"
            print(f"attention_decode batch={batch} context={span} heads={n_heads}/{n_kv} head_dim={head_dim} "
                  f"splits={splits}: {us:.1f} us, {gb / us * 1e6:.0f} GB/s{other}", flush=True)


LLAMA31_8B_SHAPE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 131072,
}


LLAMA32_1B_SHAPE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
LLAMA2_13B_SHAPE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 5120, "num_attention_heads": 40,
    "num_key_value_heads": 40, "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
MODEL_SHAPES = {"8b": LLAMA31_8B_SHAPE, "1b": LLAMA32_1B_SHAPE, "13b": LLAMA2_13B_SHAPE}


def decode_timeline(layers: int, batch: int, contexts: list[int], page: int, shape: str = "8b") -> None:
    import collections
    import re

    from torch.profiler import ProfilerActivity, profile

    from ..engine.engine import Engine
    from ..engine.runner import StepEntry
    from ..sampling.params import SamplingParams

    config = dict(MODEL_SHAPES[shape], num_hidden_layers=layers)
    # one context for everyone, or contexts spread evenly from the first to the second
    lo, hi = contexts[0], contexts[-1]
    lengths = [lo + (hi - lo) * b // max(1, batch - 1) for b in range(batch)]
    context = f"{lo}" if lo == hi else f"{lo}..{hi}"
    n_pages = sum(-(-(n + 256) // page) for n in lengths) + 64
    engine = Engine(config, dtype="bfloat16", device="cuda:0", n_pages=n_pages, page_size=page,
                    prefill_tokens_per_step=2048, max_requests=batch + 2, seed=0)
    for group in engine.cache.groups:
        group.tensor.normal_(0.0, 0.5)
    ids = []
    for b in range(batch):  # requests that hold `context` tokens, without running a prefill
        engine.cache.open(("timeline", b))
        engine.cache.reserve(("timeline", b), lengths[b])
        engine.cache.commit(("timeline", b), lengths[b])
        ids.append(("timeline", b))
    params = [SamplingParams()] * batch
    entries = [StepEntry(r, [(7 * i + 3) % 1000], [0]) for i, r in enumerate(ids)]

    def step():
        engine.runner.decode_step(entries, params, [0] * batch, [0] * batch)

    for _ in range(5):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    per_step = len(events) // 3
    last = [(e.name, e.time_range.start, e.time_range.end) for e in events[-per_step:]]

    def short(name: str) -> str:
        name = name.replace("void ", "").replace("(anonymous namespace)::", "")
        base = re.match(r"[\w:]+", name)
        args = re.search(r"<([^>]{0,40})", name)
        return (base.group(0) if base else name[:40]) + ("<" + args.group(1) + ">" if args else "")

    t0 = last[0][1]
    print(f"decode step ({shape} shape): batch {batch}, context {context}, {layers} layers: {per_step} device activities, "
          f"{last[-1][2] - t0:.1f} us from first start to last end")
    totals = collections.OrderedDict()
    for name, start, end in last:
        entry = totals.setdefault(short(name), [0, 0.0])
        entry[0] += 1
        entry[1] += end - start
    for name, (count, total) in totals.items():
        print(f"  {name:58s} x{count:3d}  resident {total / count:7.2f} us each")
    print("one layer from the middle of the step (us from the step's start; a kernel is resident from its start, "
          "its work begins when its predecessor ends):")
    middle = per_step // 2
    previous_end = None
    for name, start, end in last[middle: middle + 2 * max(1, (per_step - 4) // max(1, layers)) + 1]:
        after = "" if previous_end is None else f"  (+{end - previous_end:6.2f} after the previous end)"
        print(f"  start {start - t0:9.2f}  end {end - t0:9.2f}  {short(name)}{after}")
        previous_end = end


def mixed_steps(shape: str, layers: int, page: int, portion: int = 512, requests: int = 64) -> None:
    """Eager steps as a server under load runs them: `requests` prompts of 128 to 4,096 tokens
    fed in portions of `portion` tokens beside the single tokens of the requests already
    decoding. Prints the wall time of a step and the sum of its kernels' times (the torch
    profiler's CUDA activity trace): the difference is what the host costs."""
    import time

    from torch.profiler import ProfilerActivity, profile

    from ..engine.engine import Engine
    from ..sampling.params import SamplingParams

    config = dict(MODEL_SHAPES[shape], num_hidden_layers=layers)
    gen = torch.Generator().manual_seed(3)
    lengths = torch.randint(128, 4097, (requests,), generator=gen).tolist()
    prompts = [torch.randint(0, config["vocab_size"], (n,), generator=gen).tolist() for n in lengths]
    n_pages = sum(-(-(n + 80) // page) for n in lengths) + 64
    engine = Engine(config, dtype="bfloat16", device="cuda:0", n_pages=n_pages, page_size=page,
                    prefill_tokens_per_step=portion, max_requests=requests, seed=0)
    greedy = SamplingParams(temperature=0.0)

    def submit():
        return [engine.submit(p, sampling=greedy, max_tokens=64, ignore_eos=True) for p in prompts]

    submit()
    while engine.has_work():  # once through: libraries set up
        engine.step()
    engine.sync()
    submit()
    for _ in range(60):
        engine.step()
    torch.cuda.synchronize()
    steps = 40
    start = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - start) / steps
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    busy = sum(e.time_range.end - e.time_range.start for e in events) / steps
    print(f"mixed steps ({shape} shape, {layers} layers, portions of {portion} beside single tokens): "
          f"{wall * 1e3:.2f} ms a step by the clock, {busy / 1e3:.2f} ms of kernels ({len(events) // steps} launches)")
    while engine.has_work():
        engine.step()
    engine.sync()


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("what", choices=["gemm", "attention_prefill", "attention_decode", "decode_timeline",
                                         "mixed_steps"])
    parser.add_argument("--shapes", nargs="*", default=None, help="T,N,K triples for gemm")
    parser.add_argument("--tokens", type=int, nargs="*", default=[2048, 8192])
    parser.add_argument("--prior", type=int, default=0, help="keys in the cache before an attention_prefill portion")
    parser.add_argument("--splits", type=int, default=0, help="attention_prefill, attention_decode: split the keys this many ways "
                        "(default: as the engine would)")
    parser.add_argument("--batch", type=int, nargs="*", default=[1, 8, 64])
    parser.add_argument("--context", type=int, nargs="*", default=None)
    parser.add_argument("--shortest", type=int, default=0, help="attention_decode: the requests' lengths are spread "
                        "evenly from here up to --context (default: all at --context)")
    parser.add_argument("--items_per_slot", type=int, default=0, help="attention_decode: run the work-list form, "
                        "the keys cut into about this many items per resident CTA (the engine uses 4)")
    parser.add_argument("--cuda_cores", action="store_true", help="attention_decode, attention_prefill: also time "
                        "the CUDA-core kernel that takes every shape")
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv_heads", type=int, default=8)
    parser.add_argument("--head_dim", type=int, default=128)
    parser.add_argument("--page_size", type=int, default=16)
    parser.add_argument("--layers", type=int, default=8, help="layers of the decode_timeline model")
    parser.add_argument("--shape", default="8b", choices=sorted(MODEL_SHAPES),
                        help="decode_timeline: layer sizes of Llama-3.1-8B, Llama-3.2-1B or Llama-2-13B")
    args = parser.parse_args()
    ops.require_device()
    if args.items_per_slot and args.what == "decode_timeline":
        from ..parts import attention as attention_part

        attention_part.DECODE_ITEMS_PER_SLOT = args.items_per_slot
    if args.what == "gemm":
        shapes = LLAMA8B_SHAPES if not args.shapes else [tuple(int(v) for v in s.split(",")) for s in args.shapes]
        bench_gemm(shapes)
    elif args.what == "mixed_steps":
        mixed_steps(args.shape, args.layers, args.page_size)
    elif args.what == "decode_timeline":
        decode_timeline(args.layers, args.batch[0] if len(args.batch) == 1 else 8,
                        args.context if args.context and len(args.context) <= 2 else [2048], args.page_size,
                        args.shape)
    elif args.what == "attention_prefill":
        bench_attention_prefill(args.tokens, args.heads, args.kv_heads, args.head_dim, args.page_size, args.prior,
                                args.splits, args.cuda_cores)
    else:
        bench_attention_decode(args.batch, args.context or [2048, 4096], args.heads, args.kv_heads, args.head_dim,
                               args.page_size, args.splits, args.shortest, args.items_per_slot, args.cuda_cores)


if __name__ == "__main__":
    main()
