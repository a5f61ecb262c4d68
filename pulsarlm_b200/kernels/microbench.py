"""Device timings of single kernels at given sizes.

    python -m pulsarlm_b200.kernels.microbench gemm [--shapes T,N,K ...]
    python -m pulsarlm_b200.kernels.microbench attention_prefill [--tokens 2048 ...]
    python -m pulsarlm_b200.kernels.microbench attention_decode [--batch 8 --context 2048 ...]

Each timing replays a CUDA graph of several launches (so host time does not
count) over inputs rotated through enough copies to exceed L2, after warm-up,
between CUDA events. Prints one line per case with achieved GB/s and TFLOP/s.
`gemm` times the tcgen05 kernel beside the library product torch.mm calls.
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

        def own():
            ops.gemm_bf16(x, weights[turn[0] % copies], out)
            turn[0] += 1

        def library():
            torch.mm(x, weights[turn[0] % copies].t(), out=out)
            turn[0] += 1

        gb, tf = n * k * 2 / 1e9, 2.0 * t * n * k / 1e12
        a, b = graph_time_us(own), graph_time_us(library)
        print(f"gemm t={t} n={n} k={k}: tcgen05 {a:.1f} us ({gb / a * 1e6:.0f} GB/s, {tf / a * 1e6:.0f} TFLOP/s)"
              f" | library {b:.1f} us ({gb / b * 1e6:.0f} GB/s, {tf / b * 1e6:.0f} TFLOP/s)", flush=True)


def bench_attention_prefill(tokens_list, n_heads, n_kv, head_dim, page) -> None:
    for tokens in tokens_list:
        n_pages = tokens // page + 4
        pool = (torch.randn(n_pages, 2, n_kv, page, head_dim, device="cuda") * 0.5).to(torch.bfloat16)
        kp, vp = pool[:, 0], pool[:, 1]
        table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(1, -1)
        qkv = torch.randn(tokens, (n_heads + 2 * n_kv) * head_dim, device="cuda").to(torch.bfloat16)
        q = qkv[:, : n_heads * head_dim].view(tokens, n_heads, head_dim)
        out = torch.empty(tokens, n_heads, head_dim, device="cuda", dtype=torch.bfloat16)
        rows = ops.attention_prefill_tile_rows()
        tiles = sorted(((r, min(rows, tokens - r), r, 0) for r in range(0, tokens, rows)), key=lambda t: -(t[1] + t[2]))
        tiles = torch.tensor(tiles, dtype=torch.int32, device="cuda")
        scale = 1 / math.sqrt(head_dim)
        flops = 4.0 * n_heads * head_dim * tokens * (tokens + 1) / 2
        for name, kernel in (("tcgen05", ops.attention_prefill_tcgen05), ("mma.sync", ops.attention_prefill)):
            us = graph_time_us(lambda: kernel(q, kp, vp, table, tiles, out, page, None, scale), reps=4)
            print(f"attention_prefill {name} tokens={tokens} heads={n_heads}/{n_kv} head_dim={head_dim}: {us:.1f} us, "
                  f"{flops / us / 1e6:.0f} TFLOP/s (causal flops)", flush=True)


def bench_attention_decode(batches, contexts, n_heads, n_kv, head_dim, page) -> None:
    from ..parts.attention import decode_splits

    for batch in batches:
        for context in contexts:
            pages_each = -(-context // page)
            n_pages = batch * pages_each
            pool = (torch.randn(n_pages, 2, n_kv, page, head_dim, device="cuda") * 0.5).to(torch.bfloat16)
            kp, vp = pool[:, 0], pool[:, 1]
            table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(batch, pages_each)
            q = torch.randn(batch, n_heads, head_dim, device="cuda").to(torch.bfloat16)
            out = torch.empty_like(q)
            pos = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
            entry = torch.arange(batch, dtype=torch.int32, device="cuda")
            splits = decode_splits(batch * n_kv, context, q.device)
            scratch = torch.empty(max(1, ops.attention_decode_scratch_floats(batch, n_heads, head_dim, splits)),
                                  device="cuda")
            scale = 1 / math.sqrt(head_dim)
            us = graph_time_us(lambda: ops.attention_decode(q, kp, vp, table, pos, entry, out, page, None, scale,
                                                            splits, scratch))
            gb = batch * context * 2 * n_kv * head_dim * 2 / 1e9
            print(f"attention_decode batch={batch} context={context} heads={n_heads}/{n_kv} head_dim={head_dim} "
                  f"splits={splits}: {us:.1f} us, {gb / us * 1e6:.0f} GB/s", flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("what", choices=["gemm", "attention_prefill", "attention_decode"])
    parser.add_argument("--shapes", nargs="*", default=None, help="T,N,K triples for gemm")
    parser.add_argument("--tokens", type=int, nargs="*", default=[2048, 8192])
    parser.add_argument("--batch", type=int, nargs="*", default=[1, 8, 64])
    parser.add_argument("--context", type=int, nargs="*", default=[2048, 4096])
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv_heads", type=int, default=8)
    parser.add_argument("--head_dim", type=int, default=128)
    parser.add_argument("--page_size", type=int, default=16)
    args = parser.parse_args()
    ops.require_device()
    if args.what == "gemm":
        shapes = LLAMA8B_SHAPES if not args.shapes else [tuple(int(v) for v in s.split(",")) for s in args.shapes]
        bench_gemm(shapes)
    elif args.what == "attention_prefill":
        bench_attention_prefill(args.tokens, args.heads, args.kv_heads, args.head_dim, args.page_size)
    else:
        bench_attention_decode(args.batch, args.context, args.heads, args.kv_heads, args.head_dim, args.page_size)


if __name__ == "__main__":
    main()
