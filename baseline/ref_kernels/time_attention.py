"""Times the reference's prompt attention kernel (attn_prefill_cuda, bfloat16: its tensor-core
kernel, pulsarlm-core/inc/pulsarlm/kernels/paged_prefill.cuh) on this device at the shapes
this package's own kernels are measured at, so that profiles/ can hold a same-device column.

    python baseline/ref_kernels/build.py
    python baseline/ref_kernels/time_attention.py [--tokens 2048 8192] [--decode_batch 8 64 --context 2048 4096]

The reference stores keys unrotated and rotates them as it reads (that work is part of its
kernel's time, as it is part of its engine's). Its decode kernel (attn_decode_cuda) is in the
one file that does not build with this image's host compiler; the "single tokens" lines below
run its PROMPT kernel on portions of one token each, which is how its engine would run them if
it had no decode kernel, and are labelled so. CUDA events around graph replays, after warm-up.
"""

from __future__ import annotations

import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import build as ref_build  # noqa: E402


def graph_time_us(fn, reps: int = 4, iters: int = 10) -> float:
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


def eager_time_us(fn, iters: int = 20) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3


def case(ref, seq_lens_k: list[int], chunk: int, n_heads: int, n_kv: int, head_dim: int, page: int, rope):
    dev = "cuda"
    n_seqs = len(seq_lens_k)
    pages_each = [-(-n // page) for n in seq_lens_k]
    n_lines = sum(pages_each)
    k_pool = (torch.randn(n_lines, page, n_kv, head_dim, device=dev) * 0.5).to(torch.bfloat16)
    v_pool = (torch.randn(n_lines, page, n_kv, head_dim, device=dev) * 0.5).to(torch.bfloat16)
    width = max(pages_each)
    lines = torch.randperm(n_lines).to(torch.int32)
    tables = torch.zeros((n_seqs, width), dtype=torch.int32)
    positions = torch.zeros((n_seqs, width), dtype=torch.int32)
    at = 0
    for s, n in enumerate(pages_each):
        tables[s, :n] = lines[at:at + n]
        positions[s, :n] = torch.arange(n, dtype=torch.int32) * page
        at += n
    q = torch.randn(n_seqs * chunk, n_heads, head_dim, device=dev).to(torch.bfloat16)
    cu_q = torch.arange(0, (n_seqs + 1) * chunk, chunk, dtype=torch.int32, device=dev)
    lens = torch.tensor(seq_lens_k, dtype=torch.int32, device=dev)
    tables, positions = tables.to(dev), positions.to(dev)
    scale = 1.0 / math.sqrt(head_dim)

    def run():
        return ref.attn_prefill(q, k_pool, v_pool, tables, cu_q, lens, positions, *rope, scale, None, None, None,
                                None, None)

    try:
        return graph_time_us(run), "graph replay"
    except RuntimeError:
        torch.cuda.synchronize()
        return eager_time_us(run), "eager launches"


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--tokens", type=int, nargs="*", default=[2048, 8192])
    p.add_argument("--decode_batch", type=int, nargs="*", default=[8, 64])
    p.add_argument("--context", type=int, nargs="*", default=[2048, 4096])
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv_heads", type=int, default=8)
    p.add_argument("--head_dim", type=int, default=128)
    p.add_argument("--page_size", type=int, default=16)
    args = p.parse_args()
    ref = ref_build.load()
    rope = (500000.0, 1.0, [8.0, 1.0, 4.0, 8192.0])
    for tokens in args.tokens:
        us, how = case(ref, [tokens], tokens, args.heads, args.kv_heads, args.head_dim, args.page_size, rope)
        flops = 4.0 * args.heads * args.head_dim * tokens * (tokens + 1) / 2
        print(f"reference attn_prefill_cuda tokens={tokens} heads={args.heads}/{args.kv_heads} "
              f"head_dim={args.head_dim}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s (causal flops; {how})",
              flush=True)
    for batch in args.decode_batch:
        for context in args.context:
            us, how = case(ref, [context] * batch, 1, args.heads, args.kv_heads, args.head_dim, args.page_size, rope)
            gb = batch * context * 2 * args.kv_heads * args.head_dim * 2 / 1e9
            print(f"reference attn_prefill_cuda on single tokens batch={batch} context={context}: {us:.1f} us, "
                  f"{gb / us * 1e6:.0f} GB/s ({how})", flush=True)


if __name__ == "__main__":
    main()
