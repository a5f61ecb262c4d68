"""Runs the reference's own CUDA kernels on small fixed inputs and records their outputs.

    python baseline/ref_kernels/build.py                       # once: builds the extension
    python tests/golden/make_reference_kernel_golden.py OUT.json   # on a GPU

The kernels are cosmonomic/pulsarlm's, compiled unmodified from pulsarlm-core/src/kernels
(see baseline/ref_kernels/build.py for which files build here and which one does not):
rmsnorm_cuda (rmsnorm.cu:55), silu_mul_cuda (moe_routing.cu:170), rope_cuda (rope.cu:88),
attn_prefill_cuda in float32, which runs the scalar kernel (paged_common.cu:26-137) over
unrotated keys in paged pools, with and without a sliding window and with the attention
mass outputs, and gumbel_race_cuda at temperature 0 (gumbel_race.cu:17-21, ties).
tests/test_plain.py rebuilds the same inputs from `reference_kernel_inputs` below (plain
formulas of the element index, no random generator) and compares the plain implementation
with the recorded outputs, so that no formula of the plain implementation rests on
reading alone. The committed file was made on a B200 with this script.
"""

from __future__ import annotations

import base64
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def pack(t: torch.Tensor) -> str:
    """A float32 tensor's values as base64 of its little-endian bytes (exact, and a
    third of the size of decimal text)."""
    return base64.b64encode(t.detach().cpu().to(torch.float32).contiguous().numpy().astype("<f4").tobytes()).decode()


def unpack(text: str) -> torch.Tensor:
    return torch.from_numpy(np.frombuffer(base64.b64decode(text), dtype="<f4").copy())


def pattern(shape, a: float, b: float, scale: float = 1.0) -> torch.Tensor:
    """float32 tensor whose element i (row-major) is scale * sin(a * i + b), formed in float64."""
    n = int(math.prod(shape))
    i = torch.arange(n, dtype=torch.float64)
    return (scale * torch.sin(a * i + b)).to(torch.float32).reshape(shape)


ROPES = {
    "plain": {"theta": 10000.0, "llama3": None},
    "llama3": {"theta": 500000.0, "llama3": [8.0, 1.0, 4.0, 64.0]},
}

ATTENTION = {
    "n_heads": 4, "n_kv_heads": 2, "head_dim": 16, "page_size": 16, "scale_factor": 0.8,
    # (tokens the cache holds after the step, how many of them are this step's queries)
    "sequences": [(40, 40), (37, 7), (51, 1)],
    "decay": 0.25,
}


def reference_kernel_inputs() -> dict:
    """Every input of the recorded cases (float32 on the CPU)."""
    a = ATTENTION
    inputs = {
        "rmsnorm": [
            {"x": pattern((6, 96), 0.37, 0.1, 3.0), "w": 1.0 + pattern((96,), 0.91, 0.3, 0.1), "eps": 1e-5},
            {"x": pattern((3, 64), 0.53, 0.7, 0.05), "w": pattern((64,), 0.23, 1.1, 2.0), "eps": 1e-6},
        ],
        "silu_mul": {"x": pattern((5, 2 * 172), 0.61, 0.2, 4.0)},
        "rope": {"x": pattern((3, 7, 32), 0.41, 0.5), "positions": [0, 1, 5, 63, 64, 1000, 70000]},
        "attention": [],
        "argmax": {"scores": torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0], [3.0, 1.0, 3.0, 0.0, -2.0],
                                           [-4.0, -4.0, -5.0, -4.0, -6.0]], dtype=torch.float32)},
    }
    for s, (length, chunk) in enumerate(a["sequences"]):
        inputs["attention"].append({
            "q": pattern((length, a["n_heads"], a["head_dim"]), 0.173 + 0.01 * s, 0.2 * s, 1.5),
            "k": pattern((length, a["n_kv_heads"], a["head_dim"]), 0.291 + 0.01 * s, 0.4 + 0.3 * s, 1.5),
            "v": pattern((length, a["n_kv_heads"], a["head_dim"]), 0.117 + 0.01 * s, 0.9 + 0.1 * s, 1.0),
            "length": length, "chunk": chunk,
        })
    return inputs


def _rope_args(name: str):
    r = ROPES[name]
    return r["theta"], 1.0, r["llama3"]


def run_attention(ref, inputs, rope_name: str, window: int | None, with_mass: bool) -> dict:
    a = ATTENTION
    dev = "cuda"
    page, nkv, hd = a["page_size"], a["n_kv_heads"], a["head_dim"]
    seqs = inputs["attention"]
    pages_per = [-(-s["length"] // page) for s in seqs]
    n_lines = sum(pages_per) + 3
    # Lines handed out in a scattered order, so that a table error shows.
    order = [(7 * i + 3) % n_lines for i in range(n_lines)]
    assert len(set(order)) == n_lines
    k_pool = torch.zeros((n_lines, page, nkv, hd), dtype=torch.float32, device=dev)
    v_pool = torch.zeros_like(k_pool)
    max_pages = max(pages_per)
    tables = torch.zeros((len(seqs), max_pages), dtype=torch.int32)
    positions = torch.zeros((len(seqs), max_pages), dtype=torch.int32)
    next_line = 0
    q_rows, cu_q, lens_k = [], [0], []
    for s, seq in enumerate(seqs):
        for p in range(pages_per[s]):
            line = order[next_line]
            next_line += 1
            tables[s, p] = line
            positions[s, p] = p * page
            rows = slice(p * page, min((p + 1) * page, seq["length"]))
            n = rows.stop - rows.start
            k_pool[line, :n] = seq["k"][rows].to(dev)   # unrotated, as the reference stores keys
            v_pool[line, :n] = seq["v"][rows].to(dev)
        first = seq["length"] - seq["chunk"]
        q = seq["q"][first:].to(dev)                    # [chunk, nh, hd]
        pos = torch.arange(first, seq["length"], dtype=torch.int64, device=dev)
        # Queries arrive rotated to their own positions: by the reference's own rope_cuda ([heads, seq, hd]).
        q_rot = ref.rope(q.transpose(0, 1).contiguous(), pos, *_rope_args(rope_name)).transpose(0, 1).contiguous()
        q_rows.append(q_rot)
        cu_q.append(cu_q[-1] + seq["chunk"])
        lens_k.append(seq["length"])
    q_all = torch.cat(q_rows, dim=0)
    scale = a["scale_factor"] / math.sqrt(hd)
    mass = weight = cu_pages = qw = None
    if with_mass:
        cu = [0]
        for n in pages_per:
            cu.append(cu[-1] + n)
        cu_pages = torch.tensor(cu, dtype=torch.int32, device=dev)
        mass = torch.zeros((cu[-1], a["n_heads"]), dtype=torch.float32, device=dev)
        weight = torch.zeros((cu[-1],), dtype=torch.float32, device=dev)
        w = []
        for seq in seqs:
            w += [a["decay"] * (1.0 - a["decay"]) ** age for age in range(seq["chunk"] - 1, -1, -1)]
        qw = torch.tensor(w, dtype=torch.float32, device=dev)
    out = ref.attn_prefill(q_all, k_pool, v_pool, tables.to(dev), torch.tensor(cu_q, dtype=torch.int32, device=dev),
                           torch.tensor(lens_k, dtype=torch.int32, device=dev), positions.to(dev),
                           *_rope_args(rope_name), scale, window, mass, weight, cu_pages, qw)
    torch.cuda.synchronize()
    record = {"rope": rope_name, "window": window, "out": pack(out)}
    if with_mass:
        record["mass_sum"] = pack(mass)
        record["weight_sum"] = pack(weight)
        record["pages_per_sequence"] = pages_per
    return record


def main() -> None:
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_kernels.json")
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "baseline", "ref_kernels"))
    import build as ref_build

    ref = ref_build.load()
    inputs = reference_kernel_inputs()
    dev = "cuda"
    golden: dict = {"made_with": "cosmonomic/pulsarlm pulsarlm-core/src/kernels, unmodified, on " +
                    torch.cuda.get_device_name(0)}
    golden["rmsnorm"] = [pack(ref.rmsnorm(c["x"].to(dev), c["w"].to(dev), c["eps"])) for c in inputs["rmsnorm"]]
    golden["silu_mul"] = pack(ref.silu_mul(inputs["silu_mul"]["x"].to(dev)))
    pos = torch.tensor(inputs["rope"]["positions"], dtype=torch.int64, device=dev)
    golden["rope"] = {name: pack(ref.rope(inputs["rope"]["x"].to(dev), pos, *_rope_args(name))) for name in ROPES}
    golden["attention"] = [
        run_attention(ref, inputs, "plain", None, True),
        run_attention(ref, inputs, "llama3", None, False),
        run_attention(ref, inputs, "llama3", 8, False),
    ]
    scores = inputs["argmax"]["scores"].to(dev)
    draws = torch.zeros((2, scores.shape[0]), dtype=torch.int64, device=dev)
    golden["argmax"] = ref.gumbel_race(scores, torch.zeros(scores.shape[0], device=dev), draws).cpu().tolist()
    with open(out_path, "w") as f:
        json.dump(golden, f)
    print(f"wrote {out_path} ({os.path.getsize(out_path)} bytes)")


if __name__ == "__main__":
    main()
