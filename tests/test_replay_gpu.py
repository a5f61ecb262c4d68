"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back
from files and compared with the plain implementation."""

import json
import os
import random
import subprocess

import numpy as np
import pytest
import torch

import plain_llama
import tiny
from harness import TOLERANCE, TinyModel
from test_model_gpu import mixed_schedule

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_trace(tm, steps, out_dir, max_tokens, dtype):
    lines = []
    for i, (entries, ends) in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": r, "tokens": list(t), "want": list(w)}
                                                         for r, t, w in entries], "end": list(ends)}))
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", tm.folder, "--dtype", dtype, "--out",
                           str(out_dir), "--max-tokens", str(max_tokens)], input="\n".join(lines) + "\n",
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[: len(steps)] == [f"done {i}" for i in range(len(steps))]
    vocab = tm.cfg["vocab_size"]
    got, fed = {}, {}
    for i, (entries, ends) in enumerate(steps):
        wanted = sum(len(list(w)) for _, _, w in entries)
        path = os.path.join(out_dir, f"{i}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            for r, t, w in entries:
                fed[r] = fed.get(r, 0) + len(t)
            continue
        data = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        row = 0
        for r, t, w in entries:
            for place in w:
                got.setdefault(r, {})[fed.get(r, 0) + place] = torch.from_numpy(data[row].copy())
                row += 1
            fed[r] = fed.get(r, 0) + len(t)
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_mixed_requests_with_page_reuse(tmp_path, dtype):
    tm = TinyModel("B", dtype)
    lengths = [40, 97, 64, 33, 120, 18, 75]
    reqs = {f"r{n}": tiny.random_tokens(tm.cfg, n, seed=n) for n in lengths}
    steps = mixed_schedule(reqs, random.Random(5))
    # the most tokens live at once, each request rounded up to a multiple of 64
    live, peak = {}, 0
    for entries, ends in steps:
        for r, t, _ in entries:
            live[r] = live.get(r, 0) + len(t)
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values()))
        for r in ends:
            del live[r]
    got = run_trace(tm, steps, tmp_path, peak, dtype)
    for r, rows in got.items():
        ref = tm.plain_logits(reqs[r])
        positions = sorted(rows)
        err = plain_llama.max_relative_error(torch.stack([rows[p] for p in positions]), ref[positions])
        assert err < TOLERANCE[dtype], (r, err)


def test_trace_run_whole_then_tail_one_by_one(tmp_path):
    tm = TinyModel("A", "float32")
    tokens = tiny.random_tokens(tm.cfg, 80, seed=4)
    steps = [([("a", tokens[:48], [0, 47])], [])]
    steps += [([("a", tokens[i:i + 1], [0])], ["a"] if i == 79 else []) for i in range(48, 80)]
    got = run_trace(tm, steps, tmp_path, 128, "float32")["a"]
    ref = tm.plain_logits(tokens)
    for p, row in got.items():
        assert plain_llama.max_relative_error(row, ref[p]) < 1e-4, p
    assert sorted(got) == [0] + list(range(47, 80))
