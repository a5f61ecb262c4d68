"""The entry point for callers that cannot allocate device memory
(pulsarlm_b200/csrc/no_alloc.h): split-key decode attention whose scratch is an
array built into the library.

Some users of the kernels run where cudaMalloc and torch's allocator are off
limits: inside another framework's callback, or in a process that gave all its
device memory away at start-up. They can still pass inputs and outputs they
already own. This test stands in for such a caller: it reaches the exported C
symbol through ctypes with raw pointers, twice in a row (the second call finds
the first call's leftovers in the shared array), and checks the result against
the ordinary entry point given scratch of its own and against a dense float64
attention; that the driver's count of free device memory does not move across a
call; a split count above what a thread-block cluster merges; and a call that
fills the built-in array almost to its end. The file sorts last so that a
run that stops at the first failure has already run every other test; it also
passes when it is the only test in a fresh process.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_case(seed, lengths, nh=8, nkv=2, hd=128, page=16):
    g = torch.Generator().manual_seed(seed)
    pages_each = -(-max(lengths) // page)
    n_pages = len(lengths) * pages_each + 2
    table = torch.randperm(n_pages, generator=g)[: len(lengths) * pages_each].view(len(lengths), pages_each)
    pool = torch.randn(n_pages, 2, nkv, page, hd, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(len(lengths), nh, hd, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    entry = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
    return q, pool[:, 0], pool[:, 1], table.to(torch.int32).to(DEV), pos, entry, page


def call_static(lib, q, kp, vp, table, pos, entry, out, page, splits, status):
    fn = lib.pl_attention_decode_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    tokens, nh, hd = q.shape
    return fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vp.data_ptr(), kp.stride(0), kp.stride(1), page,
              kp.shape[0], table.data_ptr(), table.shape[1], pos.data_ptr(), entry.data_ptr(), out.data_ptr(),
              out.stride(0), tokens, nh, kp.shape[1], hd, 0, 1.0 / math.sqrt(hd), splits, status.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


def dense_attention(q, kp, vp, table, pos, entry, page):
    """Softmax attention of each query over its request's keys 0..pos, float64 on the CPU."""
    out = torch.empty(q.shape, dtype=torch.float64)
    qd, kd, vd = q.double().cpu(), kp.double().cpu(), vp.double().cpu()
    group = q.shape[1] // kp.shape[1]
    scale = 1.0 / math.sqrt(q.shape[2])
    for t in range(q.shape[0]):
        n = int(pos[t]) + 1
        row = table[int(entry[t])].tolist()
        pages = -(-n // page)
        keys = torch.cat([kd[row[j]] for j in range(pages)], dim=1)[:, :n]  # [nkv, n, hd]
        vals = torch.cat([vd[row[j]] for j in range(pages)], dim=1)[:, :n]
        for h in range(q.shape[1]):
            s = (keys[h // group] @ qd[t, h]) * scale
            out[t, h] = torch.softmax(s, 0) @ vals[h // group]
    return out


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from pulsarlm_b200.kernels import ops

    ops.require_device()
    lib = ops.library()
    lib.pl_static_scratch_floats.restype = ctypes.c_int64
    assert lib.pl_static_scratch_floats() == 4 * 1024 * 1024
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # different calls back to back: other lengths, other split counts, so a call
    # reads nothing an earlier one left behind unless the kernel is wrong. The third
    # splits 24 ways (more than a cluster merges); the fourth needs 4,193,280 of the
    # array's 4,194,304 floats.
    cases = ((1, [700, 33, 250, 1], 5, 8, 2), (2, [90, 1200], 3, 8, 2), (3, [3000, 450], 24, 8, 2),
             (4, [300 + 7 * i for i in range(42)], 24, 32, 8))
    for seed, lengths, splits, nh, nkv in cases:
        q, kp, vp, table, pos, entry, page = make_case(seed, lengths, nh=nh, nkv=nkv)
        needed = ops.attention_decode_scratch_floats(q.shape[0], q.shape[1], q.shape[2], splits)
        assert needed <= 4 * 1024 * 1024 and (seed != 4 or needed > 4 * 1024 * 1024 - 2048)
        want = torch.empty_like(q)
        scratch = torch.empty(ops.attention_decode_scratch_floats(q.shape[0], q.shape[1], q.shape[2], splits),
                              device=DEV)
        ops.attention_decode(q, kp, vp, table, pos, entry, want, page, None, 1.0 / math.sqrt(q.shape[2]), splits,
                             scratch, status)
        got = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        code = call_static(lib, q, kp, vp, table, pos, entry, got, page, splits, status)
        torch.cuda.synchronize()
        assert code == 0, lib.pl_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        assert int(status) == 0
        # Once more with the driver's own count of free memory around the call: it sees any
        # cudaMalloc, not only torch's. (Measured on a repeated call: the first launch of a
        # kernel may make the driver load its code, which is not an allocation of the call's.)
        again = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert call_static(lib, q, kp, vp, table, pos, entry, again, page, splits, status) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(again, got)
        # same kernel, same split boundaries: the two agree to the bit, which is
        # well inside the 1e-2 bar the other bfloat16 attention tests use
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < 1e-2 and torch.equal(got, want)
        # and against the dense attention, at the bar of the other bfloat16 attention tests
        dense = dense_attention(q, kp, vp, table.cpu(), pos.cpu(), entry.cpu(), page)
        assert float((got.double().cpu() - dense).abs().max() / dense.abs().max()) < 1e-2


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from pulsarlm_b200.kernels import ops

    ops.require_device()
    lib = ops.library()
    q, kp, vp, table, pos, entry, page = make_case(3, [64] * 40, nh=32, nkv=8)
    out = torch.full_like(q, 7.0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # 40 tokens x 32 heads x 30 splits x 130 floats is more than the array holds
    code = call_static(lib, q, kp, vp, table, pos, entry, out, page, 30, status)
    torch.cuda.synchronize()
    assert code != 0 and b"fewer splits" in lib.pl_last_error()
    assert bool((out == 7.0).all())  # nothing was launched
