"""Each CUDA kernel alone against a plain torch reference, at sizes other than the
engine's tests use: widths and vocabularies that are no power of two, head sizes
in steps of 16, any number of heads and groups, scattered pages. Where random
inputs would hide a fault (one far key among hundreds, a window's edge, a page's
edge) the inputs are built so that it shows."""

import math

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def ops():
    from pulsarlm_b200.kernels import ops as module

    module.require_device()
    return module


def rel(got, want):
    return float((got.double().cpu() - want.double().cpu()).abs().max() / want.double().abs().max().clamp_min(1e-30))


# ----------------------------------------------------------------------------- elementwise

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,vocab", [(100, 77), (4097, 513)])
def test_embed(ops, dtype, hidden, vocab):
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    tokens = torch.randint(0, vocab, (37,), device=DEV, dtype=torch.int32)
    out = torch.empty(37, hidden, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed(table, tokens, out, status)
    assert torch.equal(out, table[tokens.long()].float()) and int(status) == 0
    tokens[5] = vocab
    ops.embed(table, tokens, out, status)
    assert int(status) == 1 and bool((out[5] == 0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [64, 100, 4097])
@pytest.mark.parametrize("weight_dtype", ["same", "float32"])
def test_add_rmsnorm(ops, dtype, hidden, weight_dtype):
    eps = 1e-5
    x = torch.randn(19, hidden, device=DEV) * 3
    x[4] = 0  # an all-zero row must give zeros, not NaN
    delta = torch.randn(19, hidden, device=DEV).to(dtype)
    delta[4] = 0
    w = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype if weight_dtype == "same" else torch.float32)
    want_x = x + delta.float()
    want = plain_llama.rms_norm(want_x.double(), w.double(), eps)
    x1 = x.clone()
    out = torch.empty(19, hidden, device=DEV, dtype=dtype)
    ops.add_rmsnorm(x1, delta, w, eps, out)
    assert torch.equal(x1, want_x)  # the residual sum is exact fp32
    assert rel(out, want) < TOL[dtype] and bool(torch.isfinite(out.float()).all())
    # no delta: x untouched
    x2 = x.clone()
    ops.add_rmsnorm(x2, None, w, eps, out)
    assert torch.equal(x2, x) and rel(out, plain_llama.rms_norm(x.double(), w.double(), eps)) < TOL[dtype]
    # selected rows: x untouched, rows gathered
    rows = torch.tensor([18, 0, 7], device=DEV, dtype=torch.int32)
    x3 = x.clone()
    picked = torch.empty(3, hidden, device=DEV, dtype=dtype)
    ops.add_rmsnorm(x3, delta, w, eps, picked, rows)
    assert torch.equal(x3, x) and rel(picked, want[rows.long()]) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [172, 1000])
def test_swiglu(ops, dtype, width):
    gate_up = (torch.randn(23, 2 * width, device=DEV) * 4).to(dtype)
    out = torch.empty(23, width, device=DEV, dtype=dtype)
    ops.swiglu(gate_up, out)
    g, u = gate_up[:, :width].double(), gate_up[:, width:].double()
    assert rel(out, g * torch.sigmoid(g) * u) < TOL[dtype]


@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (3, 100, 172), (65, 130, 257), (200, 64, 64)])
def test_gemm_f32_and_its_row_independence(ops, m, n, k):
    a = torch.randn(m, k, device=DEV)
    w = torch.randn(n, k, device=DEV)
    out = torch.empty(m, n, device=DEV)
    ops.gemm_f32(a, w, out)
    assert rel(out, a.double() @ w.double().T) < 1e-5
    one = torch.empty(1, n, device=DEV)
    ops.gemm_f32(a[m // 2 : m // 2 + 1].contiguous(), w, one)
    assert torch.equal(one[0], out[m // 2])  # a row's bits do not depend on the batch
    acc = out.clone()
    ops.gemm_f32(a, w, acc, accumulate=True)
    assert torch.allclose(acc, 2 * out)


def test_gemm_f32_is_true_fp32(ops):
    # 1 + 2^-12 squared needs 24 bits of product mantissa: a tf32 or bf16 product
    # would round the inputs to 1.
    a = torch.full((4, 8), 1 + 2 ** -12, device=DEV)
    w = torch.full((4, 8), 1 + 2 ** -12, device=DEV)
    out = torch.empty(4, 4, device=DEV)
    ops.gemm_f32(a, w, out)
    assert abs(float(out[0, 0]) - 8 * (1 + 2 ** -12) ** 2) < 1e-5
    assert abs(float(out[0, 0]) - 8.0) > 3e-3


GEMM_SHAPES = [(1, 128, 64), (8, 256, 128), (3, 100, 96), (37, 1000, 96), (300, 515, 160), (64, 512, 1024),
               (130, 384, 512), (8, 4096, 4096), (17, 6144, 1024), (600, 1536, 2048), (2048, 1024, 512),
               (5, 128, 520), (3, 130, 4096), (8, 512, 14336), (64, 3584, 512), (33, 200, 64), (16, 28672, 256)]


@pytest.mark.parametrize("t,n,k,kernel", [(t, n, k, kernel) for (t, n, k) in GEMM_SHAPES
                                          for kernel in (("skinny", "pair") if t <= 64 else ("pair",))])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_tcgen05(ops, t, n, k, kernel, out_dtype):
    """The tensor-core products at token counts from one to thousands and widths that
    are no multiple of the tile: the skinny kernel (k ranges shared between the CTAs
    of a cluster, with more ranks than tokens and ranks with a shorter k range among
    the cases) and the kernel that runs a tile on a pair of SMs."""
    x = torch.randn(t, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / k ** 0.5).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert ops.gemm_bf16_supports(t, n, k, k, k)
    outs = []
    for _ in range(2):  # twice: the bits must be the same
        out = torch.full((t, n), float("nan"), device=DEV, dtype=out_dtype)
        ops.gemm_bf16(x, w, out, status, kernel=kernel)
        outs.append(out)
    want = x.double() @ w.double().T
    assert int(status) == 0
    # fp32 results carry the rounding of one fp32 accumulator over k terms, which grows
    # with sqrt(k) (the kernels that cut k among CTAs add shorter partial sums): four
    # standard deviations of that, and no less than 1e-5.
    fp32_bar = max(1e-5, 4 * k ** 0.5 * 2.0 ** -24)
    assert rel(outs[0], want) < (fp32_bar if out_dtype == torch.float32 else 1e-2)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("t,n,k", [(1, 64, 64), (8, 172, 64), (300, 336, 160), (600, 1000, 520), (2048, 1792, 256),
                                   (257, 96, 4096)])
def test_gemm_bf16_gated_epilogue(ops, t, n, k):
    """silu(x gate^T) * (x up^T) from the pair kernel's epilogue: against the two
    products rounded to bfloat16 and the activation in fp64, and bit for bit against
    the plain product followed by the SwiGLU kernel; widths that are no multiple of
    the 64-feature half tile, token counts that are no multiple of the tile."""
    x = torch.randn(t, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * n, k, device=DEV) / k ** 0.5 * 2).to(torch.bfloat16)
    out = torch.full((t, n), float("nan"), device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.gemm_bf16(x, w, out, status, kernel="pair", gated=True)
    both = (x.double() @ w.double().T).to(torch.bfloat16).double()
    gate, up = both[:, :n], both[:, n:]
    want = gate / (1 + torch.exp(-gate)) * up
    assert int(status) == 0
    assert rel(out, want) < 1e-2
    plain = torch.empty(t, 2 * n, device=DEV, dtype=torch.bfloat16)
    ops.gemm_bf16(x, w, plain, kernel="pair")
    two_step = torch.empty_like(out)
    ops.swiglu(plain, two_step)
    assert torch.equal(out, two_step)


@pytest.mark.parametrize("t,n,k", [(1, 64, 64), (8, 4096, 14336), (16, 172, 1000), (5, 2048, 8192), (13, 130, 72),
                                   (8, 5120, 13824)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_bf16_with_the_gated_activation_made_on_the_way_in(ops, t, n, k, out_dtype):
    """y = (silu(g) * u) w^T with the activation formed inside the product against the
    SwiGLU kernel followed by the plain product: the same bits (same expression, same
    rounding, same order of additions), and both close to float64."""
    gate_up = (torch.randn(t, 2 * k, device=DEV) * 1.5).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(torch.bfloat16)
    act = torch.empty(t, k, device=DEV, dtype=torch.bfloat16)
    ops.swiglu(gate_up, act)
    two = torch.empty(t, n, device=DEV, dtype=out_dtype)
    ops.gemm_bf16(act, w, two, kernel="skinny")
    one = torch.full((t, n), float("nan"), device=DEV, dtype=out_dtype)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.gemm_bf16_gated_in(gate_up, w, one, status)
    assert int(status) == 0 and torch.equal(one, two)
    g, u = gate_up[:, :k].double().cpu(), gate_up[:, k:].double().cpu()
    want = (torch.nn.functional.silu(g) * u).to(torch.bfloat16).double() @ w.double().cpu().t()
    assert rel(one, want) < (1e-2 if out_dtype == torch.bfloat16 else 2e-3)
    # rows of a wider buffer (a slice of a larger activation)
    wide = torch.zeros(t, 2 * k + 16, device=DEV, dtype=torch.bfloat16)
    wide[:, : 2 * k] = gate_up
    again = torch.empty_like(one)
    ops.gemm_bf16_gated_in(wide[:, : 2 * k], w, again, status)
    assert int(status) == 0 and torch.equal(again, one)


def test_gemm_bf16_finds_one_large_product_among_many(ops):
    """One x[t, k] * w[n, k] pair far larger than the rest, at the last k of a k
    block, the first of the next, and in the tail: a dropped k block or a mis-stepped
    descriptor loses it."""
    t, n, k = 5, 200, 1000
    for hot_k in (63, 64, 511, 959, 960, 999):
        x = torch.zeros(t, k, device=DEV, dtype=torch.bfloat16)
        w = torch.zeros(n, k, device=DEV, dtype=torch.bfloat16)
        x[3, hot_k] = 3.0
        w[150, hot_k] = 2.0
        for kernel in ("skinny", "pair"):
            out = torch.empty(t, n, device=DEV, dtype=torch.float32)
            ops.gemm_bf16(x, w, out, kernel=kernel)
            want = torch.zeros(t, n)
            want[3, 150] = 6.0
            assert torch.equal(out.cpu(), want), (hot_k, kernel)


def test_gemm_bf16_refuses_rows_that_do_not_start_on_16_bytes(ops):
    assert not ops.gemm_bf16_supports(4, 64, 172, 172, 172)
    x = torch.randn(4, 172, device=DEV).to(torch.bfloat16)
    w = torch.randn(64, 172, device=DEV).to(torch.bfloat16)
    with pytest.raises(ops.KernelError) as error:
        ops.gemm_bf16(x, w, torch.empty(4, 64, device=DEV, dtype=torch.bfloat16))
    assert "multiples of 8" in str(error.value)


# ----------------------------------------------------------------------------- cache helpers

def make_pools(n_pages, n_kv, page, hd, dtype, fill=None):
    pool = torch.zeros(n_pages, 2, n_kv, page, hd, device=DEV, dtype=dtype)
    if fill is not None:
        pool.normal_(0, fill)
    return pool[:, 0], pool[:, 1]


def dense_from_pool(pool, table_row, length, page):
    """[length, n_kv, hd] gathered through a block-table row."""
    rows = []
    for j in range(length):
        rows.append(pool[table_row[j // page], :, j % page, :])
    return torch.stack(rows)


def scattered_tables(n_requests, pages_each, n_pages, seed=0):
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g)[: n_requests * pages_each]
    return perm.view(n_requests, pages_each).to(torch.int32)


# ----------------------------------------------------------------------------- rope + kv write

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rotary,page", [(4, 4, 16, 16, 16), (6, 2, 48, 48, 32), (5, 1, 80, 40, 8),
                                                   (8, 2, 128, 128, 16)])
def test_rope_kv_write(ops, dtype, nh, nkv, hd, rotary, page):
    tokens = 29
    llama3 = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}
    inv_freq = plain_llama.rope_inverse_frequency(500000.0, hd, llama3)[: rotary // 2]
    if rotary != hd:
        inv_freq = plain_llama.rope_inverse_frequency(10000.0, rotary, None)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(tokens, width, device=DEV).to(dtype)
    q = qkv[:, : nh * hd].view(tokens, nh, hd)
    k = qkv[:, nh * hd : (nh + nkv) * hd].view(tokens, nkv, hd)
    v = qkv[:, (nh + nkv) * hd :].view(tokens, nkv, hd)
    q0, k0, v0 = q.clone(), k.clone(), v.clone()
    # two requests: 11 tokens from position 100 (crossing pages), 18 from position 131000
    starts, counts = [100, 131000], [11, 18]
    pos = torch.cat([torch.arange(s, s + c) for s, c in zip(starts, counts)]).to(torch.int32).to(DEV)
    entry = torch.cat([torch.full((c,), i) for i, c in enumerate(counts)]).to(torch.int32).to(DEV)
    pages_each = (131000 + 18) // page + 1
    table = torch.full((2, pages_each), -1, dtype=torch.int32)
    used = iter(torch.randperm(40, generator=torch.Generator().manual_seed(1)).tolist())
    for i, (s, c) in enumerate(zip(starts, counts)):
        for pg in range(s // page, (s + c - 1) // page + 1):
            table[i, pg] = next(used)
    kp, vp = make_pools(40, nkv, page, hd, dtype)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_kv_write(q, k, v, pos, entry, table.to(DEV), kp, vp, page, inv_freq.to(DEV), rotary, status)
    assert int(status) == 0

    def rotate(x):
        x = x.double().cpu()
        rot = plain_llama.rope_rotate(x[..., :rotary], pos.cpu().long(), inv_freq)
        return torch.cat([rot, x[..., rotary:]], dim=-1)

    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert rel(q, rotate(q0)) < tol
    want_k = rotate(k0)
    for t in range(tokens):
        p = int(pos[t])
        page_id = int(table[int(entry[t]), p // page])
        assert rel(kp[page_id, :, p % page, :], want_k[t]) < tol, t
        assert torch.equal(vp[page_id, :, p % page, :], v0[t]), t
    if rotary < hd:  # dims past the rotary width pass through bit for bit
        assert torch.equal(q[..., rotary:], q0[..., rotary:])
    # nothing else was written
    written = torch.zeros(40, page, dtype=torch.bool)
    for t in range(tokens):
        written[int(table[int(entry[t]), int(pos[t]) // page]), int(pos[t]) % page] = True
    assert bool((kp.float().abs().sum(dim=(1, 3)).cpu()[~written] == 0).all())


def test_rope_kv_write_flags_a_missing_page(ops):
    q = torch.randn(2, 2, 16, device=DEV)
    k, v = torch.randn(2, 2, 16, device=DEV), torch.randn(2, 2, 16, device=DEV)
    qkv = torch.cat([q, k, v], dim=1).contiguous()
    kp, vp = make_pools(4, 2, 16, 16, torch.float32)
    table = torch.tensor([[0, -1]], dtype=torch.int32, device=DEV)
    pos = torch.tensor([3, 16], dtype=torch.int32, device=DEV)
    entry = torch.zeros(2, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rope_kv_write(qkv[:, 0:2], qkv[:, 2:4], qkv[:, 4:6], pos, entry, table, kp, vp, 16, None, 0, status)
    assert int(status) == 2


# ----------------------------------------------------------------------------- attention

def reference_attention(q, kp, vp, table, pos, entry, page, window, scale):
    """Plain attention of each query over its request's keys 0..pos (dense gather)."""
    out = torch.empty(q.shape, dtype=torch.float64)
    qd, kd, vd = q.double().cpu(), kp.double().cpu(), vp.double().cpu()
    group = q.shape[1] // kp.shape[1]
    for t in range(q.shape[0]):
        p = int(pos[t])
        first = max(0, p - window + 1) if window else 0
        row = table[int(entry[t])].tolist()
        keys = torch.stack([kd[row[j // page], :, j % page, :] for j in range(first, p + 1)])  # [n, nkv, hd]
        vals = torch.stack([vd[row[j // page], :, j % page, :] for j in range(first, p + 1)])
        for h in range(q.shape[1]):
            s = (keys[:, h // group, :] @ qd[t, h]) * scale
            out[t, h] = torch.softmax(s, 0) @ vals[:, h // group, :]
    return out


ATTENTION_SHAPES = [
    # nh, nkv, hd, page
    (4, 4, 16, 16),
    (6, 2, 32, 32),
    (3, 1, 48, 8),
    (8, 2, 64, 16),
    (5, 5, 80, 16),
    (8, 1, 128, 16),
    (4, 2, 256, 32),
    (14, 2, 128, 64),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page", ATTENTION_SHAPES)
@pytest.mark.parametrize("window", [None, 21])
def test_attention_simt(ops, dtype, nh, nkv, hd, page, window):
    lengths = [1, 37, 130]
    pages_each = -(-max(lengths) // page)
    table = scattered_tables(len(lengths), pages_each, 3 * pages_each + 5, seed=hd)
    kp, vp = make_pools(3 * pages_each + 5, nkv, page, hd, dtype, fill=1.0)
    # queries: the last min(len, 9) positions of each request (a portion), one query for the first
    pos, entry = [], []
    for i, n in enumerate(lengths):
        for p in range(max(0, n - 9), n):
            pos.append(p)
            entry.append(i)
    q = torch.randn(len(pos), nh, hd, device=DEV).to(dtype)
    out = torch.empty_like(q)
    pos_t = torch.tensor(pos, dtype=torch.int32, device=DEV)
    entry_t = torch.tensor(entry, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    ops.attention_simt(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, window, scale, status)
    want = reference_attention(q, kp, vp, table, pos, entry, page, window, scale)
    assert int(status) == 0 and rel(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("nh,nkv,hd,page", [(8, 2, 64, 16), (8, 1, 128, 16), (32, 8, 128, 16), (16, 1, 64, 32),
                                            (6, 2, 128, 64), (4, 4, 64, 16), (6, 2, 96, 16), (5, 5, 32, 16),
                                            (9, 3, 48, 32), (4, 1, 80, 16), (14, 2, 112, 48)])
@pytest.mark.parametrize("splits", [1, 2, 5, 8, 12, 16, 20])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode(ops, nh, nkv, hd, page, splits, window):
    dtype = torch.bfloat16
    assert ops.attention_decode_supports(hd, nh // nkv, page, dtype)
    lengths = [1, 15, 16, 17, 250, 700]
    pages_each = -(-max(lengths) // page)
    n_pages = len(lengths) * pages_each + 3
    table = scattered_tables(len(lengths), pages_each, n_pages, seed=hd + page)
    kp, vp = make_pools(n_pages, nkv, page, hd, dtype, fill=1.0)
    pos = [n - 1 for n in lengths]
    entry = list(range(len(lengths)))
    q = torch.randn(len(pos), nh, hd, device=DEV).to(dtype)
    out = torch.full_like(q, float("nan"))
    pos_t = torch.tensor(pos, dtype=torch.int32, device=DEV)
    entry_t = torch.tensor(entry, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    scratch = torch.full((ops.attention_decode_scratch_floats(len(pos), nh, hd, splits),), float("nan"),
                         device=DEV) if splits > 1 else None
    ops.attention_decode(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, window, scale, splits, scratch, status)
    want = reference_attention(q, kp, vp, table, pos, entry, page, window, scale)
    assert int(status) == 0 and rel(out, want) < 1e-2


@pytest.mark.parametrize("nh,nkv,hd,page", [(8, 2, 64, 16), (8, 1, 128, 16), (32, 8, 128, 16), (16, 1, 64, 32),
                                            (6, 2, 128, 64), (4, 4, 64, 16), (6, 2, 96, 16), (9, 3, 48, 32),
                                            (3, 1, 80, 16)])
@pytest.mark.parametrize("target", [1, 7, 40, 500])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode_over_a_work_list(ops, nh, nkv, hd, page, target, window):
    """Requests of very different lengths, their keys cut into work items by the
    part's own planner (from no cut at all to items of eight tiles), the list padded with
    empty rows, twice in a row (the second call finds the counters as the first left them)."""
    from pulsarlm_b200.parts.attention import decode_work_items

    dtype = torch.bfloat16
    lengths = [1, 15, 16, 17, 250, 700, 129, 2100]
    pages_each = -(-max(lengths) // page)
    n_pages = len(lengths) * pages_each + 3
    table = scattered_tables(len(lengths), pages_each, n_pages, seed=hd + page)
    kp, vp = make_pools(n_pages, nkv, page, hd, dtype, fill=1.0)
    pos = [n - 1 for n in lengths]
    entry = list(range(len(lengths)))
    pos_t = torch.tensor(pos, dtype=torch.int32, device=DEV)
    entry_t = torch.tensor(entry, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    items, slots = decode_work_items(lengths, window, target, pad_to=target + len(lengths) + 3,
                                     min_tiles=2 if target == 500 else 32)
    real = items[items[:, 2] > 0]
    assert len(lengths) <= len(real) <= target + len(lengths)
    assert window is not None or (target == 1) == (len(real) == len(lengths))
    for t, n in enumerate(lengths):  # every attended tile of every request exactly once
        first = (max(0, n - window) if window else 0) // 16
        mine = sorted((r[1], r[2]) for r in real if r[0] == t)
        assert mine[0][0] == first and mine[-1][0] + mine[-1][1] == -(-n // 16)
        assert all(a[0] + a[1] == b[0] for a, b in zip(mine, mine[1:]))
    items_t, slots_t = torch.from_numpy(items).to(DEV), torch.from_numpy(slots).to(DEV)
    for _ in range(2):
        q = torch.randn(len(pos), nh, hd, device=DEV).to(dtype)
        out = torch.full_like(q, float("nan"))
        scratch = torch.full((items.shape[0] * nh * (hd + 2),), float("nan"), device=DEV)
        ops.attention_decode_items(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, window, scale, items_t,
                                   slots_t, scratch, status)
        want = reference_attention(q, kp, vp, table, pos, entry, page, window, scale)
        assert int(status) == 0 and rel(out, want) < 1e-2
    assert int(ops.attention_decode_counters(q.device).abs().sum()) == 0


@pytest.mark.parametrize("nh,nkv,hd,page", [(8, 2, 64, 16), (32, 8, 128, 16), (6, 6, 128, 32), (16, 1, 64, 64),
                                            (6, 2, 96, 16), (4, 4, 32, 32)])
@pytest.mark.parametrize("mode", ["splits1", "splits3", "splits12", "splits20", "items"])
@pytest.mark.parametrize("window", [None, 100])
def test_attention_decode_with_the_rotation_and_the_cache_write_folded_in(ops, nh, nkv, hd, page, mode, window):
    """One call that rotates q, rotates and stores the new keys and values, and attends,
    against the rotation kernel followed by the plain call: the same bits in the cache and
    in the output, whichever CTA and warp the token's own tile falls to (lengths that put
    it first, last and alone in a share), and nothing else written."""
    from pulsarlm_b200.parts.attention import decode_work_items

    dtype = torch.bfloat16
    lengths = [1, 16, 17, 33, 250, 700, 129, 1041]
    n = len(lengths)
    pages_each = -(-max(lengths) // page)
    n_pages = n * pages_each + 3
    table = scattered_tables(n, pages_each, n_pages, seed=hd + page).to(DEV)
    kp, vp = make_pools(n_pages, nkv, page, hd, dtype, fill=1.0)
    pos_t = torch.tensor([c - 1 for c in lengths], dtype=torch.int32, device=DEV)
    entry_t = torch.arange(n, dtype=torch.int32, device=DEV)
    inv_freq = plain_llama.rope_inverse_frequency(500000.0, hd, None).to(DEV)
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, device=DEV).to(dtype)

    def views(buffer):
        return (buffer[:, : nh * hd].view(n, nh, hd), buffer[:, nh * hd : (nh + nkv) * hd].view(n, nkv, hd),
                buffer[:, (nh + nkv) * hd :].view(n, nkv, hd))

    scale = 1 / math.sqrt(hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def attend(q, k_pool, v_pool, out, rope):
        if mode == "items":
            items, slots = decode_work_items(lengths, window, 9, min_tiles=4)
            scratch = torch.empty(items.shape[0] * nh * (hd + 2), device=DEV)
            ops.attention_decode_items(q, k_pool, v_pool, table, pos_t, entry_t, out, page, window, scale,
                                       torch.from_numpy(items).to(DEV), torch.from_numpy(slots).to(DEV), scratch,
                                       status, rope)
        else:
            splits = int(mode[6:])
            scratch = torch.empty(max(1, ops.attention_decode_scratch_floats(n, nh, hd, splits)), device=DEV)
            ops.attention_decode(q, k_pool, v_pool, table, pos_t, entry_t, out, page, window, scale, splits, scratch,
                                 status, rope=rope)

    # the two kernels
    first = qkv.clone()
    q1, k1, v1 = views(first)
    kp1, vp1 = kp.clone(), vp.clone()
    ops.rope_kv_write(q1, k1, v1, pos_t, entry_t, table, kp1, vp1, page, inv_freq, hd, status)
    out1 = torch.full((n, nh, hd), float("nan"), device=DEV, dtype=dtype)
    attend(q1, kp1, vp1, out1, None)
    # the one
    second = qkv.clone()
    q2, k2, v2 = views(second)
    kp2, vp2 = kp.clone(), vp.clone()
    out2 = torch.full((n, nh, hd), float("nan"), device=DEV, dtype=dtype)
    attend(q2, kp2, vp2, out2, (k2, v2, inv_freq, hd))
    assert int(status) == 0
    assert torch.equal(second, qkv)                       # q, k, v are left as they came
    assert torch.equal(kp1, kp2) and torch.equal(vp1, vp2)
    assert not torch.equal(kp2, kp)
    assert torch.equal(out1, out2)
    want = reference_attention(q1, kp1, vp1, table.cpu(), pos_t.tolist(), entry_t.tolist(), page, window, scale)
    assert rel(out2, want) < 1e-2


def test_attention_decode_refuses_what_it_cannot_do(ops):
    assert not ops.attention_decode_supports(160, 1, 16, torch.bfloat16)
    assert not ops.attention_decode_supports(72, 1, 16, torch.bfloat16)
    assert not ops.attention_decode_supports(16, 1, 16, torch.bfloat16)
    assert not ops.attention_decode_supports(128, 32, 16, torch.bfloat16)
    assert not ops.attention_decode_supports(128, 4, 8, torch.bfloat16)
    assert not ops.attention_decode_supports(128, 4, 16, torch.float32)
    q = torch.randn(1, 2, 160, device=DEV).to(torch.bfloat16)
    kp, vp = make_pools(2, 2, 16, 160, torch.bfloat16)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError) as error:
        ops.attention_decode(q, kp, vp, torch.zeros(1, 1, dtype=torch.int32, device=DEV), z, z, torch.empty_like(q),
                             16, None, 1.0, 1, None)
    assert "head_dim=160" in str(error.value)


@pytest.mark.parametrize("kernel", ["simt_f32", "simt_bf16", "decode", "decode_items"])
@pytest.mark.parametrize("far_key", [0, 15, 16, 511, 512, 1203])
def test_one_far_key_among_many_is_found(ops, kernel, far_key):
    """One key (at a page's first slot, last slot, far back) matches the query
    strongly; the output must be that key's value. A kernel that skips a tile, a
    page or a split loses it."""
    dtype = torch.float32 if kernel == "simt_f32" else torch.bfloat16
    nh, nkv, hd, page, n = 4, 2, 64, 16, 1204
    pages_each = -(-n // page)
    table = scattered_tables(1, pages_each, pages_each + 7, seed=3)
    kp, vp = make_pools(pages_each + 7, nkv, page, hd, dtype, fill=0.3)
    q = torch.randn(1, nh, hd, device=DEV).to(dtype)
    page_id = int(table[0, far_key // page])
    for kvh in range(nkv):
        # the key is the mean of the group's queries, scaled up: its score dominates
        direction = q[0, kvh * 2 : kvh * 2 + 2].float().mean(0)
        kp[page_id, kvh, far_key % page] = (direction * 12).to(dtype)
    vp[page_id, :, far_key % page] = 5.0
    out = torch.empty_like(q)
    pos_t = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    entry_t = torch.zeros(1, dtype=torch.int32, device=DEV)
    if kernel == "decode":
        scratch = torch.empty(ops.attention_decode_scratch_floats(1, nh, hd, 7), device=DEV)
        ops.attention_decode(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, None, 1.0, 7, scratch)
    elif kernel == "decode_items":
        from pulsarlm_b200.parts.attention import decode_work_items

        # a second, short request makes the lengths unequal, so that the long one is cut
        items, slots = decode_work_items([n, 20], None, 9, min_tiles=8)
        assert len(items) > 5
        q2 = torch.cat([q, q])
        out2 = torch.empty_like(q2)
        pos2 = torch.tensor([n - 1, 19], dtype=torch.int32, device=DEV)
        scratch = torch.empty(items.shape[0] * nh * (hd + 2), device=DEV)
        ops.attention_decode_items(q2, kp, vp, table.to(DEV), pos2, torch.zeros(2, dtype=torch.int32, device=DEV),
                                   out2, page, None, 1.0, torch.from_numpy(items).to(DEV),
                                   torch.from_numpy(slots).to(DEV), scratch)
        out = out2[:1]
    else:
        ops.attention_simt(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, None, 1.0)
    want = reference_attention(q, kp, vp, table, [n - 1], [0], page, None, 1.0)
    assert float(want.min()) > 4.0  # the construction works: the far key takes nearly all the weight
    assert rel(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)


def dense_attention(q, kp, vp, table_row, positions, page, scale):
    """Attention of query t over keys 0..positions[t] of one request, gathered through
    its block-table row in one indexing step (for histories too long for
    `reference_attention`'s loop); float64 on the device."""
    n = max(positions) + 1
    index = torch.arange(n, device=q.device)
    rows = table_row.to(q.device).long()[index // page]
    keys, vals = kp[rows, :, index % page].double(), vp[rows, :, index % page].double()  # [n, nkv, hd]
    group = q.shape[1] // kp.shape[1]
    out = torch.empty(q.shape, dtype=torch.float64, device=q.device)
    for t, p in enumerate(positions):
        for h in range(q.shape[1]):
            s = (keys[: p + 1, h // group] @ q[t, h].double()) * scale
            out[t, h] = torch.softmax(s, 0) @ vals[: p + 1, h // group]
    return out.cpu()


@pytest.mark.parametrize("kernel", ["decode", "decode_items", "simt_bf16", "tcgen05", "mma"])
@pytest.mark.parametrize("hd,far_key", [(128, 70_001), (64, 3), (128, 131_000)])
def test_one_far_key_among_a_hundred_thousand(ops, kernel, hd, far_key):
    """A history of 131,072 keys (8,192 pages): one key far back, or almost the newest,
    takes nearly all the weight. The decode kernel with the
    split count the part chooses for such a request (more than a cluster holds: through
    scratch memory and the merge kernel) and over a work list; the prompt kernels for a
    portion of 130 tokens at the history's end, split over the keys as the part chooses."""
    from pulsarlm_b200.parts.attention import decode_splits, decode_work_items, prefill_splits

    dtype = torch.bfloat16
    nh, nkv, page, n = 4, 2, 16, 131_072
    pages_each = n // page
    table = scattered_tables(1, pages_each, pages_each + 5, seed=hd)
    kp, vp = make_pools(pages_each + 5, nkv, page, hd, dtype, fill=0.3)
    direction = torch.randn(hd, device=DEV)
    n_q = 1 if kernel in ("decode", "decode_items", "simt_bf16") else 130
    q = (direction[None, None, :] + 0.05 * torch.randn(n_q, nh, hd, device=DEV)).to(dtype)
    page_id = int(table[0, far_key // page])
    kp[page_id, :, far_key % page] = (direction * (14 if hd == 128 else 20)).to(dtype)
    vp[page_id, :, far_key % page] = 5.0
    positions = list(range(n - n_q, n))
    out = torch.full_like(q, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    entry_t = torch.zeros(n_q, dtype=torch.int32, device=DEV)
    if kernel == "decode":
        splits = decode_splits(nkv, n, torch.device(DEV), hd, nh // nkv)
        assert splits > 16
        scratch = torch.empty(ops.attention_decode_scratch_floats(1, nh, hd, splits), device=DEV)
        ops.attention_decode(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, None, scale, splits, scratch, status)
    elif kernel == "decode_items":
        items, slots = decode_work_items([n, 3000], None, 150)
        assert int((items[:, 2] > 0).sum()) > 100
        q2, out2 = torch.cat([q, q]), torch.full((2, nh, hd), float("nan"), device=DEV, dtype=dtype)
        pos2 = torch.tensor([n - 1, 2999], dtype=torch.int32, device=DEV)
        scratch = torch.empty(items.shape[0] * nh * (hd + 2), device=DEV)
        ops.attention_decode_items(q2, kp, vp, table.to(DEV), pos2, torch.zeros(2, dtype=torch.int32, device=DEV),
                                   out2, page, None, scale, torch.from_numpy(items).to(DEV),
                                   torch.from_numpy(slots).to(DEV), scratch, status)
        out = out2[:1]
    elif kernel == "simt_bf16":
        ops.attention_simt(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, None, scale, status)
    elif kernel == "tcgen05":
        tiles = make_tiles([(0, n_q, n - n_q, 0)], 128)
        splits = prefill_splits(tiles.shape[0] * nh // 2, n, n_q, nh, hd, torch.device(DEV))
        assert splits > 1
        ops.attention_prefill_tcgen05(q, kp, vp, table.to(DEV), tiles, out, page, None, scale, status, splits,
                                      split_scratch(ops, q, splits))
    else:
        ops.attention_prefill(q, kp, vp, table.to(DEV), make_tiles([(0, n_q, n - n_q, 0)], 128), out, page, None,
                              scale, status)
    want = dense_attention(q, kp, vp, table[0], positions, page, scale)
    sees = torch.tensor([p >= far_key for p in positions])
    assert bool((want[sees].amin(dim=(1, 2)) > 4.0).all())  # the construction works where the key is visible
    assert int(status) == 0 and rel(out, want) < 1e-2


@pytest.mark.parametrize("kernel", ["rope_then_decode", "decode_folded", "simt_bf16", "tcgen05", "mma"])
def test_pages_more_than_two_to_the_31_elements_into_the_pool(ops, kernel):
    """A pool of 70,000 pages at the 8B model's page size (4.6 GB for one layer's keys and
    values): the request's pages lie above element 2^31 of the pool, where an offset kept
    in 32 bits would wrap. The rotation kernel writes there, the attention kernels read."""
    dtype = torch.bfloat16
    nh, nkv, hd, page, n_pages, n = 32, 8, 128, 16, 70_000, 600
    pool = torch.zeros(n_pages, 2, nkv, page, hd, device=DEV, dtype=dtype)
    kp, vp = pool[:, 0], pool[:, 1]
    assert kp.stride(0) * 65_600 > 2 ** 31
    pages_each = -(-n // page)
    g = torch.Generator().manual_seed(4)
    table = (65_600 + torch.randperm(n_pages - 65_600, generator=g)[:pages_each]).view(1, -1).to(torch.int32)
    rows = table[0].long().to(DEV)
    kp[rows] = (0.3 * torch.randn(pages_each, nkv, page, hd, device=DEV)).to(dtype)
    vp[rows] = (0.3 * torch.randn(pages_each, nkv, page, hd, device=DEV)).to(dtype)
    scale = 1 / math.sqrt(hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    if kernel in ("rope_then_decode", "decode_folded"):
        # the newest token's key and value are written by the kernels themselves
        inv_freq = plain_llama.rope_inverse_frequency(500000.0, hd, None).to(DEV)
        qkv = torch.randn(1, (nh + 2 * nkv) * hd, device=DEV).to(dtype)
        q = qkv[:, : nh * hd].view(1, nh, hd)
        k = qkv[:, nh * hd : (nh + nkv) * hd].view(1, nkv, hd)
        v = qkv[:, (nh + nkv) * hd :].view(1, nkv, hd)
        pos_t = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        entry_t = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.full((1, nh, hd), float("nan"), device=DEV, dtype=dtype)
        pos64 = torch.tensor([n - 1])
        want_k = plain_llama.rope_rotate(k.double().cpu(), pos64, inv_freq.cpu())
        want_q = plain_llama.rope_rotate(q.double().cpu(), pos64, inv_freq.cpu())
        if kernel == "rope_then_decode":
            ops.rope_kv_write(q, k, v, pos_t, entry_t, table.to(DEV), kp, vp, page, inv_freq, hd, status)
            ops.attention_decode(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, None, scale, 1, None, status)
        else:
            scratch = torch.empty(ops.attention_decode_scratch_floats(1, nh, hd, 3), device=DEV)
            ops.attention_decode(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, None, scale, 3, scratch, status,
                                 rope=(k, v, inv_freq, hd))
        at = (int(table[0, (n - 1) // page]), slice(None), (n - 1) % page)
        assert rel(kp[at], want_k[0]) < 1e-2 and torch.equal(vp[at], v[0])
        want = dense_attention(want_q.to(DEV).to(dtype), kp, vp, table[0], [n - 1], page, scale)
    else:
        n_q = 1 if kernel == "simt_bf16" else 130
        q = torch.randn(n_q, nh, hd, device=DEV).to(dtype)
        out = torch.full_like(q, float("nan"))
        positions = list(range(n - n_q, n))
        if kernel == "simt_bf16":
            ops.attention_simt(q, kp, vp, table.to(DEV), torch.tensor(positions, dtype=torch.int32, device=DEV),
                               torch.zeros(n_q, dtype=torch.int32, device=DEV), out, page, None, scale, status)
        else:
            prefill_kernel(ops, kernel)(q, kp, vp, table.to(DEV), make_tiles([(0, n_q, n - n_q, 0)], 128), out, page,
                                        None, scale, status)
        want = dense_attention(q, kp, vp, table[0], positions, page, scale)
    assert int(status) == 0 and rel(out, want) < 1e-2


@pytest.mark.parametrize("kernel", ["simt_f32", "simt_bf16", "decode"])
def test_window_edges(ops, kernel):
    """A loud key just inside the window must be read, the same key just outside
    must not."""
    dtype = torch.float32 if kernel == "simt_f32" else torch.bfloat16
    nh, nkv, hd, page, n, window = 2, 1, 64, 16, 300, 100
    pages_each = -(-n // page)
    table = scattered_tables(1, pages_each, pages_each + 2, seed=5)
    q = torch.randn(1, nh, hd, device=DEV).to(dtype)
    for loud, inside in ((n - window, True), (n - window - 1, False)):
        kp, vp = make_pools(pages_each + 2, nkv, page, hd, dtype, fill=0.3)
        page_id = int(table[0, loud // page])
        kp[page_id, 0, loud % page] = (q[0].float().mean(0) * 12).to(dtype)
        vp[page_id, 0, loud % page] = 5.0
        out = torch.empty_like(q)
        pos_t = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        entry_t = torch.zeros(1, dtype=torch.int32, device=DEV)
        if kernel == "decode":
            scratch = torch.empty(ops.attention_decode_scratch_floats(1, nh, hd, 3), device=DEV)
            ops.attention_decode(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, window, 1.0, 3, scratch)
        else:
            ops.attention_simt(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, window, 1.0)
        want = reference_attention(q, kp, vp, table, [n - 1], [0], page, window, 1.0)
        assert (float(want.min()) > 4.0) == inside
        assert rel(out, want) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_pages_before_the_window_are_never_read(ops):
    """Block-table entries before the window are -1 (given back): reading them would
    raise the status flag."""
    for kernel in ("simt", "decode"):
        nh, nkv, hd, page, n, window = 2, 1, 64, 16, 200, 40
        pages_each = -(-n // page)
        table = scattered_tables(1, pages_each, pages_each, seed=1)
        table[0, : (n - window) // page] = -1
        kp, vp = make_pools(pages_each, nkv, page, hd, torch.bfloat16, fill=1.0)
        q = torch.randn(1, nh, hd, device=DEV).to(torch.bfloat16)
        out = torch.empty_like(q)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        pos_t = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        entry_t = torch.zeros(1, dtype=torch.int32, device=DEV)
        if kernel == "decode":
            ops.attention_decode(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, window, 0.125, 1, None, status)
        else:
            ops.attention_simt(q, kp, vp, table.to(DEV), pos_t, entry_t, out, page, window, 0.125, status)
        assert int(status) == 0, kernel


def make_tiles(portions, tile_rows=128):
    """portions: [(first row, rows, first position, table row)] -> int32 [n, 4] tiles."""
    tiles = []
    for row0, n, pos0, entry in portions:
        for r in range(0, n, tile_rows):
            tiles.append((row0 + r, min(tile_rows, n - r), pos0 + r, entry))
    tiles.sort(key=lambda t: -(t[2] + t[1]))
    return torch.tensor(tiles, dtype=torch.int32, device=DEV)


def prefill_kernel(ops, name):
    return ops.attention_prefill_tcgen05 if name == "tcgen05" else ops.attention_prefill


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
@pytest.mark.parametrize("nh,nkv,hd,page", [(8, 2, 64, 16), (4, 1, 128, 16), (6, 6, 64, 32), (5, 1, 128, 8),
                                            (3, 3, 128, 64), (6, 2, 96, 16), (5, 5, 32, 8), (9, 3, 48, 32),
                                            (4, 1, 80, 16), (14, 2, 112, 48)])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_prefill(ops, kernel, nh, nkv, hd, page, window):
    dtype = torch.bfloat16
    assert ops.attention_prefill_supports(hd, page, dtype)
    if kernel == "tcgen05" and (page % 16 or hd not in (64, 128)):
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128 and pages that are multiples of 16 tokens")
    # request 0: a whole prompt of 150 from position 0; request 1: a portion of 2 at 300..301;
    # request 2: a portion of 131 starting at 77 (not aligned to anything)
    lengths = [150, 302, 208]
    portions = [(0, 150, 0, 0), (150, 2, 300, 1), (152, 131, 77, 2)]
    pages_each = -(-max(lengths) // page)
    n_pages = 3 * pages_each + 4
    table = scattered_tables(3, pages_each, n_pages, seed=hd + page)
    kp, vp = make_pools(n_pages, nkv, page, hd, dtype, fill=1.0)
    pos, entry = [], []
    for row0, n, pos0, e in portions:
        pos += list(range(pos0, pos0 + n))
        entry += [e] * n
    q = torch.randn(len(pos), nh, hd, device=DEV).to(dtype)
    out = torch.full_like(q, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    if kernel == "tcgen05":
        assert ops.attention_prefill_tcgen05_supports(q, kp, page)
    run = prefill_kernel(ops, kernel)
    run(q, kp, vp, table.to(DEV), make_tiles(portions, 128), out, page, window, scale, status)
    want = reference_attention(q, kp, vp, table, pos, entry, page, window, scale)
    assert int(status) == 0 and rel(out, want) < 1e-2
    # with an offset: the kernel is given only the rows after two leading ones, as in a mixed batch
    out2 = torch.full_like(q, float("nan"))
    later = [(row0, n, pos0, e) for row0, n, pos0, e in portions[1:]]
    run(q, kp, vp, table.to(DEV), make_tiles(later, 128), out2, page, window, scale, status)
    assert rel(out2[150:], want[150:]) < 1e-2 and bool(torch.isnan(out2[:150].float()).all())
    if kernel == "tcgen05" and (nh // nkv) % 2 == 1:
        # an odd group: one head per CTA, and tiles of twice the rows whose halves share the keys
        rows = ops.attention_prefill_tcgen05_tile_rows(nh // nkv)
        assert rows == 256
        out3 = torch.full_like(q, float("nan"))
        ops.attention_prefill_tcgen05(q, kp, vp, table.to(DEV), make_tiles(portions, rows), out3, page, window,
                                      scale, status, wide=True)
        assert int(status) == 0 and rel(out3, want) < 1e-2


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
@pytest.mark.parametrize("far_key", [0, 63, 64, 65, 1023, 1024, 1100])
def test_prefill_finds_one_far_key_and_respects_causality(ops, kernel, far_key):
    """A loud key: queries at or after it must return its value, queries before it
    must not see it (a kernel that drops a tile, or reads past the diagonal, fails)."""
    dtype = torch.bfloat16
    nh, nkv, hd, page = 2, 1, 64, 16
    n_ctx, n_q = 1204, 140  # the portion is the last 140 positions
    pages_each = -(-n_ctx // page)
    table = scattered_tables(1, pages_each, pages_each + 3, seed=9)
    kp, vp = make_pools(pages_each + 3, nkv, page, hd, dtype, fill=0.3)
    direction = torch.randn(hd, device=DEV)
    q = (direction[None, None, :] + 0.05 * torch.randn(n_q, nh, hd, device=DEV)).to(dtype)
    page_id = int(table[0, far_key // page])
    kp[page_id, 0, far_key % page] = (direction * 12).to(dtype)
    vp[page_id, 0, far_key % page] = 5.0
    pos0 = n_ctx - n_q
    out = torch.empty_like(q)
    prefill_kernel(ops, kernel)(q, kp, vp, table.to(DEV), make_tiles([(0, n_q, pos0, 0)], 128), out, page, None, 1.0)
    pos = list(range(pos0, n_ctx))
    want = reference_attention(q, kp, vp, table, pos, [0] * n_q, page, None, 1.0)
    sees = torch.tensor([p >= far_key for p in pos])
    assert bool((want[sees].amin(dim=(1, 2)) > 4.0).all()) and (sees.all() or bool((want[~sees].amax(dim=(1, 2)) < 3.0).all()))
    assert rel(out, want) < 1e-2


def split_scratch(ops, q, splits):
    """Scratch for `splits` splits of the keys, filled with NaN: what a split leaves
    unwritten must never reach the output."""
    n = ops.attention_prefill_scratch_floats(q.shape[0], q.shape[1], q.shape[2], splits)
    return torch.full((max(n, 1),), float("nan"), device=DEV)


@pytest.mark.parametrize("nh,nkv,hd,page", [(8, 2, 64, 16), (4, 1, 128, 16), (6, 6, 64, 32), (3, 3, 128, 64)])
@pytest.mark.parametrize("splits,window", [(2, None), (3, 300), (7, None), (32, 300)])
def test_attention_prefill_with_split_keys(ops, nh, nkv, hd, page, splits, window):
    """Portions after long and short histories in one launch: tiles with many 64-key
    tiles, with fewer than there are splits (some splits stay empty), and a whole
    prompt from position 0 (early rows see nothing in the later splits)."""
    dtype = torch.bfloat16
    lengths = [1500, 900, 140, 40]
    portions = [(0, 200, 1300, 0), (200, 2, 898, 1), (202, 140, 0, 2), (342, 3, 37, 3)]
    pages_each = -(-max(lengths) // page)
    n_pages = len(lengths) * pages_each + 4
    table = scattered_tables(len(lengths), pages_each, n_pages, seed=hd + page + splits)
    kp, vp = make_pools(n_pages, nkv, page, hd, dtype, fill=1.0)
    pos, entry = [], []
    for row0, n, pos0, e in portions:
        pos += list(range(pos0, pos0 + n))
        entry += [e] * n
    q = torch.randn(len(pos), nh, hd, device=DEV).to(dtype)
    scale = 1 / math.sqrt(hd)
    tiles = make_tiles(portions, 128)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    wide = (nh // nkv) % 2 == 1  # (both arrangements for odd groups are covered: see the far-key test below)
    if wide:
        tiles = make_tiles(portions, ops.attention_prefill_tcgen05_tile_rows(nh // nkv))
    whole = torch.full_like(q, float("nan"))
    ops.attention_prefill_tcgen05(q, kp, vp, table.to(DEV), tiles, whole, page, window, scale, status, wide=wide)
    out = torch.full_like(q, float("nan"))
    ops.attention_prefill_tcgen05(q, kp, vp, table.to(DEV), tiles, out, page, window, scale, status, splits,
                                  split_scratch(ops, q, splits), wide)
    want = reference_attention(q, kp, vp, table, pos, entry, page, window, scale)
    assert int(status) == 0 and rel(out, want) < 1e-2
    assert rel(out, whole.float()) <= 2.0 ** -7  # the splits change the rounding (one bfloat16 step) and nothing else


@pytest.mark.parametrize("splits,nh,wide", [(2, 2, False), (5, 2, False), (1, 1, False), (3, 1, False),
                                            (1, 1, True), (3, 1, True)])
@pytest.mark.parametrize("far_key", [0, 63, 64, 575, 576, 1023, 1100])
def test_split_prefill_finds_one_far_key_and_respects_causality(ops, splits, nh, wide, far_key):
    """As above with the keys split: the loud key lies in one split only, and the
    merge must let it dominate (and a split must not read past the diagonal). With one
    head to the kv head, in both arrangements the kernel has for odd groups: tiles of
    128 rows, and tiles of 256 rows whose halves take turns (the portion of 140 rows is
    then one tile, its second half mostly empty)."""
    dtype = torch.bfloat16
    nkv, hd, page = 1, 64, 16
    n_ctx, n_q = 1204, 140
    pages_each = -(-n_ctx // page)
    table = scattered_tables(1, pages_each, pages_each + 3, seed=9)
    kp, vp = make_pools(pages_each + 3, nkv, page, hd, dtype, fill=0.3)
    direction = torch.randn(hd, device=DEV)
    q = (direction[None, None, :] + 0.05 * torch.randn(n_q, nh, hd, device=DEV)).to(dtype)
    page_id = int(table[0, far_key // page])
    kp[page_id, 0, far_key % page] = (direction * 12).to(dtype)
    vp[page_id, 0, far_key % page] = 5.0
    pos0 = n_ctx - n_q
    out = torch.empty_like(q)
    ops.attention_prefill_tcgen05(q, kp, vp, table.to(DEV), make_tiles([(0, n_q, pos0, 0)], 256 if wide else 128),
                                  out, page, None, 1.0, None, splits, split_scratch(ops, q, splits), wide)
    pos = list(range(pos0, n_ctx))
    want = reference_attention(q, kp, vp, table, pos, [0] * n_q, page, None, 1.0)
    sees = torch.tensor([p >= far_key for p in pos])
    assert bool((want[sees].amin(dim=(1, 2)) > 4.0).all()) and (sees.all() or bool((want[~sees].amax(dim=(1, 2)) < 3.0).all()))
    assert rel(out, want) < 1e-2


def test_split_prefill_refuses_what_it_cannot_do(ops):
    q = torch.randn(4, 2, 64, device=DEV).to(torch.bfloat16)
    kp, vp = make_pools(2, 1, 16, 64, torch.bfloat16)
    table = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    tiles = make_tiles([(0, 4, 0, 0)], 128)
    with pytest.raises(ops.KernelError) as error:
        ops.attention_prefill_tcgen05(q, kp, vp, table, tiles, torch.empty_like(q), 16, None, 1.0, None, 33,
                                      split_scratch(ops, q, 33))
    assert "1 to 32 splits" in str(error.value)


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
def test_prefill_window_edges_and_released_pages(ops, kernel):
    dtype = torch.bfloat16
    nh, nkv, hd, page, window = 2, 1, 128, 16, 100
    n_ctx, n_q = 400, 70
    pos0 = n_ctx - n_q
    pages_each = -(-n_ctx // page)
    table = scattered_tables(1, pages_each, pages_each + 1, seed=2)
    first_needed = pos0 - window + 1
    table[0, : first_needed // page] = -1  # given back: must never be read
    kp, vp = make_pools(pages_each + 1, nkv, page, hd, dtype, fill=0.3)
    direction = torch.randn(hd, device=DEV)
    q = (direction[None, None, :] + 0.05 * torch.randn(n_q, nh, hd, device=DEV)).to(dtype)
    loud = pos0 - 60  # inside the window of the first 40 queries only
    page_id = int(table[0, loud // page])
    kp[page_id, 0, loud % page] = (direction * 10).to(dtype)
    vp[page_id, 0, loud % page] = 5.0
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    prefill_kernel(ops, kernel)(q, kp, vp, table.to(DEV), make_tiles([(0, n_q, pos0, 0)], 128), out, page, window,
                                1.0, status)
    pos = list(range(pos0, n_ctx))
    want = reference_attention(q, kp, vp, table, pos, [0] * n_q, page, window, 1.0)
    inside = torch.tensor([p - window + 1 <= loud for p in pos])
    assert inside.any() and (~inside).any()
    assert bool((want[inside].amin(dim=(1, 2)) > 4.0).all()) and bool((want[~inside].amax(dim=(1, 2)) < 3.0).all())
    assert int(status) == 0 and rel(out, want) < 1e-2


# ----------------------------------------------------------------------------- sampling

def run_sample(ops, logits, temperature, top_k=None, top_p=None, seeds=None, counts=None):
    rows = logits.shape[0]
    t = torch.tensor(temperature, dtype=torch.float32, device=DEV).expand(rows).contiguous()
    k = None if top_k is None else torch.tensor(top_k, dtype=torch.int32, device=DEV).expand(rows).contiguous()
    p = None if top_p is None else torch.tensor(top_p, dtype=torch.float32, device=DEV).expand(rows).contiguous()
    seeds = torch.arange(rows) if seeds is None else torch.as_tensor(seeds)
    counts = torch.zeros(rows, dtype=torch.int64) if counts is None else torch.as_tensor(counts)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, t, k, p, seeds.to(torch.int64).to(DEV), counts.to(torch.int64).to(DEV), out)
    return out.cpu()


def test_sampling_argmax_and_ties(ops):
    logits = torch.randn(9, 1000, device=DEV)
    logits[3, 17] = logits[3, 900] = 50.0  # a tie goes to the lower index
    got = run_sample(ops, logits, 0.0)
    want = logits.argmax(dim=1).cpu()
    want[3] = 17
    assert got.tolist() == want.tolist()
    assert run_sample(ops, logits, 1.0, top_k=1).tolist() == want.tolist()  # top_k = 1 is the argmax


def test_sampling_frequencies_match_the_distribution(ops):
    probabilities = torch.tensor([0.5, 0.25, 0.15, 0.07, 0.03])
    logits = torch.log(probabilities).repeat(6000, 1).to(DEV) * 0.7  # then T = 0.7 restores them
    for top_k, top_p in ((None, None), (2, None), (None, 0.8), (3, 0.6)):
        got = run_sample(ops, logits.contiguous(), 0.7, top_k, top_p)
        freq = torch.bincount(got, minlength=5).double() / 6000
        want = plain_llama.sampling_distribution(torch.log(probabilities) * 0.7, 0.7, top_k or 0, top_p or 1.0)
        assert (freq - want).abs().max() < 0.03, (top_k, top_p, freq, want)
        assert bool((freq[want == 0] == 0).all())


def test_sampling_is_keyed_by_seed_and_count_not_by_neighbours(ops):
    logits = torch.randn(6, 50000, device=DEV)
    a = run_sample(ops, logits, 1.0, seeds=[7, 7, 8, 9, 10, 11], counts=[0, 0, 0, 0, 0, 0])
    same_logits = logits.clone()
    same_logits[1] = logits[0]
    b = run_sample(ops, same_logits, 1.0, seeds=[7, 7, 8, 9, 10, 11], counts=[0, 0, 0, 0, 0, 0])
    assert b[0] == b[1] == a[0]  # same seed, count and logits: same token
    alone = run_sample(ops, logits[2:3].contiguous(), 1.0, seeds=[8], counts=[0])
    assert alone[0] == a[2]  # a row's draw does not depend on its neighbours
    later = run_sample(ops, logits, 1.0, seeds=[7, 7, 8, 9, 10, 11], counts=[1, 1, 1, 1, 1, 1])
    assert later.tolist() != a.tolist()  # another draw count: other noise
    mixed = run_sample(ops, logits, torch.tensor([0.0, 1.0, 0.0, 1.0, 0.0, 1.0]).tolist(),
                       seeds=[7, 7, 8, 9, 10, 11])
    assert mixed[0] == logits[0].argmax().cpu() and mixed[3] == a[3]  # greedy rows beside drawing rows


def test_sampling_never_picks_a_hopeless_token_in_a_wide_vocabulary(ops):
    vocab = 262144 + 3
    logits = torch.full((64, vocab), -1e4, device=DEV)
    logits[:, 1000:1010] = 0.0
    got = run_sample(ops, logits, 1.0)
    assert bool(((got >= 1000) & (got < 1010)).all())
    assert len(set(got.tolist())) > 3
