"""Python face of the CUDA kernel library: one function per entry point.

The library is loaded with ctypes on first use (and built first if stale). There
is no fallback: if it cannot be built or loaded, or the device is not sm_100,
the call raises. Every function launches on torch's current CUDA stream and
takes torch tensors on the device; shapes and dtypes are checked here, sizes a
kernel refuses come back as KernelError with the kernel's message.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

from . import build

_I32 = ctypes.c_int
_I64 = ctypes.c_int64
_F32 = ctypes.c_float
_PTR = ctypes.c_void_p

_lib = None
_lock = threading.Lock()

ABI_VERSION = 21

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


_SIGNATURES = {
    "pl_embed": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _PTR, _PTR],
    "pl_take_tokens": [_PTR, _PTR, _PTR, _I32, _I32, _PTR, _PTR],
    "pl_add_rmsnorm": [_PTR, _PTR, _PTR, _I32, _PTR, _PTR, _I32, _I32, _F32, _I32, _PTR],
    "pl_swiglu": [_PTR, _PTR, _I32, _I32, _I32, _PTR],
    "pl_bf16_to_f32": [_PTR, _PTR, _I64, _PTR],
    "pl_gemm_f32": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _PTR],
    "pl_rope_kv_write": [_PTR, _PTR, _PTR, _I64, _PTR, _PTR, _PTR, _I32, _PTR, _PTR, _I64, _I64, _I32, _I32,
                         _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _PTR, _PTR, _F32, _PTR, _PTR],
    "pl_attention_simt": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                          _I32, _I32, _I32, _I32, _I32, _F32, _F32, _I32, _PTR, _PTR, _PTR, _PTR, _PTR],
    "pl_attention_decode": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                            _I32, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _PTR, _PTR, _PTR],
    "pl_attention_decode_mass": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                                 _I32, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _PTR, _I32, _PTR, _PTR, _F32, _PTR,
                                 _PTR],
    "pl_attention_decode_items": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                                  _I32, _I32, _I32, _I32, _I32, _F32, _PTR, _I32, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR],
    "pl_attention_decode_ctas_per_sm": [_I32],
    "pl_layer_forward": [_PTR, _PTR, _PTR],
    "pl_gemm_bf16_skinny_gated_in": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I64, _I64, _I64, _I32, _PTR, _PTR],
    "pl_fill_random": [_PTR, _I64, _I32, ctypes.c_uint64, ctypes.c_uint64, _F32, _F32, _PTR],
    "pl_attention_decode_supports": [_I32, _I32, _I32, _I32],
    "pl_attention_prefill": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _I32, _PTR, _I64,
                             _I32, _I32, _I32, _I32, _F32, _PTR, _PTR],
    "pl_attention_prefill_supports": [_I32, _I32, _I32],
    "pl_attention_prefill_tcgen05": [_PTR, _I64, _I32, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _I32,
                                     _PTR, _I64, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _I32, _PTR, _PTR, _PTR],
    "pl_attention_prefill_tcgen05_tile_rows": [_I32],
    "pl_attention_prefill_tcgen05_supports": [_I32, _I32, _I32, _I64, _I64, _I64, _I32],
    "pl_attention_prefill_tile_rows": [],
    "pl_gemm_bf16_pair_supports": [_I32, _I32, _I32, _I64, _I64],
    "pl_gemm_bf16_skinny": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I64, _I64, _I64, _I32, _PTR, _PTR],
    "pl_gemm_bf16_skinny_max_tokens": [],
    "pl_gemm_bf16_pair": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I64, _I64, _I64, _I32, _I32, _PTR, _PTR],
    "pl_attention_decode_resident_clusters": [_I32, _I32, _I32],
    "pl_gemm_bf16_skinny_splits": [_I32, _I32, _I32],
    "pl_sample": [_PTR, _I64, _I32, _I32, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build.library_path(build=True)
        lib = ctypes.CDLL(path)
        lib.pl_last_error.restype = ctypes.c_char_p
        lib.pl_abi_version.restype = _I32
        if lib.pl_abi_version() != ABI_VERSION:
            raise KernelError(f"{path}: ABI version {lib.pl_abi_version()} does not match the package's "
                              f"{ABI_VERSION}; delete the build folder and try again")
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _I32
        lib.pl_device_arch.restype = _I32
        lib.pl_attention_decode_scratch_floats.argtypes = [_I32, _I32, _I32, _I32]
        lib.pl_attention_decode_scratch_floats.restype = _I64
        lib.pl_attention_prefill_scratch_floats.argtypes = [_I32, _I32, _I32, _I32]
        lib.pl_attention_prefill_scratch_floats.restype = _I64
        lib.pl_set_overlap.argtypes = [_I32]
        lib.pl_set_overlap.restype = _I32
        if os.environ.get("PULSARLM_B200_OVERLAP", "1") == "0":
            lib.pl_set_overlap(0)
        _lib = lib
    return _lib


def set_overlap(enabled: bool) -> bool:
    """Lets consecutive kernels of a stream overlap (programmatic dependent launch:
    a kernel's set-up and weight loads run under its predecessor's tail). On by
    default; `PULSARLM_B200_OVERLAP=0` starts with it off. Returns the old setting."""
    return bool(library().pl_set_overlap(int(enabled)))


_device_checked = False


def require_device() -> None:
    """Raises unless a CUDA device of compute capability 10.x is current."""
    global _device_checked
    if _device_checked:
        return
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: the engine runs on a B200 (sm_100) only and has no CPU path")
    torch.cuda.init()
    arch = library().pl_device_arch()
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a; the current device is sm_{arch}")
    _device_checked = True


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (torch's; inside a graph capture, the capturing stream).
    Asked through torch's C entry point when it has one: the Python object costs 15 us a
    call, which a step of a few hundred launches notices."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_launches = 0


def launch_count() -> int:
    """How many kernel entry points of this library have been called so far."""
    return _launches


def _call(name: str, *args) -> None:
    global _launches
    _launches += 1
    code = getattr(library(), name)(*args)
    if code != 0:
        raise KernelError(library().pl_last_error().decode("utf-8", "replace"))


def call_native(name: str, *args, launches: int = 1) -> None:
    """Calls an entry point that takes structs and the stream (the caller has checked what
    the structs point at); `launches`: how many of the library's kernels it launches."""
    global _launches
    _launches += launches - 1
    _call(name, *args, _stream())


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16") from None


def _dev(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")


# ----------------------------------------------------------------------------- ops

def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, status: torch.Tensor | None = None) -> None:
    """out[t] (fp32 [T, H]) = table[tokens[t]]; tokens int32 [T]."""
    _dev(table, tokens, out, status)
    assert table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32
    assert tokens.dtype == torch.int32 and tokens.is_contiguous()
    vocab, hidden = table.shape
    _call("pl_embed", _p(table), _p(tokens), _p(out), tokens.numel(), hidden, vocab, _code(table.dtype),
          _p(status), _stream())


def take_tokens(tokens: torch.Tensor, source: torch.Tensor, ids: torch.Tensor,
                status: torch.Tensor | None = None) -> None:
    """tokens[i] = ids[source[i]] for the rows with source[i] >= 0 (all int32, on the
    device): the tokens of entries that go on from a step whose ids are still being drawn."""
    _dev(tokens, source, ids, status)
    assert tokens.dtype == source.dtype == ids.dtype == torch.int32
    assert tokens.is_contiguous() and source.is_contiguous() and ids.is_contiguous()
    assert source.numel() <= tokens.numel()
    _call("pl_take_tokens", _p(tokens), _p(source), _p(ids), source.numel(), ids.numel(), _p(status), _stream())


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> None:
    """x fp32 [T, H] residual stream; x += delta (when rows is None); out = norm(x + delta) * weight.
    With rows (int32 [R]), output row r is made from source row rows[r] and x is left as it was."""
    _dev(x, delta, weight, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    hidden = x.shape[-1]
    n_rows = rows.numel() if rows is not None else x.shape[0]
    assert out.shape == (n_rows, hidden) and weight.shape == (hidden,) and weight.is_contiguous()
    if delta is not None:
        assert delta.shape == x.shape and delta.dtype == out.dtype and delta.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    _call("pl_add_rmsnorm", _p(x), _p(delta), _p(weight), _code(weight.dtype), _p(out), _p(rows), n_rows, hidden,
          float(eps), _code(out.dtype), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _dev(gate_up, out)
    tokens, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (tokens, two_i // 2) and out.dtype == gate_up.dtype
    assert gate_up.is_contiguous() and out.is_contiguous()
    _call("pl_swiglu", _p(gate_up), _p(out), tokens, two_i // 2, _code(out.dtype), _stream())


def fill_random(out: torch.Tensor, seed: int, tensor_hash: int, scale: float, offset: float = 0.0) -> None:
    """out = offset + scale * noise(seed, tensor_hash, element index): random weights drawn in
    place, the same bits as the host core draws (weights/random_init.py)."""
    _dev(out)
    assert out.is_contiguous()
    _call("pl_fill_random", _p(out), out.numel(), _code(out.dtype), seed, tensor_hash, float(scale), float(offset),
          _stream())


def bf16_to_f32(src: torch.Tensor, dst: torch.Tensor) -> None:
    _dev(src, dst)
    assert src.dtype == torch.bfloat16 and dst.dtype == torch.float32 and src.numel() == dst.numel()
    assert src.is_contiguous() and dst.is_contiguous()
    _call("pl_bf16_to_f32", _p(src), _p(dst), src.numel(), _stream())


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T in true fp32 (CUDA-core FMA)."""
    _dev(a, w, out)
    assert a.dtype == w.dtype == out.dtype == torch.float32
    assert a.dim() == 2 and w.dim() == 2 and out.dim() == 2
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _call("pl_gemm_f32", _p(a), _p(w), _p(out), m, n, k, a.stride(0) if m > 1 else k, w.stride(0) if n > 1 else k,
          out.stride(0) if m > 1 else n, int(accumulate), _stream())


def gemm_bf16_supports(t: int, n: int, k: int, ldx: int, ldw: int) -> bool:
    """True when the tcgen05 products take these sizes: rows of both operands must start
    on 16 bytes (k and the leading dimensions multiples of 8)."""
    return bool(library().pl_gemm_bf16_pair_supports(t, n, k, ldx, ldw))


GEMM_SKINNY_MAX_TOKENS = 64


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor | None = None,
              kernel: str | None = None, gated: bool = False) -> None:
    """out[T, N] (bf16 or fp32) = x[T, K] @ w[N, K]^T on the tcgen05 tensor cores.

    Two kernels: "skinny" for up to 64 tokens (one tile and part of k per CTA, the parts
    added inside a thread-block cluster) and "pair" (256 x 256 tiles on pairs of SMs,
    any token count, meant for prompts). `kernel=None` picks by the token count.

    gated (pair only): w is [2N, K], a gate matrix over an up matrix, and
    out = silu(x gate^T) * (x up^T), both products rounded to bfloat16 first."""
    _dev(x, w, out, status)
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    t, k = x.shape
    n = w.shape[0] // 2 if gated else w.shape[0]
    assert w.shape[1] == k and out.shape == (t, n) and (not gated or w.shape[0] == 2 * n)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    ldx = x.stride(0) if t > 1 else k
    ldw = w.stride(0) if w.shape[0] > 1 else k
    if kernel is None:
        kernel = "skinny" if t <= GEMM_SKINNY_MAX_TOKENS and not gated else "pair"
    if kernel == "skinny":
        assert not gated, "only the pair kernel has the gated epilogue"
        _call("pl_gemm_bf16_skinny", _p(x), _p(w), _p(out), t, n, k, ldx, ldw, out.stride(0) if t > 1 else n,
              int(out.dtype == torch.float32), _p(status), _stream())
        return
    if kernel == "pair":
        _call("pl_gemm_bf16_pair", _p(x), _p(w), _p(out), t, n, k, ldx, ldw, out.stride(0) if t > 1 else n,
              int(out.dtype == torch.float32), int(gated), _p(status), _stream())
        return
    raise ValueError(f"gemm_bf16: unknown kernel {kernel!r}")

GEMM_GATED_IN_MAX_TOKENS = 16


def gemm_bf16_gated_in(gate_up: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                       status: torch.Tensor | None = None) -> None:
    """out[T, N] = (silu(g) * u) @ w[N, K]^T for gate_up = [g | u] of [T, 2K] (a gate/up
    projection's output): the skinny kernel forms the gated activation as it reads it
    (fp32, one rounding, the SwiGLU kernel's expression) and never writes it. T <= 16."""
    _dev(gate_up, w, out, status)
    assert gate_up.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    t, two_k = gate_up.shape
    n, k = w.shape
    assert two_k == 2 * k and out.shape == (t, n) and t <= GEMM_GATED_IN_MAX_TOKENS
    assert gate_up.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _call("pl_gemm_bf16_skinny_gated_in", _p(gate_up), _p(w), _p(out), t, n, k,
          gate_up.stride(0) if t > 1 else two_k, w.stride(0) if n > 1 else k, out.stride(0) if t > 1 else n,
          int(out.dtype == torch.float32), _p(status), _stream())


def rope_kv_write(q: torch.Tensor, k: torch.Tensor | None, v: torch.Tensor | None, pos: torch.Tensor,
                  entry: torch.Tensor, table: torch.Tensor, k_pool: torch.Tensor | None,
                  v_pool: torch.Tensor | None, page_size: int, inv_freq: torch.Tensor | None, rotary: int,
                  status: torch.Tensor | None = None, q_norm: torch.Tensor | None = None,
                  k_norm: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """Rotates q [T, nh, hd] in place and writes rotated k and v [T, nkv, hd] into
    the pools [pages, nkv, page_size, hd] (views of one layer's K and V). q_norm and
    k_norm (fp32 [hd]): each head of q, of k, is first normalised over its hd
    (x * rsqrt(mean(x^2) + norm_eps) * scale) in fp32."""
    _dev(q, k, v, pos, entry, table, k_pool, v_pool, inv_freq, status, q_norm, k_norm)
    for scale_ in (q_norm, k_norm):
        if scale_ is not None:
            assert scale_.dtype == torch.float32 and scale_.shape == (q.shape[2],) and scale_.is_contiguous()
    tokens, n_heads, head_dim = q.shape
    assert q.stride(2) == 1 and q.stride(1) == head_dim
    row_stride = q.stride(0)
    n_kv = n_heads
    page_stride = head_stride = n_pages = 0
    if k_pool is not None:
        assert k is not None and v is not None and v_pool is not None
        n_kv = k.shape[1]
        for t in (k, v):
            assert t.shape == (tokens, n_kv, head_dim) and t.stride(2) == 1 and t.stride(1) == head_dim
            assert (tokens == 1 or t.stride(0) == row_stride) and t.dtype == q.dtype
        n_pages = k_pool.shape[0]
        assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
        assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
        assert k_pool.dtype == q.dtype == v_pool.dtype
        page_stride, head_stride = k_pool.stride(0), k_pool.stride(1)
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    assert pos.numel() == tokens and entry.numel() == tokens and table.dim() == 2 and table.is_contiguous()
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary // 2 and inv_freq.is_contiguous()
    _call("pl_rope_kv_write", _p(q), _p(k), _p(v), row_stride, _p(pos), _p(entry), _p(table), table.shape[1],
          _p(k_pool), _p(v_pool), page_stride, head_stride, page_size, n_pages, _p(inv_freq), rotary, tokens,
          n_heads, n_kv, head_dim, _code(q.dtype), _p(q_norm), _p(k_norm), float(norm_eps), _p(status), _stream())


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                   pos: torch.Tensor, entry: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None,
                   scale: float, status: torch.Tensor | None = None, mass_sum: torch.Tensor | None = None,
                   weight_sum: torch.Tensor | None = None, query_weights: torch.Tensor | None = None,
                   softcap: float = 0.0) -> None:
    """Causal paged attention; q and out [T, nh, hd] (row strides free), pools
    [pages, nkv, page_size, hd]. With mass_sum fp32 [pages, nh] and weight_sum fp32
    [pages], the attention mass of every attended page is added to them
    (query_weights fp32 [T], all 1 when None). softcap > 0: scaled scores pass through
    softcap * tanh(s / softcap) before the softmax."""
    _dev(q, k_pool, v_pool, table, pos, entry, out, status, mass_sum, weight_sum, query_weights)
    if mass_sum is not None:
        assert mass_sum.dtype == torch.float32 and mass_sum.shape == (k_pool.shape[0], q.shape[1])
        assert mass_sum.is_contiguous() and weight_sum is not None and weight_sum.dtype == torch.float32
        assert weight_sum.shape == (k_pool.shape[0],) and weight_sum.is_contiguous()
        if query_weights is not None:
            assert query_weights.dtype == torch.float32 and query_weights.numel() == q.shape[0]
            assert query_weights.is_contiguous()
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape and out.dtype == q.dtype == k_pool.dtype == v_pool.dtype
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    assert table.dim() == 2 and table.is_contiguous()
    _call("pl_attention_simt", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0), k_pool.stride(1),
          page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out), out.stride(0), tokens,
          n_heads, n_kv, head_dim, int(window or 0), float(scale), float(softcap or 0.0), _code(q.dtype),
          _p(mass_sum), _p(weight_sum), _p(query_weights), _p(status), _stream())


def attention_decode_supports(head_dim: int, group: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core decode kernel takes this shape."""
    return bool(library().pl_attention_decode_supports(head_dim, group, page_size, DTYPE_CODE.get(dtype, -1)))


def attention_decode_scratch_floats(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(library().pl_attention_decode_scratch_floats(n_tokens, n_heads, head_dim, n_splits))


class _DecodeRope(ctypes.Structure):
    _fields_ = [("k_new", _PTR), ("v_new", _PTR), ("inv_freq", _PTR), ("rotary", _I32)]


def _decode_rope(rope: tuple | None, q: torch.Tensor, n_kv: int):
    """The PlDecodeRope argument of the decode attention calls from (k_new, v_new,
    inv_freq, rotary), or None. k_new, v_new [T, nkv, hd] share q's row stride (slices of
    one projection output); None for both when the layer writes no keys."""
    if rope is None:
        return None
    k_new, v_new, inv_freq, rotary = rope
    tokens, _, head_dim = q.shape
    _dev(k_new, v_new, inv_freq)
    assert rotary == head_dim and inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary // 2
    assert inv_freq.is_contiguous()
    for t in (k_new, v_new):
        if t is not None:
            assert t.dtype == q.dtype and t.shape == (tokens, n_kv, head_dim) and t.stride(2) == 1
            assert t.stride(1) == head_dim and (tokens == 1 or t.stride(0) == q.stride(0))
    return ctypes.byref(_DecodeRope(_p(k_new), _p(v_new), _p(inv_freq), int(rotary)))


_DECODE_COUNTERS: dict[torch.device, torch.Tensor] = {}
DECODE_COUNTERS = 1 << 20


def attention_decode_counters(device: torch.device) -> torch.Tensor:
    """The zeroed counters attention_decode_items works with (int32, DECODE_COUNTERS of
    them, one set per device: launches on one stream share it, each leaves it zero)."""
    device = torch.device(device)
    if device not in _DECODE_COUNTERS:
        _DECODE_COUNTERS[device] = torch.zeros(DECODE_COUNTERS, dtype=torch.int32, device=device)
    return _DECODE_COUNTERS[device]


def attention_decode_items(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                           pos: torch.Tensor, entry: torch.Tensor, out: torch.Tensor, page_size: int,
                           window: int | None, scale: float, items: torch.Tensor, token_slot: torch.Tensor,
                           scratch: torch.Tensor, status: torch.Tensor | None = None,
                           rope: tuple | None = None) -> None:
    """bf16 attention of single decode tokens over a work list (shapes as
    attention_decode). items: int32 [n, 4] rows {token, first 16-key tile, tiles, split |
    splits << 12}, rows of no tiles are padding; the rows of a token cover its tiles once.
    token_slot int32 [tokens]: first slot of a token's partial results in `scratch`
    (fp32, n * n_heads * (head_dim + 2) floats). The CTA that finishes a token's kv head
    last merges its splits in split order. `rope` as in attention_decode."""
    _dev(q, k_pool, v_pool, table, pos, entry, out, items, token_slot, scratch, status)
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == k_pool.dtype == out.dtype
    assert k_pool.shape == v_pool.shape and k_pool.stride() == v_pool.stride()
    assert k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert table.dtype == torch.int32 and table.is_contiguous() and pos.dtype == torch.int32 == entry.dtype
    assert pos.numel() == tokens == entry.numel() == token_slot.numel()
    assert items.dtype == torch.int32 == token_slot.dtype and items.dim() == 2 and items.shape[1] == 4
    assert items.is_contiguous() and token_slot.is_contiguous()
    n_items = items.shape[0]
    assert scratch.dtype == torch.float32 and scratch.is_contiguous()
    assert scratch.numel() >= n_items * n_heads * (head_dim + 2)
    if 2 + tokens * n_kv > DECODE_COUNTERS:
        raise KernelError(f"attention_decode_items: {tokens} tokens x {n_kv} kv heads need more than "
                          f"{DECODE_COUNTERS} counters")
    counters = attention_decode_counters(q.device)
    _call("pl_attention_decode_items", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0),
          k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out),
          out.stride(0), tokens, n_heads, n_kv, head_dim, int(window or 0), float(scale), _p(items), n_items,
          _p(token_slot), _p(scratch), _p(counters), _decode_rope(rope, q, n_kv), _p(status), _stream())


def attention_decode_ctas_per_sm(head_dim: int) -> int:
    """How many CTAs of the decode attention kernel an SM holds at once."""
    return int(library().pl_attention_decode_ctas_per_sm(head_dim))


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                     pos: torch.Tensor, entry: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None,
                     scale: float, n_splits: int, scratch: torch.Tensor | None,
                     status: torch.Tensor | None = None, mass: tuple | None = None,
                     rope: tuple | None = None) -> None:
    """bf16 attention of single decode tokens, split over the keys `n_splits` ways;
    shapes as attention_simt. `scratch`: fp32, attention_decode_scratch_floats long.
    `mass` = (tile_max, mass_sum, weight_sum, decay): also measures attention mass.
    tile_max is fp32 scratch of tokens * heads * (table width * page_size / 16) floats;
    mass_sum fp32 [pages, nh] and weight_sum fp32 [pages] are the running accumulators:
    what the request's pages hold is scaled by 1 - decay (the page the token opens
    restarts at zero) and decay * (the token's largest scaled score in the page), per
    head, and decay, per page, are added.
    `rope` = (k_new, v_new, inv_freq, rotary): q is unrotated; the kernel rotates it as it
    loads it, and rotates and stores each token's new key (with its value) at the token's
    place in the pools before reading it: the position encoding and the cache write
    folded into the attention (whole-head rotation only; not together with `mass`)."""
    _dev(q, k_pool, v_pool, table, pos, entry, out, scratch, status)
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == out.dtype == k_pool.dtype == v_pool.dtype
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    assert table.dim() == 2 and table.is_contiguous() and pos.numel() == tokens == entry.numel()
    if n_splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
        assert scratch.numel() >= attention_decode_scratch_floats(tokens, n_heads, head_dim, n_splits)
    if mass is not None:
        assert rope is None, "the mass-measuring call does not fold the position encoding in"
        tile_max, mass_sum, weight_sum, decay = mass
        max_tiles = table.shape[1] * page_size // 16
        _dev(tile_max, mass_sum, weight_sum)
        assert tile_max.dtype == torch.float32 and tile_max.is_contiguous()
        assert tile_max.numel() >= tokens * n_heads * max_tiles
        assert mass_sum.dtype == torch.float32 and mass_sum.shape == (n_pages, n_heads) and mass_sum.is_contiguous()
        assert weight_sum.dtype == torch.float32 and weight_sum.shape == (n_pages,) and weight_sum.is_contiguous()
        _call("pl_attention_decode_mass", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0),
              k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out),
              out.stride(0), tokens, n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits),
              _p(scratch), _p(tile_max), max_tiles, _p(mass_sum), _p(weight_sum), float(decay), _p(status),
              _stream())
        return
    _call("pl_attention_decode", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0), k_pool.stride(1),
          page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out), out.stride(0), tokens,
          n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits), _p(scratch),
          _decode_rope(rope, q, n_kv), _p(status),
          _stream())


def attention_prefill_supports(head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core kernel for prompt portions takes this shape."""
    return bool(library().pl_attention_prefill_supports(head_dim, page_size, DTYPE_CODE.get(dtype, -1)))


def attention_prefill_tile_rows() -> int:
    return int(library().pl_attention_prefill_tile_rows())


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                      tiles: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None, scale: float,
                      status: torch.Tensor | None = None) -> None:
    """bf16 causal attention of prompt portions. tiles int32 [n, 4]: {first token
    row, rows, position of the first row, block-table row}; q, out [T, nh, hd]."""
    _dev(q, k_pool, v_pool, table, tiles, out, status)
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == out.dtype == k_pool.dtype == v_pool.dtype
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 4 and tiles.is_contiguous()
    _call("pl_attention_prefill", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0), k_pool.stride(1),
          page_size, n_pages, _p(table), table.shape[1], _p(tiles), tiles.shape[0], _p(out), out.stride(0),
          n_heads, n_kv, head_dim, int(window or 0), float(scale), _p(status), _stream())


def attention_prefill_tcgen05_supports(q: torch.Tensor, k_pool: torch.Tensor, page_size: int) -> bool:
    """Whether the tcgen05 kernel for prompt portions takes this shape and cache layout."""
    return bool(library().pl_attention_prefill_tcgen05_supports(
        q.shape[2], page_size, k_pool.shape[1], k_pool.stride(0), k_pool.stride(1), q.stride(0),
        DTYPE_CODE.get(q.dtype, -1)))


PREFILL_SPLITS_MAX = 32


def attention_prefill_scratch_floats(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(library().pl_attention_prefill_scratch_floats(n_tokens, n_heads, head_dim, n_splits))


def attention_prefill_tcgen05_tile_rows(group: int) -> int:
    """The most rows of a tile that attention_prefill_tcgen05 takes with `wide=True` for
    this GQA group: 256 when the group is odd (a CTA then works on one head, and the
    two halves of a tile share its keys), else 128."""
    return int(library().pl_attention_prefill_tcgen05_tile_rows(group))


class _PrefillMass(ctypes.Structure):
    _fields_ = [("query_weights", _PTR), ("scratch", _PTR), ("pages", _I32), ("table_rows", _I32),
                ("step_mass", _PTR), ("step_weight", _PTR)]


def attention_prefill_tcgen05_measures_mass(group: int, page_size: int, wide: bool) -> bool:
    """Whether attention_prefill_tcgen05 can measure attention mass for this shape: two
    heads (an even group) or two halves of a wide tile per CTA, pages of 16, 32 or 64."""
    return (group % 2 == 0 or wide) and page_size in (16, 32, 64)


def attention_prefill_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                              tiles: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None,
                              scale: float, status: torch.Tensor | None = None, n_splits: int = 1,
                              scratch: torch.Tensor | None = None, wide: bool = False,
                              mass: tuple | None = None) -> None:
    """As attention_prefill, on the tcgen05 tensor cores. With n_splits > 1 every tile's
    keys are shared out over that many CTAs and merged through `scratch` (float32,
    attention_prefill_scratch_floats elements): for few tiles over many keys. `wide`: the
    tiles have up to attention_prefill_tcgen05_tile_rows(group) rows instead of 128.
    `mass` = (query_weights fp32 [T], step_mass fp32 [pages, nh], step_weight fp32
    [pages]): also adds to the step's attention mass: per page and head the sum over the
    query rows of weight * (the row's largest scaled score among the page's keys it
    attends), and per page the sum of the weights of the rows that attend it; the rows'
    sums are added in a fixed order (see attention_prefill_tcgen05_measures_mass)."""
    _dev(q, k_pool, v_pool, table, tiles, out, status, scratch)
    mass_arg = None
    if mass is not None:
        query_weights, step_mass, step_weight = mass
        _dev(query_weights, step_mass, step_weight)
        assert query_weights.dtype == torch.float32 and query_weights.numel() >= q.shape[0]
        assert query_weights.is_contiguous() and step_mass.is_contiguous() and step_weight.is_contiguous()
        assert step_mass.dtype == torch.float32 and step_mass.shape == (k_pool.shape[0], q.shape[1])
        assert step_weight.dtype == torch.float32 and step_weight.shape == (k_pool.shape[0],)
        pages = table.shape[1]
        mass_scratch = torch.zeros(tiles.shape[0] * q.shape[1] * 8 * pages, dtype=torch.float32, device=q.device)
        mass_arg = ctypes.byref(_PrefillMass(_p(query_weights), _p(mass_scratch), pages, table.shape[0],
                                             _p(step_mass), _p(step_weight)))
    if n_splits > 1:
        need = attention_prefill_scratch_floats(q.shape[0], q.shape[1], q.shape[2], n_splits)
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == out.dtype == k_pool.dtype == v_pool.dtype
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 4 and tiles.is_contiguous()
    _call("pl_attention_prefill_tcgen05", _p(q), q.stride(0), tokens, _p(k_pool), _p(v_pool), k_pool.stride(0),
          k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(tiles), tiles.shape[0], _p(out),
          out.stride(0), n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits), _p(scratch),
          int(wide), mass_arg, _p(status), _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor | None,
           top_p: torch.Tensor | None, seed: torch.Tensor, draw_count: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] (int32) = a token drawn from row r of fp32 logits [R, V]."""
    _dev(logits, temperature, top_k, top_p, seed, draw_count, out)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and temperature.numel() == rows
    assert seed.dtype == torch.int64 and draw_count.dtype == torch.int64 and out.dtype == torch.int32
    assert seed.numel() == rows and draw_count.numel() == rows and out.numel() == rows
    if top_k is not None:
        assert top_k.dtype == torch.int32 and top_k.numel() == rows
    if top_p is not None:
        assert top_p.dtype == torch.float32 and top_p.numel() == rows
    _call("pl_sample", _p(logits), logits.stride(0) if rows > 1 else vocab, rows, vocab, _p(temperature),
          _p(top_k), _p(top_p), _p(seed), _p(draw_count), _p(out), _stream())
