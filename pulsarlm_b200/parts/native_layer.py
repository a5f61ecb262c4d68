"""A decoder layer launched from one native call (csrc/block_forward.cu).

The pre-norm block's parts each launch their own kernels from Python; a step of a few
hundred launches then costs the host more than the device. When a block's norm, mixer
and feed-forward are the package's standard ones in bfloat16, the block hands the layer
to `pl_layer_forward` instead: the same entry points in the same order, launched from
C++. Everything that is a decision stays with the parts: this module asks the attention
part what it would do for the step (`native_choice`), the product route for each
projection (`linear.own_kernel_for`), and passes the answers on. Any other combination
of parts, dtype or step (mass being measured, a score cap, q/k norms, a layer reading
another's cache, a shape a kernel does not take) keeps the block's own path.
`PULSARLM_B200_NATIVE_LAYERS=0` switches it off.

The reference runs its layers from C++ (pulsarlm-core/src/engine/model/llama.cpp:61-94).
"""

from __future__ import annotations

import ctypes
import os

import torch

from ..kernels import ops
from . import linear

ENABLED = os.environ.get("PULSARLM_B200_NATIVE_LAYERS", "1") != "0"
# (0: the two attention kernels of a step with both kinds of tokens one after the other)
SIDE_BY_SIDE = os.environ.get("PULSARLM_B200_ATTENTION_SIDE_BY_SIDE", "1") != "0"

_PTR, _I32, _I64, _F32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


class LayerWeights(ctypes.Structure):
    _fields_ = [("mixer_norm", _PTR), ("ff_norm", _PTR), ("norm_dtype", _I32), ("eps", _F32),
                ("qkv", _PTR), ("o", _PTR), ("gate_up", _PTR), ("down", _PTR),
                ("hidden", _I32), ("n_heads", _I32), ("n_kv_heads", _I32), ("head_dim", _I32), ("inter", _I32),
                ("inv_freq", _PTR), ("rotary", _I32), ("scale", _F32), ("window", _I32),
                ("k_pool", _PTR), ("v_pool", _PTR), ("page_stride", _I64), ("head_stride", _I64),
                ("page_size", _I32), ("n_pages", _I32)]


class LayerStep(ctypes.Structure):
    _fields_ = [("x", _PTR), ("delta_in", _PTR), ("delta_out", _PTR), ("n_tokens", _I32), ("n_decode", _I32),
                ("pos", _PTR), ("entry", _PTR), ("table", _PTR), ("table_width", _I32), ("status", _PTR),
                ("h", _PTR), ("qkv", _PTR), ("attended", _PTR), ("mixed", _PTR), ("gate_up", _PTR), ("act", _PTR),
                ("route_qkv", _I32), ("route_o", _I32), ("route_gate_up", _I32), ("route_down", _I32),
                ("fold_rope", _I32), ("items", _PTR), ("n_items", _I32), ("item_slots", _PTR), ("counters", _PTR),
                ("decode_splits", _I32), ("decode_scratch", _PTR),
                ("tiles", _PTR), ("n_tiles", _I32), ("wide", _I32), ("prefill_splits", _I32),
                ("prefill_scratch", _PTR),
                ("library_workspace", _PTR), ("library_workspace_bytes", _I64), ("attention_side_by_side", _I32)]


ROUTES = {None: 0, "skinny": 1, "pair": 2}
ROUTE_PAIR_GATED = 3
ROUTE_SKINNY_GATED_IN = 4
_WORKSPACES: dict[torch.device, torch.Tensor] = {}
# (With 32 MB cuBLAS picked a slower kernel for a 256-token down projection of the 8B shape than
# with 8 MB, 37 against 30 us; 8 MB gives the choices torch's own calls get.)
LIBRARY_WORKSPACE_BYTES = 8 << 20


def library_workspace(device: torch.device) -> torch.Tensor:
    """The buffer cuBLAS works in when the native call runs a library product (one per
    device, made at first use, so that nothing is allocated while a stream is captured)."""
    if device not in _WORKSPACES:
        _WORKSPACES[device] = torch.empty(LIBRARY_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    return _WORKSPACES[device]


def _route(tokens: int, n: int, k: int, device: torch.device) -> int:
    """The route parts/linear.py gives a contiguous [tokens, k] x [n, k] product."""
    kernel = linear.own_kernel_for(tokens, n, device, k)
    if kernel is not None and not ops.gemm_bf16_supports(tokens, n, k, k, k):
        kernel = None
    return ROUTES[kernel]


def eligible(block) -> bool:
    """Whether the block's parts are the ones the native call strings together."""
    from .attention import Attention
    from .basic import GatedMLP, RMSNorm

    if not ENABLED or block.mixer_norm.ctx.dtype != torch.bfloat16:
        return False
    if type(block.mixer_norm) is not RMSNorm or type(block.ff_norm) is not RMSNorm:
        return False
    if type(block.mixer) is not Attention or type(block.feed_forward) is not GatedMLP:
        return False
    if block.mixer_norm.eps != block.ff_norm.eps or block.mixer_norm.weight.dtype != block.ff_norm.weight.dtype:
        return False
    mixer, ff = block.mixer, block.feed_forward
    if mixer.hidden != ff.hidden or mixer.hidden != block.mixer_norm.hidden:
        return False
    return all(t is not None and t.is_contiguous() for t in (mixer.qkv, mixer.o, ff.gate_up, ff.down))


def layer_weights(block) -> LayerWeights:
    """The layer's tensors and constants for the native call, with the cache the mixer is
    bound to at the moment."""
    mixer, ff, cache = block.mixer, block.feed_forward, block.mixer.cache
    inv_freq, rotary = mixer.position.table()
    norm = block.mixer_norm
    return LayerWeights(
        norm.weight.data_ptr(), block.ff_norm.weight.data_ptr(), ops.DTYPE_CODE[norm.weight.dtype], norm.eps,
        mixer.qkv.data_ptr(), mixer.o.data_ptr(), ff.gate_up.data_ptr(), ff.down.data_ptr(),
        mixer.hidden, mixer.n_heads, mixer.n_kv, mixer.head_dim, ff.inter,
        inv_freq.data_ptr() if inv_freq is not None else None, int(rotary), mixer.scale, int(mixer.window or 0),
        cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), cache.k_pool.stride(0), cache.k_pool.stride(1),
        cache.page_size, cache.k_pool.shape[0])


class StepState:
    """One step's struct and the tensors it points into, shared by the layers of one shape."""

    def __init__(self, block, x: torch.Tensor, batch):
        mixer, ff = block.mixer, block.feed_forward
        tokens, hidden = x.shape
        device = x.device
        qkv_width = (mixer.n_heads + 2 * mixer.n_kv) * mixer.head_dim
        q_width = mixer.n_heads * mixer.head_dim
        self.choice = mixer.native_choice(tokens, batch, qkv_width)
        if self.choice is None:
            return
        c = self.choice
        gate_up = linear.own_kernel_for(tokens, 2 * ff.inter, device, hidden)
        gated = gate_up == "pair" and ops.gemm_bf16_supports(tokens, ff.inter, hidden, hidden, hidden)
        # (as linear.gated_feed_forward decides: the down product makes the gated activation itself)
        gated_in = (linear.GATED_IN and not gated and tokens <= ops.GEMM_GATED_IN_MAX_TOKENS
                    and linear.own_kernel_for(tokens, hidden, device, ff.inter) == "skinny"
                    and ops.gemm_bf16_supports(tokens, hidden, ff.inter, 2 * ff.inter, ff.inter))
        # one bf16 buffer for the activations, carved into parts that start on 512 bytes
        sizes = [tokens * hidden, tokens * qkv_width, tokens * q_width, tokens * hidden,
                 0 if gated else tokens * 2 * ff.inter, tokens * ff.inter, tokens * hidden, tokens * hidden]
        starts, total = [], 0
        for size in sizes:
            starts.append(total)
            total += -(-size // 256) * 256
        self.buffer = torch.empty(max(total, 8), dtype=torch.bfloat16, device=device)
        views = [self.buffer[at : at + size] for at, size in zip(starts, sizes)]
        self.deltas = [views[6].view(tokens, hidden), views[7].view(tokens, hidden)]
        self.turn = 0
        decode_floats = -(-int(c["decode_scratch"]) // 128) * 128  # (the prompt kernel's part starts on 512 bytes)
        self.scratch = torch.empty(max(decode_floats + int(c["prefill_scratch"]), 4), dtype=torch.float32,
                                   device=device)
        table = batch.tables[mixer.cache.group]
        workspace = library_workspace(device)
        items, tiles = c["items"], c["tiles"]
        self.keep = (table, items, c["slots"], tiles, workspace)
        self.struct = LayerStep(
            x.data_ptr(), None, None, tokens, c["n_decode"], batch.pos.data_ptr(), batch.entry.data_ptr(),
            table.data_ptr(), table.shape[1], batch.status.data_ptr() if batch.status is not None else None,
            views[0].data_ptr(), views[1].data_ptr(), views[2].data_ptr(), views[3].data_ptr(),
            views[4].data_ptr() if not gated else None, views[5].data_ptr(),
            _route(tokens, qkv_width, hidden, device), _route(tokens, hidden, q_width, device),
            ROUTE_PAIR_GATED if gated else _route(tokens, 2 * ff.inter, hidden, device),
            ROUTE_SKINNY_GATED_IN if gated_in else _route(tokens, hidden, ff.inter, device),
            int(c["fold_rope"]), items.data_ptr() if items is not None else None,
            items.shape[0] if items is not None else 0, c["slots"].data_ptr() if items is not None else None,
            ops.attention_decode_counters(device).data_ptr() if items is not None else None,
            int(c["decode_splits"]), self.scratch.data_ptr(),
            tiles.data_ptr() if tiles is not None else None, tiles.shape[0] if tiles is not None else 0,
            int(c["wide"]), int(c["prefill_splits"]),
            self.scratch[decode_floats:].data_ptr(),
            workspace.data_ptr(), workspace.numel(), int(SIDE_BY_SIDE))
        # how many of the package's own kernels one call launches (library products are not ours)
        routes = (self.struct.route_qkv, self.struct.route_o, self.struct.route_gate_up, self.struct.route_down)
        self.launches = (2 + sum(1 for r in routes if r != 0) + (0 if c["fold_rope"] else 1)
                         + (1 if c["n_decode"] > 0 else 0)
                         + (1 if c["n_decode"] > 0 and items is None and c["decode_splits"] > 16 else 0)
                         + ((1 if c["prefill_splits"] == 1 else 2) if tiles is not None else 0)
                         + (0 if gated or gated_in else 1))


def forward(block, x: torch.Tensor, delta: torch.Tensor | None, batch):
    """The block's forward through the native call, or None when this step is not one it
    takes (the block then runs its parts itself)."""
    mixer = block.mixer
    if mixer.cache is None or x.dtype != torch.float32 or not x.is_contiguous():
        return None
    if delta is not None and (delta.dtype != torch.bfloat16 or not delta.is_contiguous()):
        return None
    key = ("native_layer", mixer.plan_key(), mixer.native_key(), mixer.hidden, block.feed_forward.inter, mixer.scale)
    states = batch.extras.setdefault("native_layers", {})
    state = states.get(key)
    if state is None:
        state = states[key] = StepState(block, x, batch)
    if state.choice is None:
        return None
    # The weights struct holds the cache's addresses: made anew when the mixer is bound elsewhere.
    bound = getattr(block, "_native_bound", None)
    if bound is None or bound[0] is not mixer.cache:
        block._native_bound = bound = (mixer.cache, layer_weights(block))
    step = state.struct
    step.x = x.data_ptr()
    step.delta_in = delta.data_ptr() if delta is not None else None
    out = state.deltas[state.turn]
    if delta is not None and out.data_ptr() == delta.data_ptr():
        state.turn ^= 1
        out = state.deltas[state.turn]
    state.turn ^= 1
    step.delta_out = out.data_ptr()
    ops.call_native("pl_layer_forward", ctypes.byref(bound[1]), ctypes.byref(step), launches=state.launches)
    return x, out
