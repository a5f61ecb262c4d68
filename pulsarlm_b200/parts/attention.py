"""The attention mixer: grouped-query causal attention over the paged cache."""

from __future__ import annotations

import dataclasses
import math
import os

import numpy as np
import torch

from ..kernels import ops
from ..kernels.device import describe as describe_device
from .linear import linear
from .registry import BuildContext, Part, build_part, register_part
from .spec import KVCacheNeed, PartSpec, TensorNeed


@dataclasses.dataclass
class KVBinding:
    """What the cache manager hands a mixer that asked for a KVCacheNeed: this
    layer's key and value pools [pages, n_kv_heads, page_size, head_dim] and the
    group whose block table (`batch.tables[group]`) indexes them."""

    group: int
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    page_size: int
    # This step's attention mass [pages, n_heads] and weights [pages] of the layer,
    # when the cache manager measures it (else None).
    mass_sum: torch.Tensor | None = None
    weight_sum: torch.Tensor | None = None
    # The running accumulators themselves [pages, n_heads] and [pages], and the decay: the
    # tensor-core decode kernel folds a step's mass into them on the device.
    mass_total: torch.Tensor | None = None
    weight_total: torch.Tensor | None = None
    mass_decay: float | None = None


_SM_COUNT: dict = {}


_CLUSTER_ROOM: dict[tuple, int] = {}


def _cluster_room(device: torch.device, head_dim: int, group: int, splits: int) -> int:
    key = (device, head_dim, group, splits)
    if key not in _CLUSTER_ROOM:
        _CLUSTER_ROOM[key] = ops.library().pl_attention_decode_resident_clusters(head_dim, group, splits)
    return _CLUSTER_ROOM[key]


def decode_splits(n_ctas: int, max_context: int, device: torch.device, head_dim: int = 128, group: int = 4) -> int:
    """(Remembered per argument list: every layer of a step asks the same question.)"""
    key = (n_ctas, max_context, device, head_dim, group)
    if key not in _DECODE_SPLITS:
        if len(_DECODE_SPLITS) > 4096:
            _DECODE_SPLITS.clear()
        _DECODE_SPLITS[key] = _decode_splits(*key)
    return _DECODE_SPLITS[key]


_DECODE_SPLITS: dict[tuple, int] = {}


def _decode_splits(n_ctas: int, max_context: int, device: torch.device, head_dim: int, group: int) -> int:
    """Ways to split each request's keys among CTAs (`n_ctas` = tokens x kv heads without
    splits): the count with the least estimated time. The CTAs of a launch run in rounds
    of what the device holds at once (two CTAs per SM; with splits, the thread-block
    clusters that fit); a round streams at the memory's bandwidth if it has CTAs enough
    and at one CTA's own rate times their number if it has few, so few long CTAs, and a
    sparse last round of them, are what splitting avoids. The rates and fixed costs are the
    device description's (kernels/device.py: measured with this kernel, they reproduce its
    times at batch 1 to 64 within a tenth). No split shorter than eight 16-key tiles."""
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    # what the device holds of the kernel at once: two CTAs per SM at head sizes above 64, four below
    slots = (4 if head_dim <= 64 else 2) * _SM_COUNT[device]
    most = max(1, min(-(-max_context // 16) // 8, max(16, slots // max(1, n_ctas))))
    key_bytes = 4.0 * head_dim  # K and V of one key and kv head

    dev = describe_device(device)
    # (a CTA's own rate is the bytes its warps keep in flight over the memory's answer time:
    # measured at head size 128, half of that with rows half as long)
    cta_rate = dev.cta_bytes_per_second * min(1.0, head_dim / 128)

    def round_seconds(ctas: int, bytes_each: float, rate: float) -> float:
        return ctas * bytes_each / min(dev.stream_bytes_per_second, ctas * rate) + dev.round_seconds

    best, best_cost = 1, float("inf")
    for splits in range(most, 0, -1):  # on a tie, the finer split
        if splits == 1:
            room = slots
        elif splits <= 16:
            clusters = _cluster_room(device, head_dim, group, splits) or slots // splits
            if splits > 4:  # (clusters of up to four CTAs all find their room inside a step, larger ones do not)
                clusters = max(1, int(clusters * (1.0 - dev.cluster_room_loss_per_cta * splits)))
            room = clusters * splits
        else:
            room = slots
        total = n_ctas * splits
        bytes_each = max_context / splits * key_bytes
        rate = cta_rate * (dev.scratch_cta_fraction if splits > 16 else 1.0)
        cost = (total // room) * round_seconds(room, bytes_each, rate)
        if total % room:
            cost += round_seconds(total % room, bytes_each, rate)
        if splits > 1:
            cost += (dev.cluster_merge_seconds if splits <= 16
                     else dev.merge_kernel_seconds + splits * dev.merge_split_seconds)
        if cost < best_cost:
            best, best_cost = splits, cost
    return best


_CTAS_PER_SM: dict[tuple, int] = {}
DECODE_ITEM_MIN_TILES = 32     # no work item much shorter than 32 16-key tiles (a warp's ring must fill)
DECODE_ITEMS_PER_SLOT = 1      # unequal requests are cut into about this many items per resident CTA
DECODE_ITEMS = os.environ.get("PULSARLM_B200_DECODE_ITEMS", "1") != "0"  # (0: equal shares only, for comparison)
FOLD_ROPE = os.environ.get("PULSARLM_B200_FOLD_ROPE", "1") != "0"  # (0: always the separate rotation kernel)
FOLD_ROPE_SPLITS = (2, 8)      # the rotation is folded into the decode kernel where the keys go in this many shares
DECODE_EVEN_ENOUGH = 1.3       # longest / mean length up to which nothing is cut
DECODE_ITEMS_MOST_SPLITS = 3   # unequal requests walk a work list where equal shares would split in up to this many


def _uneven(context_lens) -> bool:
    """Whether the longest request is more than DECODE_EVEN_ENOUGH times the mean."""
    n = len(context_lens)
    return n > 1 and max(context_lens) * n > DECODE_EVEN_ENOUGH * sum(context_lens)


def decode_item_ctas(device: torch.device, head_dim: int, n_kv: int) -> int:
    """How many CTAs per kv head walk a work list: what the device holds at once of the
    decode kernel, over the kv heads (the kernel launches the same number)."""
    key = (device, head_dim)
    if key not in _CTAS_PER_SM:
        _CTAS_PER_SM[key] = max(1, ops.attention_decode_ctas_per_sm(head_dim))
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return max(1, -(-_CTAS_PER_SM[key] * _SM_COUNT[device] // n_kv))


def decode_work_items(context_lens: list[int], window: int | None, target: int, pad_to: int | None = None,
                      min_tiles: int = DECODE_ITEM_MIN_TILES, leave_even: bool = True) -> tuple[np.ndarray, np.ndarray]:
    """The work list of a step's single tokens for ops.attention_decode_items: int32
    [items, 4] rows {token, first 16-key tile, tiles, split | splits << 12}, longest first,
    and int32 [tokens] first scratch slot of each token's splits. Requests of about equal
    length (longest within DECODE_EVEN_ENOUGH of the mean) are not cut: one item each
    (unless `leave_even` is off: few requests, which need cutting to fill the device).
    Else the tiles are cut into about `target` items of equal size, a request's share
    rounded to whole items, so that the CTAs in flight stay many until the end instead of
    the longest requests streaming alone. At most target + tokens items; `pad_to` pads the
    list with empty rows to a fixed length (the last row then holds the count of real
    rows). Made by the host core (csrc_host/host_core.cpp: plh_decode_work_items)."""
    from ..host import core

    n = len(context_lens)
    lengths = np.asarray(context_lens, dtype=np.int32)
    capacity = max(pad_to or 0, target + n, 1)
    items = np.empty((capacity, 4), dtype=np.int32)
    slots = np.empty(max(n, 1), dtype=np.int32)
    used = core.library().plh_decode_work_items(
        lengths.ctypes.data, n, int(window or 0), int(target), int(min_tiles),
        int(round(DECODE_EVEN_ENOUGH * 100)) if leave_even else 0,
        items.ctypes.data, capacity, slots.ctypes.data)
    if used < 0:
        raise ValueError(f"decode_work_items: the host core refused the list (code {used})")
    return items[: max(pad_to or 0, used, 1)], slots[:n]


def prefill_splits(n_ctas: int, max_keys: int, n_tokens: int, n_heads: int, head_dim: int,
                   device: torch.device) -> int:
    """Ways to split every prompt tile's keys when the tiles alone (`n_ctas` CTAs, one per
    SM) leave SMs idle: a short portion of a long prompt. Picks the count with the least
    estimated time: rounds of CTAs, each a fixed start plus its share of the keys, plus
    what the partial rows cost to write and merge; the constants are the device
    description's (kernels/device.py: measurements of the kernel at head size 128). Splits
    only if that saves a tenth."""
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    sms = _SM_COUNT[device]
    most = min(max_keys // 256, 16, ops.PREFILL_SPLITS_MAX)
    if n_ctas <= 0 or n_ctas >= sms or most < 2:
        return 1
    dev = describe_device(device)
    # (a key's softmax costs the same at every head size, only its share of the products shrinks:
    # measured 15 ns a key at head size 64 against 17.3 at 128)
    per_key = dev.prefill_key_seconds * (0.75 + 0.25 * head_dim / 128)

    def cost(splits: int) -> float:
        rounds = -(-n_ctas * splits // sms)
        seconds = rounds * (dev.prefill_round_seconds + max_keys / splits * per_key)
        if splits > 1:
            seconds += dev.prefill_merge_seconds + (n_tokens * n_heads * splits * (head_dim + 2) * 8
                                                    / dev.prefill_scratch_bytes_per_second)
        return seconds

    best = min(range(1, most + 1), key=cost)
    return best if cost(best) < 0.9 * cost(1) else 1


@register_part("mixer", "attention")
class Attention(Part):
    """q, k, v projections (bias-free), position encoding on q and k, causal
    softmax attention with scale (default 1/sqrt(head_dim)) where query head h
    reads kv head h // (n_heads / n_kv_heads), then the o projection
    (pulsarlm-core/src/engine/model/llama.cpp:61-82).

    params: hidden_size, n_heads, n_kv_heads, head_dim, position (a PartSpec of the
    "position" registry), scale (optional), window (optional: a query reads only
    the last `window` keys), cache_from (optional: index of the layer whose cache
    this layer reads; it then has no k and v projections and writes nothing),
    softcap (optional: scaled scores pass through softcap * tanh(s / softcap) before
    the softmax; such a layer attends on the CUDA-core kernel, the only one that
    squashes scores), qk_norm_eps (with the q_norm / k_norm tensors: eps of the
    per-head RMS norm applied to q and k before the position encoding).
    tensors: q [nh*hd, H], k and v [nkv*hd, H], o [H, nh*hd]; optional q_norm and
    k_norm [hd] (kept in float32). q, k and v are stacked into one operand at load.
    """

    def __init__(self, spec: PartSpec, ctx: BuildContext):
        super().__init__(spec, ctx)
        p = spec.params
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.n_kv = int(self.param("n_kv_heads"))
        self.head_dim = int(self.param("head_dim"))
        if self.n_heads % self.n_kv:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(p["window"]) if p.get("window") else None
        self.cache_from = p.get("cache_from")
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.qk_norm_eps = float(p.get("qk_norm_eps") or 0.0)
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None
        self.position = build_part("position", self.param("position"), ctx)
        self.qkv: torch.Tensor | None = None
        self.o: torch.Tensor | None = None
        self.cache: KVBinding | None = None
        self._decode_kernel: bool | None = None
        self._prefill_kernel: bool | None = None
        self._prefill_tcgen05: bool | None = None

    @classmethod
    def tensor_needs(cls, spec: PartSpec) -> dict[str, TensorNeed]:
        p, t = spec.params, spec.tensors
        h, nh, nkv, hd = (int(p[k]) for k in ("hidden_size", "n_heads", "n_kv_heads", "head_dim"))
        needs = {t["q"]: TensorNeed((nh * hd, h)), t["o"]: TensorNeed((h, nh * hd))}
        if p.get("cache_from") is None:
            needs[t["k"]] = TensorNeed((nkv * hd, h))
            needs[t["v"]] = TensorNeed((nkv * hd, h))
            if t.get("k_norm"):
                needs[t["k_norm"]] = TensorNeed((hd,), role="vector")
        if t.get("q_norm"):
            needs[t["q_norm"]] = TensorNeed((hd,), role="vector")
        return needs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        t = self.spec.tensors
        if self.cache_from is None:
            self.qkv = torch.cat([tensors[t["q"]], tensors[t["k"]], tensors[t["v"]]], dim=0).contiguous()
        else:
            self.qkv = tensors[t["q"]].contiguous()
        self.o = tensors[t["o"]].contiguous()
        if t.get("q_norm"):
            self.q_norm = tensors[t["q_norm"]].float().contiguous()
        if t.get("k_norm") and self.cache_from is None:
            self.k_norm = tensors[t["k_norm"]].float().contiguous()

    def cache_need(self) -> KVCacheNeed | None:
        if self.cache_from is not None:
            return None
        return KVCacheNeed(self.n_kv, self.head_dim, self.window, self.n_heads)

    def cache_read_need(self) -> KVCacheNeed:
        """How this layer reads a cache, its own or the one `cache_from` names."""
        return KVCacheNeed(self.n_kv, self.head_dim, self.window, self.n_heads)

    def bind_cache(self, binding: KVBinding) -> None:
        self.cache = binding

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        tokens = h.shape[0]
        nh, nkv, hd = self.n_heads, self.n_kv, self.head_dim
        cache = self.cache
        table = batch.tables[cache.group]
        qkv = linear(h, self.qkv)
        q = qkv[:, : nh * hd].view(tokens, nh, hd)
        inv_freq, rotary = self.position.table()
        if self._folds_rope(tokens, batch, inv_freq, rotary):
            # Single tokens only, all for the tensor-core decode kernel: it rotates q as it loads
            # it and stores each token's rotated key and value itself, one launch fewer.
            rope = (qkv[:, nh * hd : (nh + nkv) * hd].view(tokens, nkv, hd),
                    qkv[:, (nh + nkv) * hd :].view(tokens, nkv, hd), inv_freq, rotary)
            out = torch.empty((tokens, nh, hd), dtype=h.dtype, device=h.device)
            self.attend(q, out, table, batch, rope)
            return linear(out.view(tokens, nh * hd), self.o)
        if self.cache_from is None:
            k = qkv[:, nh * hd : (nh + nkv) * hd].view(tokens, nkv, hd)
            v = qkv[:, (nh + nkv) * hd :].view(tokens, nkv, hd)
            ops.rope_kv_write(q, k, v, batch.pos, batch.entry, table, cache.k_pool, cache.v_pool, cache.page_size,
                              inv_freq, rotary, batch.status, self.q_norm, self.k_norm, self.qk_norm_eps)
        else:
            ops.rope_kv_write(q, None, None, batch.pos, batch.entry, table, None, None, cache.page_size, inv_freq,
                              rotary, batch.status, self.q_norm, None, self.qk_norm_eps)
        out = torch.empty((tokens, nh, hd), dtype=h.dtype, device=h.device)
        self.attend(q, out, table, batch)
        return linear(out.view(tokens, nh * hd), self.o)

    def _folds_rope(self, tokens: int, batch, inv_freq, rotary: int) -> bool:
        """Whether this step's position encoding and cache write go into the decode
        attention kernel: a step of single tokens that all take that kernel, a layer with a
        cache of its own, whole-head rotation, no q/k norm, no score cap, no mass measured,
        and a launch of few, short CTAs (the keys in 2 to 8 equal shares; or a work list at
        head sizes up to 64). There the launch
        saved counts (Llama-3.1-8B shape at batch 8: 3.350 -> 3.321 ms a step, batch 16 1.7 %;
        1B shape at batch 8 4 %); every CTA rotates q for itself, which costs more than the
        rotation kernel where CTAs are many or take several (token, kv head) pairs in turn
        (8B shape at batch 64 10,280 against 10,460 tokens/s, 13B shape at batch 32 3.4 %),
        and at batch 1, where sixteen CTAs rotate the same q (338 against 342 tokens/s)."""
        if not FOLD_ROPE or int(batch.n_decode) != tokens or self.cache_from is not None or inv_freq is None:
            return False
        if rotary != self.head_dim or self.q_norm is not None or self.k_norm is not None or self.softcap:
            return False
        if self.head_dim % 32 != 0:  # (the kernel rotates q in its fragments: pairs must not straddle one)
            return False
        if self.cache.mass_sum is not None:
            return False
        if not self._kernels(self.ctx.dtype)[0]:
            return False
        plan = batch.plans.get(self.plan_key()) or {}
        if plan.get("decode_items") is not None:
            # Over a work list: where an SM holds four CTAs of the kernel (head sizes up to 64) the
            # others stream while one rotates (Llama-3.2-1B shape with 300 to 4,500 keys, 16 layers:
            # batch 32 1,458 -> 1,404 us a step, batch 48 1,736 -> 1,644, batch 64 unchanged); with two
            # per SM it does not pay (8B shape at batch 32 and 64: 0.2 - 0.4 % slower).
            return self.head_dim <= 64
        max_context = plan.get("max_context") or max(batch.host_context_lens[:tokens])
        if self.window:
            max_context = min(max_context, self.window + 16)
        splits = decode_splits(tokens * self.n_kv, max_context, self.ctx.device, self.head_dim,
                               self.n_heads // self.n_kv)
        return FOLD_ROPE_SPLITS[0] <= splits <= FOLD_ROPE_SPLITS[1]

    def native_choice(self, tokens: int, batch, row_stride: int) -> dict | None:
        """What `attend` would decide for this step, as plain values, for a caller that
        launches the kernels itself (the block's native layer call): the number of leading
        single tokens, whether the position encoding is folded in, the work list or the
        split count of the decode kernel, the tile list, width and split count of the tcgen05
        prompt kernel, and the fp32 scratch each needs. None when the step needs anything
        else (another kernel, mass, a score cap, q/k norms, another layer's cache): the
        caller then leaves the layer to `forward`. `row_stride`: elements between the tokens'
        rows of q."""
        cache = self.cache
        if cache is None or self.softcap or self.cache_from is not None or self.q_norm is not None \
                or self.k_norm is not None or cache.mass_sum is not None:
            return None
        dtype = self.ctx.dtype
        decode_kernel, prefill_kernel = self._kernels(dtype)
        if not decode_kernel:
            return None
        plan = batch.plans.get(self.plan_key()) or {}
        n_decode = min(int(batch.n_decode), tokens)
        inv_freq, rotary = self.position.table()
        choice = {"n_decode": n_decode, "fold_rope": self._folds_rope(tokens, batch, inv_freq, rotary), "items": None,
                  "slots": None, "decode_splits": 1, "decode_scratch": 0, "tiles": None, "wide": False,
                  "prefill_splits": 1, "prefill_scratch": 0}
        group = self.n_heads // self.n_kv
        if n_decode > 0 and plan.get("decode_items") is not None:
            choice["items"], choice["slots"] = plan["decode_items"], plan["decode_slots"]
            choice["decode_scratch"] = plan["decode_items"].shape[0] * self.n_heads * (self.head_dim + 2)
        elif n_decode > 0:
            max_context = plan.get("max_context") or max(batch.host_context_lens[:n_decode])
            if self.window:
                max_context = min(max_context, self.window + 16)
            splits = decode_splits(n_decode * self.n_kv, max_context, self.ctx.device, self.head_dim, group)
            choice["decode_splits"] = splits
            choice["decode_scratch"] = ops.attention_decode_scratch_floats(n_decode, self.n_heads, self.head_dim, splits)
        if n_decode < tokens:
            tiles = plan.get("tiles")
            if not prefill_kernel or tiles is None or n_decode != int(batch.n_decode):
                return None
            if self._prefill_tcgen05 is None or not self._prefill_tcgen05:
                supported = ops.library().pl_attention_prefill_tcgen05_supports(
                    self.head_dim, cache.page_size, self.n_kv, cache.k_pool.stride(0), cache.k_pool.stride(1),
                    row_stride, ops.DTYPE_CODE.get(dtype, -1))
                if not supported:
                    return None
            wide = group % 2 == 1 and plan.get("tiles_wide") is not None
            if wide:
                tiles = plan["tiles_wide"]
            ctas = tiles.shape[0] * (self.n_heads if wide or group % 2 else self.n_heads // 2)
            max_keys = int(plan.get("max_keys") or 0)
            if self.window:
                max_keys = min(max_keys, self.window + ops.attention_prefill_tile_rows())
            splits = prefill_splits(ctas, max_keys, tokens - n_decode, self.n_heads, self.head_dim, self.ctx.device)
            choice.update(tiles=tiles, wide=wide, prefill_splits=splits,
                          prefill_scratch=ops.attention_prefill_scratch_floats(tokens, self.n_heads, self.head_dim,
                                                                               splits))
        return choice

    # ------------------------------------------------------------------ planning a step
    def _kernels(self, dtype: torch.dtype) -> tuple[bool, bool]:
        """Whether the tensor-core kernels for single tokens and for prompt portions take
        this layer's shape (asked once)."""
        if self._decode_kernel is None:
            self._decode_kernel = ops.attention_decode_supports(
                self.head_dim, self.n_heads // self.n_kv, self.cache.page_size, dtype)
            self._prefill_kernel = ops.attention_prefill_supports(self.head_dim, self.cache.page_size, dtype)
        return self._decode_kernel, self._prefill_kernel

    def slow_path_note(self) -> str | None:
        """A sentence for the user when this layer's shape keeps bfloat16 attention off the
        tensor-core kernels (it then runs on the CUDA-core kernel: right, but several times
        slower), else None. float32 attends on CUDA cores by design."""
        if self.cache is None or self.ctx.dtype != torch.bfloat16:
            return None
        decode_kernel, prefill_kernel = self._kernels(self.ctx.dtype)
        if self.softcap:
            return (f"attention with a score cap ({self.softcap:g}) runs on the CUDA-core attention kernel, the "
                    f"only one that squashes scores; expect it several times slower than uncapped attention")
        if decode_kernel and prefill_kernel:
            return None
        return (f"attention with head size {self.head_dim}, {self.n_heads // self.n_kv} query heads per kv head and "
                f"pages of {self.cache.page_size} tokens runs on the CUDA-core attention kernel (the tensor-core "
                f"kernels take head sizes 32 to 128 in steps of 16, groups up to 16 and pages that are multiples of 16 tokens); "
                f"expect it several times slower")

    def measures_mass_in_captured_steps(self) -> bool:
        """Whether this layer can measure attention mass inside a captured decode step
        (the tensor-core decode kernel takes its shape and it has no score cap)."""
        if self.cache is None or self.softcap:
            return False
        return self._kernels(self.ctx.dtype)[0]

    def plan_key(self):
        """Layers of equal tiling share one plan: the tile lists depend on the kernels'
        tile heights only (twice as high when a CTA works on one head: an odd group)."""
        if self.cache is None:
            return None
        wide = (self.n_heads // self.n_kv) % 2 == 1
        return ("attention", self.cache.page_size, self.head_dim, self.n_heads // self.n_kv, wide,
                self.ctx.dtype, bool(self.softcap), self.n_kv, self.window)

    def native_key(self):
        """What `native_choice` depends on beyond `plan_key`: layers that agree in both get
        the same answer for a step, so a caller may ask once for all of them."""
        inv_freq, rotary = self.position.table()
        return (self.n_heads, inv_freq is not None, int(rotary), self.q_norm is None, self.k_norm is None,
                self.cache_from is None, self.cache is not None and self.cache.mass_sum is not None)

    def plan_variant(self, step):
        """For a captured step of single tokens: "work list" when the requests' lengths
        differ and there are enough of them that equal shares would split in two or three
        only; such replays get a capture of their own, whose decode attention walks a work
        list (see plan_step). Else None."""
        decode_kernel, _ = self._kernels(self.ctx.dtype)
        if not decode_kernel or self.softcap or not DECODE_ITEMS or not step.n_decode:
            return None
        if self.cache.mass_sum is not None and self.cache_from is None:
            return None
        reach = min(step.context_bound, self.window + 16) if self.window else step.context_bound
        splits = decode_splits(step.n_decode * self.n_kv, reach, self.ctx.device, self.head_dim,
                               self.n_heads // self.n_kv)
        if 1 < splits <= DECODE_ITEMS_MOST_SPLITS and _uneven(self._keys_read(step.context_lens[: step.n_decode])):
            return "work list"
        return None

    def _keys_read(self, context_lens) -> list[int]:
        """How many keys a single token of each request reads (its history, or the window)."""
        return [min(c, self.window) for c in context_lens] if self.window else list(context_lens)

    def plan_step(self, step) -> dict:
        """The tile list of the prompt-portion kernels: int32 [tiles, 4] rows of {first
        token row, rows, position of the first row, block-table row}, the tiles that read
        the most keys first; `tiles_wide` the same in tiles twice as high (odd groups, and
        only when some portion is longer than one narrow tile); `max_keys` the most keys a
        tile reads; `max_context` the most keys a single decode token reads (in a step that
        is captured and replayed: the most it may come to read)."""
        decode_kernel, prefill_kernel = self._kernels(self.ctx.dtype)
        plan: dict = {"tiles": None, "tiles_wide": None, "max_keys": 0, "max_context": 0}
        if self.softcap:
            return plan  # every token goes to the CUDA-core kernel, which needs no plan
        n_decode = step.n_decode if decode_kernel else 0
        if n_decode:
            plan["max_context"] = step.context_bound if step.fixed_shape else max(step.context_lens[:n_decode])
            # Many single tokens (so many that their keys would not be split at all): a work
            # list cut by the requests' true lengths instead of one CTA per request and kv
            # head, unless attention mass is measured (that path keeps equal shares).
            measuring = self.cache.mass_sum is not None and self.cache_from is None
            device = self.ctx.device
            reach = min(plan["max_context"], self.window + 16) if self.window else plan["max_context"]
            # Also for fewer requests, where equal shares would split in two or three, when their
            # lengths differ (`_uneven`): batch 24 at head size 128 with 300 to 4,500 keys 55.6 -> 43.4
            # us, batch 12 29.2 -> 23.6; with equal lengths the shares in a cluster are ahead (batch 20
            # at 8,192 keys: 101 against 144 us), so a captured step is captured for either case
            # (`plan_variant`). Few requests with long histories keep their equal shares.
            splits = decode_splits(n_decode * self.n_kv, reach, device, self.head_dim, self.n_heads // self.n_kv)
            listed = splits == 1
            if 1 < splits <= DECODE_ITEMS_MOST_SPLITS:
                listed = (step.variants.get(self.plan_key()) == "work list" if step.fixed_shape
                          else _uneven(self._keys_read(step.context_lens[:n_decode])))
            if DECODE_ITEMS and not measuring and 2 + n_decode * self.n_kv <= ops.DECODE_COUNTERS and listed:
                ctas = decode_item_ctas(device, self.head_dim, self.n_kv)
                target = DECODE_ITEMS_PER_SLOT * ctas
                items, slots = decode_work_items(step.context_lens[:n_decode], self.window, target,
                                                 target + n_decode if step.fixed_shape else None)
                plan["decode_items"], plan["decode_slots"] = items, slots
        if not prefill_kernel or step.n_decode == step.n_entries:
            return plan
        rows = ops.attention_prefill_tile_rows()
        wide_rows = ops.attention_prefill_tcgen05_tile_rows(self.n_heads // self.n_kv)
        tiles, wide_tiles = [], []
        for e in range(step.n_decode, step.n_entries):
            n, at = step.query_lens[e], step.first_rows[e]
            start = step.context_lens[e] - n
            for r in range(0, n, rows):
                tiles.append((at + r, min(rows, n - r), start + r, e))
            if wide_rows > rows:
                for r in range(0, n, wide_rows):
                    wide_tiles.append((at + r, min(wide_rows, n - r), start + r, e))
        tiles.sort(key=lambda t: -(t[2] + t[1]))
        plan["tiles"] = np.array(tiles, dtype=np.int32).reshape(len(tiles), 4)
        plan["max_keys"] = max((t[2] + t[1] for t in tiles), default=0)
        if any(t[1] > rows for t in wide_tiles):
            wide_tiles.sort(key=lambda t: -(t[2] + t[1]))
            plan["tiles_wide"] = np.array(wide_tiles, dtype=np.int32).reshape(len(wide_tiles), 4)
        return plan

    def attend(self, q: torch.Tensor, out: torch.Tensor, table: torch.Tensor, batch, rope: tuple | None = None) -> None:
        """out = attention of q over the cache. The batch's leading `n_decode` tokens
        are single tokens of their requests: in bfloat16 they go to the split-key
        tensor-core kernel and prompt portions to the tiled tensor-core kernel (tcgen05
        when the cache layout allows TMA, else mma.sync) when those take the shape;
        everything else (float32, unusual shapes) goes to the CUDA-core kernel."""
        cache = self.cache
        tokens = q.shape[0]
        measuring = cache.mass_sum is not None and self.cache_from is None
        if measuring and batch.extras.get("graph") and self.measures_mass_in_captured_steps() \
                and int(batch.n_decode) == tokens:
            # A captured step of single tokens: the tensor-core kernel records every tile's
            # largest score and a second kernel folds them into the accumulators.
            max_context = (batch.plans.get(self.plan_key()) or {}).get("max_context") or 0
            if self.window:
                max_context = min(max_context, self.window + 16)
            splits = decode_splits(tokens * self.n_kv, max_context, q.device, self.head_dim, self.n_heads // self.n_kv)
            scratch = None
            if splits > 1:
                scratch = torch.empty(ops.attention_decode_scratch_floats(tokens, self.n_heads, self.head_dim, splits),
                                      dtype=torch.float32, device=q.device)
            tile_max = torch.empty(tokens * self.n_heads * (table.shape[1] * cache.page_size // 16),
                                   dtype=torch.float32, device=q.device)
            ops.attention_decode(q, cache.k_pool, cache.v_pool, table, batch.pos, batch.entry, out, cache.page_size,
                                 self.window, self.scale, splits, scratch, batch.status,
                                 mass=(tile_max, cache.mass_total, cache.weight_total, cache.mass_decay))
            return
        if measuring and batch.extras.get("query_weights") is not None:
            # Measuring attention mass in an eager step. Prompt portions: the tcgen05 kernel adds up
            # its rows' sums itself where it takes the shape; single tokens, and every shape it
            # does not take: the CUDA-core kernel, which writes mass beside its output.
            weights = batch.extras["query_weights"]
            plan = batch.plans.get(self.plan_key()) or {}
            n_single = min(int(batch.n_decode), tokens)
            group = self.n_heads // self.n_kv
            wide = group % 2 == 1 and plan.get("tiles_wide") is not None
            tiles = plan.get("tiles_wide") if wide else plan.get("tiles")
            fast = (not self.softcap and tiles is not None and n_single < tokens and self._kernels(q.dtype)[1]
                    and ops.attention_prefill_tcgen05_measures_mass(group, cache.page_size, wide)
                    and ops.attention_prefill_tcgen05_supports(q, cache.k_pool, cache.page_size))
            n_simt = n_single if fast else tokens
            if n_simt > 0:
                ops.attention_simt(q[:n_simt], cache.k_pool, cache.v_pool, table, batch.pos[:n_simt],
                                   batch.entry[:n_simt], out[:n_simt], cache.page_size, self.window, self.scale,
                                   batch.status, cache.mass_sum, cache.weight_sum, weights[:n_simt],
                                   softcap=self.softcap)
            if fast:
                ops.attention_prefill_tcgen05(q, cache.k_pool, cache.v_pool, table, tiles, out, cache.page_size,
                                              self.window, self.scale, batch.status, 1, None, wide,
                                              mass=(weights, cache.mass_sum, cache.weight_sum))
            return
        if self.softcap:
            ops.attention_simt(q, cache.k_pool, cache.v_pool, table, batch.pos, batch.entry, out, cache.page_size,
                               self.window, self.scale, batch.status, softcap=self.softcap)
            return
        plan = batch.plans.get(self.plan_key()) or {}
        decode_kernel, prefill_kernel = self._kernels(q.dtype)
        n_decode = min(int(batch.n_decode), tokens) if decode_kernel else 0
        if n_decode > 0 and plan.get("decode_items") is not None:
            items = plan["decode_items"]
            scratch = torch.empty(items.shape[0] * self.n_heads * (self.head_dim + 2), dtype=torch.float32,
                                  device=q.device)
            ops.attention_decode_items(q[:n_decode], cache.k_pool, cache.v_pool, table, batch.pos[:n_decode],
                                       batch.entry[:n_decode], out[:n_decode], cache.page_size, self.window,
                                       self.scale, items, plan["decode_slots"], scratch, batch.status, rope)
        elif n_decode > 0:
            max_context = plan.get("max_context") or max(batch.host_context_lens[:n_decode])
            if self.window:
                max_context = min(max_context, self.window + 16)
            splits = decode_splits(n_decode * self.n_kv, max_context, q.device, self.head_dim,
                                   self.n_heads // self.n_kv)
            scratch = None
            if splits > 1:
                scratch = torch.empty(ops.attention_decode_scratch_floats(n_decode, self.n_heads, self.head_dim,
                                                                          splits),
                                      dtype=torch.float32, device=q.device)
            ops.attention_decode(q[:n_decode], cache.k_pool, cache.v_pool, table, batch.pos[:n_decode],
                                 batch.entry[:n_decode], out[:n_decode], cache.page_size, self.window, self.scale,
                                 splits, scratch, batch.status, rope=rope)
        tiles = plan.get("tiles")
        if n_decode < tokens and prefill_kernel and tiles is not None and n_decode == int(batch.n_decode):
            # The tile list covers exactly the tokens after the leading single tokens.
            if self._prefill_tcgen05 is None:
                self._prefill_tcgen05 = ops.attention_prefill_tcgen05_supports(q, cache.k_pool, cache.page_size)
            if self._prefill_tcgen05:
                # Two heads of a kv head share a CTA when the group is even; else a CTA takes one
                # head, and a tile of twice the rows if the step has portions that long (the two
                # halves then share the keys; for shorter portions the narrow tiles are ahead).
                wide = (self.n_heads // self.n_kv) % 2 == 1 and plan.get("tiles_wide") is not None
                if wide:
                    tiles = plan["tiles_wide"]
                ctas = tiles.shape[0] * (self.n_heads if wide or (self.n_heads // self.n_kv) % 2 else self.n_heads // 2)
                max_keys = int(plan.get("max_keys") or 0)
                if self.window:
                    max_keys = min(max_keys, self.window + ops.attention_prefill_tile_rows())
                splits = prefill_splits(ctas, max_keys, tokens - n_decode, self.n_heads, self.head_dim, q.device)
                scratch = None
                if splits > 1:
                    scratch = torch.empty(ops.attention_prefill_scratch_floats(tokens, self.n_heads, self.head_dim,
                                                                               splits),
                                          dtype=torch.float32, device=q.device)
                ops.attention_prefill_tcgen05(q, cache.k_pool, cache.v_pool, table, tiles, out, cache.page_size,
                                              self.window, self.scale, batch.status, splits, scratch, wide)
            else:
                ops.attention_prefill(q, cache.k_pool, cache.v_pool, table, tiles, out, cache.page_size,
                                      self.window, self.scale, batch.status)
        elif n_decode < tokens:
            ops.attention_simt(q[n_decode:], cache.k_pool, cache.v_pool, table, batch.pos[n_decode:],
                               batch.entry[n_decode:], out[n_decode:], cache.page_size, self.window, self.scale,
                               batch.status)
