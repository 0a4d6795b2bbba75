"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import HostBatch, Mixer, PagedKV, Plan, PreNormed
from .linear import Linear, SMS
from .registry import register_mixer, POSITION_ENCODINGS


# What a block of the tcgen05 attention kernel costs beside its key tiles (tensor memory, barriers, the chain of
# loads to its first keys, the pipeline's fill and the write of its rows), in key tiles of one pair of row tiles:
# with one block per SM a stream of n key tiles takes 7.5 + 1.03 n us, of which about 3 us are the launch, and a
# block that writes partial sums for the merge a few more.  The shortest piece of a stream that is worth a block of
# its own is as long.
SEGMENT_COST = 8.0
MIN_SEGMENT = 8
TO_THE_END = 1 << 30


def plan_segments(key_tiles, heads: int, sms: int = 0):
    """Which block takes which keys.  `key_tiles[p]` is the number of 64-key tiles in the stream of pair p of the
    tile list (two row tiles of a request, the same for every head).  An item is a (pair, head); normally one
    block takes one item, and the answer is None: the kernel's grid is (heads, pairs).  Where that would leave SMs
    idle for long (few items, each over a long stream: a portion of a prompt on top of thousands of tokens), all
    items' streams are laid end to end, heaviest first, and cut into `sms` equal ranges; a range's share of an item
    is a segment, one block.  Segments of a cut item write partial sums (slots), which a second kernel merges.

    Returns None (whole items: nothing to say) or (segments [n, 5] int32: pair, head, first key tile, key tiles
    (TO_THE_END for an item's last), slot or -1, longest first; items [m, 4] int32: pair, head, first slot, slots of
    the cut items; number of slots).  Every item's segments cover its stream exactly once whatever the kernel takes
    the stream's length to be: the first starts at 0 and the last runs to the end."""
    sms = sms or SMS
    pairs = len(key_tiles)
    if pairs == 0 or heads <= 0:
        return None
    n = pairs * heads
    total = heads * sum(key_tiles)
    # Whole items take as long as the longest one, or as all of them spread evenly, or as the items of the SM that
    # has most of them (some SM takes at least ceil(n / sms) items: the lightest ones at best).  Cut streams: equal
    # ranges, 1.4 blocks per SM on the average, and the merge.  (Measured: 81.5 against 64.5 us for 80 items of 68
    # key tiles, 372 against 90 us for 28 items of 514; 28.6 against 36.9 us for a whole prompt of 1,024 tokens,
    # which is not cut.)
    most, lightest = -(-n // sms), 0.0
    for tiles in sorted(key_tiles):
        lightest += min(most, heads) * (tiles + SEGMENT_COST)
        most -= min(most, heads)
        if most == 0:
            break
    whole = max(max(key_tiles) + SEGMENT_COST, (total + n * SEGMENT_COST) / sms, lightest)
    shortest = max(MIN_SEGMENT, 1)
    ranges = min(sms, total // (shortest + 1))        # (cuts are then at least `shortest` apart after rounding)
    if ranges <= 1 or whole <= 1.15 * (total / ranges + 2.4 * SEGMENT_COST):
        # (whole items of several requests listed longest first, instead of the grid's order, which is the
        # list's backwards: measured, 63.0 against 60.7 us for prompts of 512, 2,048, 256 and 1,024 tokens)
        return None
    lengths = np.asarray(key_tiles, dtype=np.int64)
    order = np.argsort(-lengths, kind="stable")
    size = np.repeat(lengths[order], heads)           # item i is (order[i // heads], i % heads)
    ends = np.cumsum(size)
    at = np.rint(total / ranges * np.arange(1, ranges)).astype(np.int64)
    item = np.searchsorted(ends, at, side="right")
    offset = at - (ends[item] - size[item])
    keep = (offset >= shortest) & (size[item] - offset >= shortest)
    # a segment starts at 0 in every item and at every cut that is kept
    seg_item = np.concatenate([np.arange(n, dtype=np.int64), item[keep]])
    seg_first = np.concatenate([np.zeros(n, dtype=np.int64), offset[keep]])
    by_place = np.argsort(seg_item * (int(lengths[order[0]]) + 1) + seg_first, kind="stable")
    seg_item, seg_first = seg_item[by_place], seg_first[by_place]
    goes_on = np.append(seg_item[1:] == seg_item[:-1], False)        # another segment of the item follows
    until = np.where(goes_on, np.append(seg_first[1:], 0), size[seg_item])
    work = until - seg_first
    pieces = np.bincount(seg_item, minlength=n)
    is_cut = pieces[seg_item] > 1
    slot = np.where(is_cut, np.cumsum(is_cut) - 1, -1)
    segments = np.stack([order[seg_item // heads], seg_item % heads, seg_first,
                         np.where(goes_on, work, TO_THE_END), slot], axis=1)
    segments = segments[np.argsort(-work, kind="stable")].astype(np.int32)
    cut = np.nonzero(pieces > 1)[0]
    first_slot = np.cumsum(pieces[cut]) - pieces[cut]
    items = np.stack([order[cut // heads], cut % heads, first_slot, pieces[cut]], axis=1).astype(np.int32)
    return segments, items, int(is_cut.sum())


@register_mixer("attention")
class Attention(Mixer):
    """q, k, v projections (with optional biases), position encoding of q and k, causal
    softmax attention with scale 1/sqrt(head_dim) in which query head h reads kv head
    floor(h * kv_heads / heads), output projection
    (AIR: src/reference/reference_executor.cpp:74-138, 349-384).

    params: hidden, heads, kv_heads, head_dim, qkv_bias, window (None: all keys),
            position (a PartSpec of a position encoding).
    Tensors: <prefix>{q,k,v}_proj.weight [heads*d | kv*d, hidden], <prefix>{q,k,v}_proj.bias
    (absent tensors mean no bias, as in AIR: src/model/qwen2_contract.cpp:133-136),
    <prefix>o_proj.weight [hidden, heads*d].

    At load the three projections become one matrix [(heads + 2 kv) d, hidden].  One kernel
    then adds the bias, rotates q and k and writes k and v into the request's pages; the
    attention kernel reads keys and values only from the pages, for prompt portions and
    decoded tokens alike."""

    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.heads, self.kv_heads, self.head_dim = p["hidden"], p["heads"], p["kv_heads"], p["head_dim"]
        self.window = p.get("window")
        self.qkv_bias = bool(p.get("qkv_bias", False))
        if self.heads % self.kv_heads:
            raise ConfigError("data_error", "attention: heads must be a multiple of kv_heads")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ConfigError("unsupported", f"attention: head size {self.head_dim} is not a multiple of 16 up to "
                                             "256, which is what the attention kernels take")
        pos = p["position"]
        self.position = POSITION_ENCODINGS.get(pos.kind)(pos)

    def cache_needs(self):
        return (PagedKV(self.kv_heads, self.head_dim, self.window),)

    # ------------------------------------------------------------------ the step's plan
    PLAN = "attention.tiles"

    def plan_key(self):
        return (self.PLAN, self.heads, self.window)

    def plan(self, batch: HostBatch) -> Plan:
        """What the tile kernels want to know of a step, worked out once for all attention layers with this many
        heads and this window: `decode_prefix`, the number of leading entries that bring a single next token (they
        take the decode kernel), and for the tokens after them `tiles` [16n, 4] int32 = (slot, first row, its
        position, rows <= 16): 16-token tiles in groups of 16, filled up with rows = 0.  A group is a pair of row
        tiles, 256 consecutive tokens of a request on one stream of keys; `segments`, `items` and `slots` say which
        block of the tcgen05 kernel takes which part of which pair's stream (plan_segments)."""
        prefix = 0
        while prefix < len(batch.counts) and batch.counts[prefix] == 1:
            prefix += 1
        tiles, key_tiles = [], []
        for i in range(prefix, len(batch.counts)):
            n, pos0 = batch.counts[i], batch.lengths[i]
            pairs = -(-n // 256)
            first = np.arange(pairs * 16, dtype=np.int32) * 16          # the entry's 16-token tiles, pairs filled up
            rows = np.clip(n - first, 0, 16)
            tile = np.zeros((pairs * 16, 4), dtype=np.int32)
            tile[:, 0] = batch.slots[i]
            tile[:, 1] = np.where(rows > 0, batch.q_start[i] + first, 0)
            tile[:, 2] = np.where(rows > 0, pos0 + first, 0)
            tile[:, 3] = rows
            tiles.append(tile)
            for g0 in range(0, n, 256):
                # the pair's keys: from the first one that its first row sees to its last row's own
                lowest = max(0, pos0 + g0 - self.window + 1) if self.window else 0
                key_tiles.append((pos0 + min(n, g0 + 256) - 1) // 64 + 1 - lowest // 64)
        tiles = np.concatenate(tiles) if tiles else np.zeros((0, 4), dtype=np.int32)
        arrays, values = {"tiles": tiles}, {"decode_prefix": prefix, "segments": None, "items": None, "slots": 0}
        cut = plan_segments(key_tiles, self.heads)
        if cut is not None:
            arrays["segments"], arrays["items"], values["slots"] = cut
            del values["segments"], values["items"]
        return Plan(arrays=arrays, values=values)

    def tensor_specs(self):
        d, p = self.head_dim, self.prefix
        specs = [TensorSpec(p + "q_proj.weight", (self.heads * d, self.hidden)),
                 TensorSpec(p + "k_proj.weight", (self.kv_heads * d, self.hidden)),
                 TensorSpec(p + "v_proj.weight", (self.kv_heads * d, self.hidden)),
                 TensorSpec(p + "o_proj.weight", (self.hidden, self.heads * d))]
        if self.qkv_bias:
            specs += [TensorSpec(p + "q_proj.bias", (self.heads * d,), optional=True, wide=True),
                      TensorSpec(p + "k_proj.bias", (self.kv_heads * d,), optional=True, wide=True),
                      TensorSpec(p + "v_proj.bias", (self.kv_heads * d,), optional=True, wide=True)]
        return specs + self.position.tensor_specs()

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p = self.prefix
        ws = [tensors[p + f"{n}_proj.weight"] for n in "qkv"]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{p}: q, k and v projections are stored in different precisions")
        self.qkv = Linear(torch.cat(ws, dim=0).contiguous(), rt.status)
        self.q_only = self.qkv.rows(0, self.heads * self.head_dim)
        self.o = Linear(tensors[p + "o_proj.weight"], rt.status)
        self.bias = None
        if any((p + f"{n}_proj.bias") in tensors for n in "qkv"):
            parts = []
            for n, rows in zip("qkv", (self.heads, self.kv_heads, self.kv_heads)):
                b = tensors.get(p + f"{n}_proj.bias")
                parts.append(b.to(torch.float32) if b is not None
                             else torch.zeros(rows * self.head_dim, dtype=torch.float32, device=rt.device))
            self.bias = torch.cat(parts).contiguous()
        self.position.load(tensors, rt)
        self.scale = 1.0 / math.sqrt(self.head_dim)

    def _fresh(self, ctx) -> bool:
        """Whether a step of single next tokens takes the decode kernel that starts from the q/k/v product."""
        table = self.position.table()
        d = self.head_dim
        return (self.rt.dtype == torch.bfloat16 and ctx.all_decode and d in ops.DECODE_HEAD_DIMS and table is not None
                and table.shape[1] == d and ops.tile_pages(self.rt.page_tokens))

    def accepts_prenormed(self, ctx, owns_cache=True):
        # only on the road of a decode step: the q/k/v product for few rows applies the scale per row and hands
        # partial sums to the attention kernel
        return owns_cache and self.qkv.takes_prenormed(ctx.num_tokens) and self._fresh(ctx)

    def forward(self, x, ctx, cache, owns_cache=True):
        (pages,) = cache
        T = x.shape[0]
        H, K, d = self.heads, self.kv_heads, self.head_dim
        rt = self.rt
        if owns_cache:
            qkv = self.qkv.partial(x) if self.qkv.small(x) else self.qkv(x, torch.float32)
        else:
            # this run reads another run's keys and values: only q is computed
            qkv = torch.zeros((T, (H + 2 * K) * d), dtype=torch.float32, device=x.device)
            qkv[:, : H * d] = self.q_only(x, torch.float32)
        bt = ctx.block_tables[pages.group]
        table = self.position.table()
        if (rt.dtype == torch.bfloat16 and ctx.all_decode
                and ops.decode_attention_fresh_ok(qkv, table, pages.kv, d)):
            # single next tokens only: the attention kernel itself adds the bias, rotates, writes the new keys
            # and values and attends (one launch less, and the keys stream as soon as the product has ended)
            out = torch.empty((T, H, d), dtype=rt.dtype, device=x.device)
            ops.decode_attention_fresh(qkv, self.bias, table, pages.kv, bt, ctx.token_seq, ctx.positions, out, H,
                                       self.window, self.scale, write_kv=owns_cache, status=ctx.status)
            return self._project(out.view(T, H * d), ctx)
        if isinstance(x, PreNormed):
            raise ops.KernelError("attention: rows without their norm's scale reached a road that does not apply it")
        q = torch.empty((T, H, d), dtype=rt.dtype, device=x.device)
        ops.qkv_rope_store(qkv, self.bias, table, ctx.positions, ctx.token_seq, bt, q, pages.kv,
                           H, K, d, write_kv=owns_cache, status=ctx.status)
        out = torch.empty_like(q)
        if rt.dtype == torch.bfloat16 and d in ops.DECODE_HEAD_DIMS and ctx.all_decode:
            ops.decode_attention(q, pages.kv, bt, ctx.token_seq, ctx.positions, out, self.window, self.scale)
        elif (rt.dtype == torch.bfloat16 and d in ops.DECODE_HEAD_DIMS and self.plan_key() in ctx.plans
              and ops.tile_pages(pages.kv.shape[3])):
            # a mixed step: the single next tokens at the head of the batch take the decode kernel (a row
            # tile of 128 queries for one token would read its request's whole context for one row), the
            # prompt portions the tile kernels
            plan = ctx.plans[self.plan_key()]
            n = plan.decode_prefix
            if n:
                ops.decode_attention(q[:n], pages.kv, bt, ctx.token_seq[:n], ctx.positions[:n], out[:n], self.window,
                                     self.scale)
            if plan.tiles.shape[0] == 0:
                pass
            elif d in ops.TC_ATTENTION_HEAD_DIMS:     # both products on the tcgen05 tensor cores
                if plan.slots and getattr(plan, "scratch", None) is None:
                    # (the step's layers run one after the other on one stream and share the partial sums' memory)
                    plan.scratch = ops.prefill_attention_scratch(plan.slots, d, q.device)
                ops.prefill_attention_tc(q, pages.kv, bt, plan.tiles, out, self.window, self.scale, status=ctx.status,
                                         segments=plan.segments, items=plan.items, slots=plan.slots,
                                         scratch=getattr(plan, "scratch", None))
            else:
                ops.prefill_attention(q, pages.kv, bt, plan.tiles, out, self.window, self.scale, status=ctx.status)
        else:
            ops.paged_attention_ref(q, pages.kv, bt, ctx.token_seq, ctx.positions, out, self.window, self.scale)
        return self._project(out.view(T, H * d), ctx)

    def _project(self, out, ctx):
        if self.o.small(out):
            return self.o.partial(out)
        residual = getattr(ctx, "residual", None)
        if self.o.adds_into(out, residual):
            return self.o.add_into(out, residual)
        return self.o(out, torch.float32)
