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
        return (self.PLAN, self.heads)

    def plan(self, batch: HostBatch) -> Plan:
        """What the tile kernels want to know of a step, worked out once for all attention layers with this many
        heads: `decode_prefix`, the number of leading entries that bring a single next token (they take the decode
        kernel), and for the tokens after them `tiles` [16n, 4] int32 = (slot, first row, its position, rows <= 16):
        16-token tiles in groups of 16, filled up with rows = 0.  A group is what one block of the tcgen05 kernel
        takes per head: two row tiles of 128 consecutive tokens of a request on one stream of keys.  Where that
        would give fewer blocks than half the SMs (a short portion on top of a long prefix: every block walks the
        whole prefix), a group holds ONE row tile and eight empty entries instead: twice the blocks, each with
        half the work, the keys read twice from L2."""
        prefix = 0
        while prefix < len(batch.counts) and batch.counts[prefix] == 1:
            prefix += 1
        portions = range(prefix, len(batch.counts))
        pairs = sum(-(-batch.counts[i] // 256) for i in portions)
        rows_per_group = 128 if 0 < pairs * self.heads <= SMS // 2 else 256
        tiles = []
        for i in portions:
            n = batch.counts[i]
            for g0 in range(0, n, rows_per_group):
                rows = min(rows_per_group, n - g0)
                count = -(-rows // 16)
                tile = np.zeros((16, 4), dtype=np.int32)
                tile[:, 0] = batch.slots[i]
                first = g0 + np.arange(count, dtype=np.int32) * 16
                tile[:count, 1] = batch.q_start[i] + first
                tile[:count, 2] = batch.lengths[i] + first
                tile[:count, 3] = np.minimum(16, n - first)
                tiles.append(tile)
        tiles = np.concatenate(tiles) if tiles else np.zeros((0, 4), dtype=np.int32)
        return Plan(arrays={"tiles": tiles}, values={"decode_prefix": prefix})

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
                ops.prefill_attention_tc(q, pages.kv, bt, plan.tiles, out, self.window, self.scale, status=ctx.status)
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
