"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import FeedForward
from .linear import Linear, SMS
from .registry import register_feed_forward


# Up to so many rows the package's product with the activation in its epilogue is faster than the library's
# product followed by the activation kernel (measured at 18944 x 3584: 776 against 803 us at 4,096 rows,
# 1,261 against 1,203 us at 6,144).
FUSED_ROWS = 4096


def fused_gate_up_pays(rows: int, out_features: int) -> bool:
    """Whether the package's product with the activation in its epilogue is at least as fast as the library's
    product followed by the activation kernel, for this many rows and 2 x intermediate output features.

    Measured on B200 at the 7B, 14B and 32B widths, CUDA events, cold L2.  Up to 128 rows the two are equal (the
    kernel for up to 64 rows is another matter and is not asked about here).  From 129 to 511 rows the package's
    kernel works on tiles of 128 rows, which wait for their operands a third of the time: the library is up to 36 %
    faster (14B, 384 rows: 124 against 91 us).  From 512 rows on its tiles are 256 x 256 and it is as fast as the
    library where those tiles fill whole rounds over the SMs and the rows fill the tiles (7B 768 rows: 149.5
    against 148.3 us; 14B 1,024: 197.7 / 195.5; 2,048: 369.6 / 375.8), and up to 55 % slower where they do not
    (14B 544 rows, 324 tiles of which the last third is nearly empty: 185.5 against 119.9 us)."""
    if rows <= 128:
        return True
    if rows < 512 or rows > FUSED_ROWS:
        return False
    row_tiles, col_tiles = -(-rows // 256), -(-out_features // 256)
    tiles = row_tiles * col_tiles
    rounds = -(-tiles // SMS)
    return (tiles / (rounds * SMS)) * (rows / (row_tiles * 256)) >= 0.9


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)) with silu(x) = x / (1 + exp(-x)), no biases
    (AIR: src/reference/reference_executor.cpp:33-35, 394-408).
    params: hidden, intermediate.  Tensors: <prefix>{gate,up}_proj.weight [intermediate, hidden],
    <prefix>down_proj.weight [hidden, intermediate].  gate and up become one matrix at load, so
    the input is read once: blocks of gate rows and of up rows for the same outputs in turn (the
    block is the largest of 128, 64, 32 that divides `intermediate`, else all of it), so that a
    tile of the product holds both factors of its outputs and the tcgen05 kernel can apply the
    activation in its epilogue, for few rows and for many; where that kernel does not apply (32-bit
    weights, an odd width) the library's product is followed by the activation kernel, which reads
    the same arrangement."""

    graph_safe = True

    def tensor_specs(self):
        e, i, p = self.spec["hidden"], self.spec["intermediate"], self.prefix
        return [TensorSpec(p + "gate_proj.weight", (i, e)), TensorSpec(p + "up_proj.weight", (i, e)),
                TensorSpec(p + "down_proj.weight", (e, i))]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        p = self.prefix
        g, u = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError(f"{p}: gate and up projections are stored in different precisions")
        inter = self.intermediate = self.spec["intermediate"]
        block = next((b for b in (128, 64, 32) if inter % b == 0), inter)
        if g.dtype != torch.bfloat16:
            block = inter
        self.block = block
        if block == inter:
            w = torch.cat([g, u], dim=0)
        else:
            w = torch.stack([g.view(inter // block, block, -1), u.view(inter // block, block, -1)], dim=1)
            w = w.reshape(2 * inter, -1)
        self.gate_up = Linear(w.contiguous(), rt.status, gate_up_block=block if block != inter else 0)
        self.down = Linear(tensors[p + "down_proj.weight"], rt.status)

    def accepts_prenormed(self, ctx, owns_cache=True):
        return self.rt.dtype == torch.bfloat16 and self.gate_up.takes_prenormed(ctx.num_tokens, silu=True)

    def forward(self, x, ctx):
        if (self.gate_up.gate_up_block and self.gate_up.tc_ok and x.dtype == torch.bfloat16
                and (self.gate_up.small(x) or fused_gate_up_pays(x.shape[0], self.gate_up.out_features))):
            # few rows or many: the tcgen05 product with SiLU(gate) * up in its epilogue (the 2 I wide
            # intermediate is never written)
            act = self.gate_up.silu_mul(x)
        else:
            gu = self.gate_up(x, torch.float32 if self.rt.is_fp32 else self.rt.dtype)
            act = torch.empty((x.shape[0], self.intermediate), dtype=self.rt.dtype, device=x.device)
            ops.silu_mul(gu, act, block=self.block)
        if self.down.small(act):
            return self.down.partial(act)
        residual = getattr(ctx, "residual", None)
        if self.down.adds_into(act, residual):
            return self.down.add_into(act, residual)
        return self.down(act, torch.float32)
