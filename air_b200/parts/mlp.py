"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import FeedForward
from .linear import Linear
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)) with silu(x) = x / (1 + exp(-x)), no biases
    (AIR: src/reference/reference_executor.cpp:33-35, 394-408).
    params: hidden, intermediate.  Tensors: <prefix>{gate,up}_proj.weight [intermediate, hidden],
    <prefix>down_proj.weight [hidden, intermediate].  gate and up become one matrix at load, so
    the input is read once; the activation kernel reads both halves of its output."""

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
        self.gate_up = Linear(torch.cat([g, u], dim=0).contiguous())
        self.down = Linear(tensors[p + "down_proj.weight"])
        self.intermediate = self.spec["intermediate"]

    def forward(self, x, ctx):
        gu = self.gate_up(x, torch.float32 if self.rt.is_fp32 else self.rt.dtype)
        act = torch.empty((x.shape[0], self.intermediate), dtype=self.rt.dtype, device=x.device)
        ops.silu_mul(gu, act)
        return self.down(act, torch.float32)
