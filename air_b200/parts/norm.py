"""RMSNorm fused with the residual addition that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Norm, PreNormed
from .registry import register_norm


@register_norm("rms")
class RMSNorm(Norm):
    """x * rsqrt(mean(x^2) + eps) * w, product order x*scale*w, no bias, no offset on w
    (AIR: src/reference/reference_executor.cpp:17-27; src/cuda/cuda_backend.cu:789-831).
    params: size, eps.  Tensor: <prefix>weight [size].  The sum of squares and the residual
    sum are 32-bit."""

    graph_safe = True

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "weight", (self.spec["size"],), init="one_plus_normal", wide=True)]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        self.weight = tensors[self.prefix + "weight"]
        self.eps = float(self.spec["eps"])

    prenorm = True      # x * scale(row) * w: forward_prenormed writes bfloat16(x * w) and leaves the scale to the consumer

    def forward(self, h, delta, rows=None):
        n = h.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, h.shape[1]), dtype=self.rt.dtype, device=h.device)
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows=rows)

    def forward_prenormed(self, h, delta) -> PreNormed:
        """As forward() without rows, for a part that takes its input as PreNormed: the stream is completed and
        the rows are written short of their scale, by many small blocks that do not wait for one another."""
        T, E = h.shape
        xg = torch.empty((T, E), dtype=torch.bfloat16, device=h.device)
        ss = torch.empty((-(-E // ops.PRENORM_CHUNK), T), dtype=torch.float32, device=h.device)
        ops.add_prenorm(h, delta, self.weight, xg, ss)
        return PreNormed(xg, ss, self.eps)
