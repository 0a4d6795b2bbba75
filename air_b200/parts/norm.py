"""RMSNorm fused with the residual addition that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Norm
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

    def forward(self, h, delta, rows=None):
        n = h.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, h.shape[1]), dtype=self.rt.dtype, device=h.device)
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows=rows)
