"""Rotary position encoding as a table of cos and sin per position."""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rope_half")
class RopeHalf(PositionEncoding):
    """Half-split rotation: pairs (i, i + rot/2), angle p * theta^(-2i/rot)
    (AIR: src/reference/reference_executor.cpp:37-72; src/cuda/cuda_backend.cu:862-906).
    params: rotary_dim, theta, max_positions.  No tensors.

    The angles are evaluated once, in 64-bit like AIR's CPU executor, and kept as float32
    cos|sin [max_positions, rotary_dim]; the mixer's kernel reads a token's row by its
    position.  Another frequency rule (scaled, interpolated) is another table of the same
    shape.  Layers whose encodings have equal parameters share one table (Runtime.shared), so a
    step reads one row per token whatever the number of layers."""

    def load(self, tensors, rt):
        super().load(tensors, rt)
        rot, theta, n = int(self.spec["rotary_dim"]), float(self.spec["theta"]), int(self.spec["max_positions"])
        if rot % 2:
            raise ValueError("rope_half needs an even rotary width")
        self.rotary_dim = rot
        key = ("rope_half", rot, theta, n)
        table = rt.shared.get(key)
        if table is None:
            i = torch.arange(rot // 2, dtype=torch.float64)
            inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), (2.0 * i) / rot)
            angle = torch.arange(n, dtype=torch.float64)[:, None] * inv_freq[None, :]
            table = rt.shared[key] = torch.cat([torch.cos(angle), torch.sin(angle)], dim=1).to(torch.float32).to(rt.device)
        self._table = table

    def table(self):
        return self._table


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    """No position encoding: the mixer's kernel rotates nothing."""
