"""What every part must offer.

A part is built from its description alone (sizes and constants are parameters, nothing is
read from a model's configuration), says which tensors it needs, takes them when they are
loaded, and computes.  No part knows which model it is in, which layer it is, or what the
other parts of its block are.

  Norm              forward(h, delta, rows=None) -> normalised rows in the compute dtype; h (the
                    float32 residual stream) has delta added in place on the way (rows=None)
  PositionEncoding  table() -> float32 [positions, rotary width] cos|sin, consumed by mixers
  Mixer             cache_needs() -> what it keeps per request (pages of keys and values, a
                    state of fixed size, both, or nothing);
                    forward(x, ctx, cache, owns_cache) -> [T, hidden], or float32 [parts, T, hidden]
                    partial sums that the next norm adds up in order
  FeedForward       forward(x, ctx) -> [T, hidden] (or partial sums, as above)
  Block             forward(h, pending, ctx, cache, owns_cache) -> (h, pending): the arrangement
                    of two norms, a mixer and a feed-forward around the residual stream
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..weights.loader import TensorSpec
from .spec import PartSpec


@dataclass
class Runtime:
    """Where and how the parts compute: the device, the compute dtype (bfloat16 or
    float32; float32 means no reduced-precision step anywhere) and the page size."""
    device: torch.device
    dtype: torch.dtype
    page_tokens: int = 64
    status: Optional[torch.Tensor] = None    # [1] int32 on the device: kernels report impossible states here

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


# ------------------------------------------------------------------ what a mixer keeps per request
@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token, in pages.  window: None keeps all keys, a number
    keeps the last `window` of them (older pages are given back).  Layers with equal needs
    share a group: one pool of pages and one block table."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class SlotState:
    """A state of fixed size per request (zeroed when the request opens), as a recurrent
    or convolutional mixer keeps it."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


CacheNeed = object  # PagedKV | SlotState


class Part:
    def __init__(self, spec: PartSpec, prefix: str = ""):
        self.spec = spec
        self.prefix = prefix

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt


class Norm(Part):
    def forward(self, h, delta, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    rotary_dim: int = 0

    def table(self) -> Optional[torch.Tensor]:
        return None


class Mixer(Part):
    # True if forward() only launches work on the current stream from device data (no host
    # reads of the batch), so that a decode step can be captured in a CUDA graph.
    graph_safe: bool = False

    def cache_needs(self) -> Tuple[CacheNeed, ...]:
        return ()

    def forward(self, x, ctx, cache, owns_cache: bool):
        raise NotImplementedError


class FeedForward(Part):
    graph_safe: bool = False    # as for Mixer: nothing in forward() reads the batch or a result on the host

    def forward(self, x, ctx):
        raise NotImplementedError
