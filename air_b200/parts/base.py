"""What every part must offer.

A part is built from its description alone (sizes and constants are parameters, nothing is
read from a model's configuration), says which tensors it needs, takes them when they are
loaded, and computes.  No part knows which model it is in, which layer it is, or what the
other parts of its block are.

  Norm              forward(h, delta, rows=None) -> normalised rows in the compute dtype.  h is the
                    float32 residual stream [T, hidden]; `delta` is what the part before the norm
                    produced and has NOT yet been added to the stream: None, a tensor [T, hidden]
                    (float32 or the compute dtype), or float32 partial sums [parts, T, hidden] that
                    are to be added in the order of `parts`.  Without `rows` the norm adds delta into
                    h in place and normalises every row; with `rows` (int32 indices) it leaves h as it
                    is and returns the norm of h[rows] + delta[rows].  A norm that does not want to
                    know about the forms of delta calls `self.add_delta(h, delta)` first, which is the
                    package's kernel for exactly that sum, and then works on h alone.
  PositionEncoding  table() -> float32 [positions, rotary width] cos|sin, consumed by mixers
  Mixer             cache_needs() -> what it keeps per request (CacheNeed objects: pages of keys and
                    values, pages of something else, a state of fixed size, several, or nothing);
                    plan(batch) -> what it wants worked out on the host once per step (optional);
                    forward(x, ctx, cache, owns_cache) -> [T, hidden], or float32 [parts, T, hidden]
                    partial sums, or None after adding its output into ctx.residual itself
  FeedForward       forward(x, ctx) -> as a mixer
  Block             forward(h, pending, ctx, cache, owns_cache) -> (h, pending): an arrangement of
                    parts around the residual stream; `pending` is a delta in the sense above
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..weights.loader import TensorSpec
from .spec import PartSpec


@dataclass
class Runtime:
    """Where and how the parts compute: the device, the compute dtype (bfloat16 or
    float32; float32 means no reduced-precision step anywhere) and the page size.  `shared`
    holds what equal parts of different layers make once and share (a position table)."""
    device: torch.device
    dtype: torch.dtype
    page_tokens: int = 64
    status: Optional[torch.Tensor] = None    # [1] int32 on the device: kernels report impossible states here
    shared: Dict[Hashable, object] = field(default_factory=dict)

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


# ------------------------------------------------------------------ what a mixer keeps per request
class CacheNeed:
    """One thing a mixer keeps per request.  The cache manager knows no kinds of need: it asks
    each need for the shape of its memory and hands the mixer what `view` returns.

    A *paged* need keeps something for every token: the manager makes one slab
    [pages, *page_shape(page_tokens)] per run and gives the request pages of it, through a block
    table that runs with an equal `group_key()` share.  `window` (None: everything is kept) lets
    the manager take back pages whose tokens no later query can see.  A need that is not paged
    keeps `slot_shape()` per request, zeroed when the request opens."""
    paged: bool = False
    window: Optional[int] = None

    def group_key(self) -> Hashable:
        return self

    def page_shape(self, page_tokens: int) -> Tuple[int, ...]:
        raise NotImplementedError

    def slot_shape(self) -> Tuple[int, ...]:
        raise NotImplementedError

    def element_dtype(self, compute_dtype: torch.dtype) -> torch.dtype:
        return compute_dtype

    def view(self, tensor: Optional[torch.Tensor], group: Optional[int]):
        """What the mixer's forward() receives for this need."""
        raise NotImplementedError

    def bytes_per_page(self, page_tokens: int, compute_dtype: torch.dtype) -> int:
        n = 1
        for s in self.page_shape(page_tokens):
            n *= s
        return n * torch.empty((), dtype=self.element_dtype(compute_dtype)).element_size()


@dataclass
class PagedKVView:
    """What a mixer gets for a PagedKV need: its slab [pages, 2, kv_heads, page_tokens, head_dim]
    and the index of its group (for the step's block table)."""
    kv: Optional[torch.Tensor]
    group: int
    need: "PagedKV"


@dataclass
class SlotStateView:
    """What a mixer gets for a SlotState need: [slots, *shape]; row = the request's slot."""
    state: Optional[torch.Tensor]
    need: "SlotState"


@dataclass(frozen=True)
class PagedKV(CacheNeed):
    """Keys and values of every token, in pages.  window: None keeps all keys, a number
    keeps the last `window` of them (older pages are given back).  Layers with equal needs
    share a group: one pool of pages and one block table."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    paged = True

    def page_shape(self, page_tokens):
        return (2, self.kv_heads, page_tokens, self.head_dim)

    def view(self, tensor, group):
        return PagedKVView(tensor, group, self)


@dataclass(frozen=True)
class SlotState(CacheNeed):
    """A state of fixed size per request (zeroed when the request opens), as a recurrent
    or convolutional mixer keeps it."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
    paged = False

    def slot_shape(self):
        return tuple(self.shape)

    def element_dtype(self, compute_dtype):
        return getattr(torch, self.dtype)

    def view(self, tensor, group):
        return SlotStateView(tensor, self)


# ------------------------------------------------------------------ what a part may plan on the host
@dataclass
class HostBatch:
    """One step's batch as the host knows it, for parts that work something out per step before
    the kernels run (lists of tiles, schedules).  Entry i brings counts[i] next tokens of a request
    that holds lengths[i] tokens already; its tokens are rows q_start[i] .. q_start[i + 1] of the
    step; slots[i] is the request's state slot."""
    counts: List[int]
    lengths: List[int]
    slots: List[int]
    q_start: List[int]


@dataclass
class Plan:
    """What `plan` returns: int32 arrays that the step copies to the device with the rest of the
    batch (the part finds them as device tensors under the same names), and plain host values."""
    arrays: Dict[str, "object"] = field(default_factory=dict)     # name -> numpy int32 array (any shape)
    values: Dict[str, object] = field(default_factory=dict)


@dataclass
class PreNormed:
    """Rows that an RMSNorm would produce, short of the scale per row: x = bfloat16(h * weight), and the sums
    of squares of h per row in parts (ss [parts, T], to be added in order): the row's scale is
    rsqrt(sum / width + eps).  One number per row commutes with a matrix product, so a product that takes these
    rows applies the scale to its accumulators.  A norm of the form x * scale(row) * weight writes its rows so
    (Norm.forward_prenormed) where the part behind it says that it takes them in this step
    (Part.accepts_prenormed): the kernel that writes them has no block that waits for a row's other blocks."""
    x: torch.Tensor
    ss: torch.Tensor
    eps: float

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device


class Part:
    # True if forward() only launches work on the current stream from device data (no host
    # reads of the batch or of a result), so that a decode step can be captured in a CUDA graph.
    graph_safe: bool = False

    def __init__(self, spec: PartSpec, prefix: str = ""):
        self.spec = spec
        self.prefix = prefix

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt

    # A part that wants something worked out on the host once per step names it with a key (parts
    # with equal keys share one plan: 28 attention layers plan once) and builds it in plan().  The
    # result is at ctx.plans[key]: a namespace with the arrays as device tensors and the values.
    def plan_key(self) -> Optional[Hashable]:
        return None

    def plan(self, batch: HostBatch) -> Optional[Plan]:
        return None

    def accepts_prenormed(self, ctx, owns_cache: bool = True) -> bool:
        """Whether forward() in this step takes its input as a PreNormed (see there)."""
        return False


class Norm(Part):
    def forward(self, h, delta, rows=None):
        raise NotImplementedError

    @staticmethod
    def add_delta(h: torch.Tensor, delta) -> torch.Tensor:
        """h += delta for every form of delta that a part may hand on (see the module's text)."""
        if delta is not None:
            from ..csrc import ops
            ops.add_parts(h, delta)
        return h


class PositionEncoding(Part):
    rotary_dim: int = 0

    def table(self) -> Optional[torch.Tensor]:
        return None


class Mixer(Part):
    def cache_needs(self) -> Tuple[CacheNeed, ...]:
        return ()

    def forward(self, x, ctx, cache, owns_cache: bool):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError
