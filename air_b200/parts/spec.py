"""Descriptions of a model as data: which parts a layer is made of, with their sizes and
constants, and the order in which layers run.  A description holds no tensors; the
classes in this package are built from it.

Each part is named by a ``kind`` string that a registry (air_b200.parts.registry) maps
to a class, so another mixer, feed-forward, norm or position encoding is a new class and
a new kind, and the description of a model may pick a different one for every layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """kind: registry key.  params: sizes and constants of the part."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: how its parts are arranged (kind: a registered block class), the parts by the
    role they have in that arrangement, the prefix of the layer's tensors in the checkpoint and
    what follows the prefix for each role.  The block class decides which roles it wants (the
    pre-norm block: mixer_norm, mixer, feed_forward_norm, feed_forward); another arrangement
    (norms after the parts, a third sub-layer, parts side by side) is another block class with
    roles of its own and needs no change here."""
    kind: str
    prefix: str
    parts: Mapping[str, PartSpec]
    names: Mapping[str, str] = field(default_factory=dict)

    def part(self, role: str) -> PartSpec:
        try:
            return self.parts[role]
        except KeyError:
            raise ValueError(f"block '{self.kind}' at '{self.prefix}' needs a part in the role '{role}' "
                             f"(it has: {', '.join(sorted(self.parts))})") from None

    def name(self, role: str) -> str:
        """Prefix of the tensors of the part in this role."""
        return self.prefix + self.names.get(role, role + ".")


@dataclass(frozen=True)
class RunStep:
    """One run of a layer.  cache_from: None for a run that keeps a cache of its own, else
    the index (in the order list) of the earlier run whose cache this run reads."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[BlockSpec, ...]
    order: Tuple[RunStep, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_prefix: str
    output_name: Optional[str]  # None: the output matrix is the embedding table (tied)
    eos_token_id: Optional[int] = None
    # Off for the Qwen2 decoder; other decoders of the same skeleton differ in them:
    embedding_multiplier: float = 1.0        # the embedding rows are multiplied by this (in 32-bit)
    output_bias_name: Optional[str] = None   # a float32 [vocab] tensor added to the logits
    logit_scale: float = 1.0                 # logits = (x W^T + bias) * logit_scale
    logit_softcap: float = 0.0               # > 0: logits = cap * tanh(logits / cap), after the scale

    def validate(self) -> None:
        for i, run in enumerate(self.order):
            if not (0 <= run.layer < len(self.layers)):
                raise ValueError(f"order[{i}] names layer {run.layer}, the model has {len(self.layers)}")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < i):
                    raise ValueError(f"order[{i}] reads the cache of run {run.cache_from}, which is not earlier")
                if self.order[run.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}] reads the cache of run {run.cache_from}, which has none of its own")
