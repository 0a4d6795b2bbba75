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
    """One layer: how its parts are arranged (kind), the parts, and the prefix of its
    tensors' names in the checkpoint."""
    kind: str
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    # what follows the prefix in the names of each part's tensors
    names: Mapping[str, str] = field(default_factory=lambda: {
        "mixer_norm": "input_layernorm.", "mixer": "self_attn.",
        "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."})


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

    def validate(self) -> None:
        for i, run in enumerate(self.order):
            if not (0 <= run.layer < len(self.layers)):
                raise ValueError(f"order[{i}] names layer {run.layer}, the model has {len(self.layers)}")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < i):
                    raise ValueError(f"order[{i}] reads the cache of run {run.cache_from}, which is not earlier")
                if self.order[run.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}] reads the cache of run {run.cache_from}, which has none of its own")
