"""A model put together from its description: the embedding, the blocks in the order of the
run list, the final norm and the output matrix.  Nothing here knows an architecture: the
description (air_b200.parts.spec.ModelSpec) is data that the architecture's entry in the
registry produced from config.json.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from ..parts import registry
from ..parts.base import Runtime
from ..parts.linear import Linear
from ..parts.spec import ModelSpec
from ..weights.loader import TensorSpec


class Model:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks = [registry.BLOCKS.get(b.kind)(b) for b in spec.layers]
        self.final_norm = registry.NORMS.get(spec.final_norm.kind)(spec.final_norm, spec.final_norm_prefix)

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> List[TensorSpec]:
        s = self.spec
        specs = [TensorSpec(s.embedding_name, (s.vocab_size, s.hidden_size))]
        for b in self.blocks:
            specs += b.tensor_specs()
        specs += self.final_norm.tensor_specs()
        if s.output_name is not None:
            specs.append(TensorSpec(s.output_name, (s.vocab_size, s.hidden_size)))
        if s.output_bias_name is not None:
            specs.append(TensorSpec(s.output_bias_name, (s.vocab_size,), init="zeros", wide=True))
        seen = set()
        for t in specs:
            if t.name in seen:
                raise ValueError(f"two parts claim the tensor '{t.name}'")
            seen.add(t.name)
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.embedding = tensors[self.spec.embedding_name]
        for b in self.blocks:
            b.load(tensors, rt)
        self.final_norm.load(tensors, rt)
        out = self.embedding if self.spec.output_name is None else tensors[self.spec.output_name]
        self.output = Linear(out, rt.status)
        bias = None if self.spec.output_bias_name is None else tensors[self.spec.output_bias_name]
        self.output_bias = None if bias is None else bias.to(torch.float32)
        self._planners = None

    def planners(self):
        """The parts that plan on the host, one for every plan key (Part.plan_key)."""
        if self._planners is None:
            found = {}
            for b in self.blocks:
                for part in b.parts():
                    key = part.plan_key()
                    if key is not None and key not in found:
                        found[key] = part
            self._planners = tuple(found.values())
        return self._planners

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step may be captured in a CUDA graph: no part reads the batch on the host."""
        return all(b.graph_safe for b in self.blocks) and getattr(self.final_norm, "graph_safe", False)

    def cache_needs(self):
        """Per run of the order list: the needs of the layer's mixer, or nothing for a run that
        reads another run's cache."""
        return [self.blocks[run.layer].cache_needs() if run.cache_from is None else ()
                for run in self.spec.order]

    def weight_bytes(self) -> int:
        """Bytes of the tensors that one step reads (every weight once)."""
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        for run in {r.layer for r in self.spec.order}:
            b = self.blocks[run]
            for part in b.parts():
                for v in vars(part).values():
                    if isinstance(v, Linear):
                        add(v.weight)
                    else:
                        add(v)
        add(self.output.weight)
        add(self.final_norm.weight)
        return total

    # ------------------------------------------------------------------ computing
    def forward(self, ctx, cache) -> torch.Tensor:
        """Runs the batch's tokens through every run of the order list, writing the caches,
        and returns float32 logits [wanted rows, vocab]."""
        rt = self.rt
        h = torch.empty((ctx.num_tokens, self.spec.hidden_size), dtype=torch.float32, device=rt.device)
        ops.embedding(self.embedding, ctx.token_ids, h, status=ctx.status, last_token=ctx.last_token,
                      multiplier=self.spec.embedding_multiplier)
        pending = None
        for i, run in enumerate(self.spec.order):
            owner = i if run.cache_from is None else run.cache_from
            h, pending = self.blocks[run.layer].forward(h, pending, ctx, cache.views(owner),
                                                        owns_cache=run.cache_from is None)
        R = ctx.logit_rows.shape[0]
        if R == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        y = self.final_norm.forward(h, pending, rows=ctx.logit_rows)
        logits = self.output.full(y) if self.output.small(y) else self.output(y, torch.float32)
        s = self.spec
        if self.output_bias is not None or s.logit_scale != 1.0 or s.logit_softcap > 0.0:
            ops.logits_post(logits, self.output_bias, s.logit_scale, s.logit_softcap)
        return logits
