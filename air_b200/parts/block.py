"""How the parts of one layer stand around the residual stream."""
from __future__ import annotations

from .registry import register_block, MIXERS, FEED_FORWARDS, NORMS
from .spec import BlockSpec


class Block:
    """What an arrangement offers to the model: its parts, their tensors, what the layer keeps per
    request, and forward(h, pending, ctx, cache, owns_cache) -> (h, pending).  A subclass builds its
    parts from `spec.part(role)` with the registry of the role's kind and `spec.name(role)` as the
    prefix of their tensors."""

    def __init__(self, spec: BlockSpec):
        self.spec = spec

    def parts(self):
        raise NotImplementedError

    def tensor_specs(self):
        return [s for part in self.parts() for s in part.tensor_specs()]

    def load(self, tensors, rt):
        for part in self.parts():
            part.load(tensors, rt)

    def cache_needs(self):
        """What the layer keeps per request (CacheNeed objects); forward() receives their views as `cache`,
        in the same order."""
        return ()

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def forward(self, h, pending, ctx, cache, owns_cache=True):
        raise NotImplementedError


@register_block("pre_norm")
class PreNormBlock(Block):
    """h = h + mixer(norm1(h)); h = h + feed_forward(norm2(h))
    (AIR: src/reference/reference_executor.cpp:343-413).
    Roles: mixer_norm, mixer, feed_forward_norm, feed_forward.

    The residual stream h is float32.  Each addition is fused into the norm that follows
    it: the block receives the previous block's output still pending, and hands its own
    feed-forward output on in the same way; the model's final norm adds the last one.  A part may
    instead add its output into the stream itself (StepContext.residual) and return None: with
    many rows the library's product does that addition in its epilogue, in 32-bit, and the norm
    that follows reads the stream alone."""

    def __init__(self, spec: BlockSpec):
        super().__init__(spec)
        self.mixer_norm = NORMS.get(spec.part("mixer_norm").kind)(spec.part("mixer_norm"), spec.name("mixer_norm"))
        self.mixer = MIXERS.get(spec.part("mixer").kind)(spec.part("mixer"), spec.name("mixer"))
        self.ff_norm = NORMS.get(spec.part("feed_forward_norm").kind)(spec.part("feed_forward_norm"),
                                                                      spec.name("feed_forward_norm"))
        self.feed_forward = FEED_FORWARDS.get(spec.part("feed_forward").kind)(spec.part("feed_forward"),
                                                                              spec.name("feed_forward"))

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward)

    def cache_needs(self):
        return self.mixer.cache_needs()

    @staticmethod
    def _norm(norm, h, delta, part, ctx, owns_cache=True):
        """The norm before `part`: where the part takes rows short of their scale in this step and the norm can
        write them so, the wide kernel whose blocks do not wait for one another."""
        if getattr(norm, "prenorm", False) and part.accepts_prenormed(ctx, owns_cache):
            return norm.forward_prenormed(h, delta)
        return norm.forward(h, delta)

    def forward(self, h, pending, ctx, cache, owns_cache=True):
        ctx.residual = h
        x = self._norm(self.mixer_norm, h, pending, self.mixer, ctx, owns_cache)
        a = self.mixer.forward(x, ctx, cache, owns_cache)      # None: the mixer has added its output to h itself
        x = self._norm(self.ff_norm, h, a, self.feed_forward, ctx)
        return h, self.feed_forward.forward(x, ctx)
