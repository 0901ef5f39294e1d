"""Pre-norm residual block: h += mixer(norm1(h)); h += ffn(norm2(h))
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:14-36).  The residual stream h is
float32; the normed activations have the engine's compute type."""
from __future__ import annotations

from .base import PartSpec, Prenormed, build_part, register_part


class PreNormBlock:
    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, feed_forward: PartSpec):
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.norm2 = build_part("norm", norm2)
        self.feed_forward = build_part("feed_forward", feed_forward)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    # -- what the model asks a block (never its parts): one entry per mixer it holds ---------------
    def cache_needs(self) -> list:
        return [self.mixer.cache_need()]

    def state_bytes(self) -> list:
        return [int(self.mixer.state_bytes())]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def tensors(self):
        t = {}
        for p in self.parts():
            t.update(p.tensors())
        return t

    def load(self, weights, device, dtype):
        for p in self.parts():
            p.load(weights, device, dtype)

    def first_norm(self):
        """The norm that this block applies to the residual first, if the part behind it can take a norm's output in
        two pieces (parts.base.Prenormed): the block before may then prepare it in its last product."""
        return self.norm1 if getattr(self.mixer, "takes_prenormed", False) else None

    def forward(self, residual, ctx, slots) -> None:
        x = self.norm1.forward(residual, ctx, ctx.dtype)      # what the block before left behind, or the norm's own kernel
        if isinstance(x, Prenormed) and not getattr(self.mixer, "takes_prenormed", False):
            x = x.materialize(ctx)
        # what the feed-forward streams first, for a mixer whose last kernel can ask for it ahead of time
        ctx.weights_ahead = getattr(self.feed_forward, "first_weights", lambda: None)()
        # the norm that comes next, for a mixer whose last product can prepare it
        ctx.norm_ahead = self.norm2 if getattr(self.feed_forward, "takes_prenormed", False) else None
        self.mixer.forward(x, residual, ctx, slots[0])
        ctx.weights_ahead = ctx.norm_ahead = None
        x = self.norm2.forward(residual, ctx, ctx.dtype)
        if isinstance(x, Prenormed) and not getattr(self.feed_forward, "takes_prenormed", False):
            x = x.materialize(ctx)
        ctx.norm_ahead = ctx.next_first_norm
        self.feed_forward.forward(x, residual, ctx)
        ctx.norm_ahead = None


register_part("block", "pre_norm", PreNormBlock)
