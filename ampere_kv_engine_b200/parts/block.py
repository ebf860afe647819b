"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))`` (ampere_kv/runner.py:117-121
and 156-179).  The residual stream is float32; each branch output is handed to the next norm
as a pending ``delta`` so that the sum and the norm are one kernel.  On decode steps the branch's
last product may add to the stream itself and the next product apply the norm (``Summed``,
``LazyNorm``): then no kernel stands between the two products.
"""

from __future__ import annotations

from ..kernels import ops
from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    """roles: ``mixer_norm``, ``mixer``, ``feed_forward_norm``, ``feed_forward``.  A layer spec without a
    feed-forward makes a layer of the mixer branch alone."""

    def __init__(self, layer, **kw):
        super().__init__(layer, **kw)
        self.mixer_norm = self.build_role("mixer_norm")
        self.mixer = self.build_role("mixer")
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = self.build_role("feed_forward_norm")
            self.feed_forward = self.build_role("feed_forward")

    def forward(self, hidden, delta, ctx, cache):
        x = self.run_norm(self.mixer_norm, hidden, delta, ctx, consumer=self.mixer)
        attn = self.run_branch(self.mixer, hidden, x, ctx, cache)
        if self.feed_forward is None:
            return hidden, attn
        x = self.run_norm(self.feed_forward_norm, hidden, attn, ctx, consumer=self.feed_forward)
        return hidden, self.run_branch(self.feed_forward, hidden, x, ctx)


@register_block("postnorm")
class PostNormBlock(Block):
    """``h += norm1(mixer(h)); h += norm2(feed_forward(h))``: the branches read the stream itself and each norm sits
    on its branch's output.  roles as ``prenorm``; the norms must offer ``add_normed``.  The stream is float32; in
    bfloat16 every ``add_normed`` also leaves the stream's rounded copy, which the next branch reads and which
    travels to the next block as an ``ops.Mirrored`` in place of a pending delta."""

    def __init__(self, layer, **kw):
        super().__init__(layer, **kw)
        self.mixer = self.build_role("mixer")
        self.mixer_norm = self.build_role("mixer_norm")
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward = self.build_role("feed_forward")
            self.feed_forward_norm = self.build_role("feed_forward_norm")
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError(f"block kind 'postnorm': norm kind {norm.spec.kind!r} cannot norm a branch's output")

    def forward(self, hidden, delta, ctx, cache):
        if isinstance(delta, ops.Mirrored) and delta.hidden is hidden:
            x = delta.copy
        else:
            if isinstance(delta, ops.PendingPhases):
                delta.launch()
                delta = None
            if delta is not None and not isinstance(delta, (ops.Summed, ops.Mirrored)):
                raise ValueError("block kind 'postnorm' follows a block that leaves its last branch unadded; "
                                 "put a norm that adds it between them")
            x = ops.stream_copy(hidden, self.dtype)
        x = self.mixer_norm.add_normed(hidden, self.mixer.forward(x, ctx, cache), ctx)
        if self.feed_forward is not None:
            # a feed-forward whose result is still a sum of rows leaves the sum to a norm that can do it
            if getattr(self.feed_forward, "defers_sum", False) and getattr(self.feed_forward_norm, "takes_parts", False):
                branch = self.feed_forward.forward(x, ctx, defer_sum=True)
            else:
                branch = self.feed_forward.forward(x, ctx)
            x = self.feed_forward_norm.add_normed(hidden, branch, ctx)
        return hidden, ops.Mirrored(hidden, x)
