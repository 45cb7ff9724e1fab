"""Arrangements of a layer's parts.

`PreNormBlock`, the reference's decoder layer (src/paged/qwen3.rs:932-939):
    h = norm1(x); x = x + mixer(h); h = norm2(x); x = x + feed_forward(h)

The residual stream x is float32.  A sublayer's output is not added at once:
it travels as `delta` to the next norm, whose kernel forms x + delta in float32,
stores it and norms it in one pass.  A block therefore takes (residual, delta)
and returns (residual, delta); the model adds the last delta in its final norm.

`SandwichNormBlock`: a norm before AND after each sublayer, and a multiplier m on both branches:
    x = x + m * norm1b(mixer(norm1(x)));  x = x + m * norm2b(feed_forward(norm2(x)))
(the second line falls away in a layer without a feed-forward).  The norm after a sublayer, the scaled
residual update and the norm before the next sublayer are one kernel; a mixer made of two members
(`forward_branches`) has its members' norms and their sum done there too.  The residual is complete when the
block returns, so it hands on no delta.

`PostNormBlock`: a norm on each sublayer's OUTPUT only; the sublayers read the stream itself:
    x = x + norm1(mixer(x));  x = x + norm2(feed_forward(x))
(the second line falls away in a layer without a feed-forward).  The sublayers' input is the float32 stream
rounded to the engine's element type; the kernel that norms a sublayer's output and updates the residual
also writes that rounding for the next sublayer, and the last one of a block leaves it in `ctx.rounded` for
the next block.
"""
from __future__ import annotations

from ..csrc import ops
from .base import Block


class PreNormBlock(Block):
    norm_names = ("mixer", "feed_forward")

    def forward(self, residual, delta, ctx, cache):
        h = self.norms["mixer"].add_norm(residual, delta)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norms["feed_forward"].add_norm(residual, a)
        f = self.feed_forward.forward(h, ctx)
        return residual, f


class PostNormBlock(Block):
    needs_feed_forward = False
    leaves_rounded = True

    def __init__(self, mixer, feed_forward, norms):
        self.norm_names = ("mixer_out",) + (("feed_forward_out",) if feed_forward is not None else ())
        super().__init__(mixer, feed_forward, norms)
        for name, n in self.norms.items():
            if not hasattr(n, "weight") or not hasattr(n, "eps"):
                raise ValueError("PostNormBlock fuses its norms into the residual update and takes RMS norms; %r is %s"
                                 % (name, type(n).__name__))

    def forward(self, residual, delta, ctx, cache):
        n = self.norms
        dtype = self.mixer.runtime.dtype
        if delta is not None:   # (a block before this one left a sublayer's output to be added)
            residual.add_(delta)
            ctx.rounded = None
        carried = ctx.rounded
        if carried is not None and carried[0] is residual and carried[1].dtype == dtype:
            h = carried[1]
        else:
            h = ops.cast_rows(residual, dtype)
        y = self.mixer.forward(h, ctx, cache)
        h = ops.merge_norm_add_norm(residual, y, n["mixer_out"].weight, 1.0, n["mixer_out"].eps, rounded=True)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, ctx)
            h = ops.merge_norm_add_norm(residual, f, n["feed_forward_out"].weight, 1.0, n["feed_forward_out"].eps, rounded=True)
        ctx.rounded = (residual, h)
        return residual, None


class SandwichNormBlock(Block):
    needs_feed_forward = False

    def __init__(self, mixer, feed_forward, norms, residual_mult: float = 1.0):
        self.norm_names = ("mixer", "mixer_out") + (("feed_forward", "feed_forward_out") if feed_forward is not None else ())
        super().__init__(mixer, feed_forward, norms)
        self.residual_mult = float(residual_mult)
        for name, n in self.norms.items():
            if not hasattr(n, "weight") or not hasattr(n, "eps"):
                raise ValueError("SandwichNormBlock fuses its norms into one kernel and takes RMS norms; %r is %s"
                                 % (name, type(n).__name__))

    def forward(self, residual, delta, ctx, cache):
        n, m = self.norms, self.residual_mult
        h = n["mixer"].add_norm(residual, delta)
        after, eps = n["mixer_out"], n["mixer_out"].eps
        w_next = n["feed_forward"].weight if self.feed_forward is not None else None
        if hasattr(self.mixer, "forward_branches") and getattr(self.mixer, "eps", eps) == eps:
            (y0, w0, c0), (y1, w1, c1) = self.mixer.forward_branches(h, ctx, cache)
            h = ops.merge_norm_add_norm(residual, y0, after.weight, m, eps, w0, c0, y1, w1, c1, w_next=w_next)
        else:
            h = ops.merge_norm_add_norm(residual, self.mixer.forward(h, ctx, cache), after.weight, m, eps, w_next=w_next)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, ctx)
            ops.merge_norm_add_norm(residual, f, n["feed_forward_out"].weight, m, n["feed_forward_out"].eps)
        return residual, None
