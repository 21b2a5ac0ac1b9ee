"""Arrangement of a layer's parts.  `prenorm_residual` is the reference's
(src/models/turbo_generic.rs:1959-1981): h += mixer(norm1(h));
h += feed_forward(norm2(h)), with the sums done in float32 on the residual
stream.

A block kind is a class built from a `LayerSpec` with `parts()` (every part
it holds, for weights and binding), `mixer` (the one part that may ask for a
cache or state) and `forward(h, ctx)`.  It takes the parts it arranges from
the layer by name (`spec.part("mixer")`, or any name of `extra_parts`)."""
from __future__ import annotations

from .. import kernels
from ..config import LayerSpec
from .base import StepContext
from .registry import make_part


class PrenormResidualBlock:
    padded_rows_ok = True               # as far as its parts are

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = make_part(spec.part("mixer_norm"))
        self.mixer = make_part(spec.part("mixer"))
        # a layer may name no feed-forward: it then has the mixer's sublayer only
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = make_part(spec.part("feed_forward_norm"))
            self.feed_forward = make_part(spec.part("feed_forward"))

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def forward(self, h, ctx: StepContext) -> None:
        act = ctx.runtime.act_dtype
        x = self._normed(self.mixer_norm, self.mixer, h, act)
        kernels.mark("norms")
        self.mixer.forward(x, ctx, h)
        if self.feed_forward is None:
            return
        x = self._normed(self.feed_forward_norm, self.feed_forward, h, act)
        kernels.mark("norms")
        self.feed_forward.forward(x, ctx, h)

    @staticmethod
    def _normed(norm, consumer, h, act):
        """The norm's result for `consumer` — left pending if the consumer only hands it to `kernels.linear`
        (it says so with `takes_pending_norm`) and the norm can be deferred, so that the product may fold it in."""
        if getattr(consumer, "takes_pending_norm", False) and getattr(norm, "pending", None) is not None:
            return norm.pending(h, act)
        return norm.forward(h, act)


class ParallelResidualBlock:
    """h += mult * (mixer(n) + feed_forward(n)) with ONE norm n = norm(h): both sublayers read the same normed
    rows, their results are added in float32 and enter the residual stream times `residual_mult` (a block
    parameter, 1 by default).  A layer may name no feed-forward."""
    padded_rows_ok = True               # as far as its parts are

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mult = float(spec.block_params.get("residual_mult", 1.0))
        self.mixer_norm = make_part(spec.part("mixer_norm"))
        self.mixer = make_part(spec.part("mixer"))
        self.feed_forward = make_part(spec.part("feed_forward")) if spec.feed_forward is not None else None

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward) if p is not None]

    def forward(self, h, ctx: StepContext) -> None:
        x = self.mixer_norm.forward(h, ctx.runtime.act_dtype)       # run once: two readers
        kernels.mark("norms")
        if self.mult == 1.0:
            self.mixer.forward(x, ctx, h)
            if self.feed_forward is not None:
                self.feed_forward.forward(x, ctx, h)
            return
        import torch
        y = torch.zeros_like(h)                                     # the sublayers add their results into it
        self.mixer.forward(x, ctx, y)
        if self.feed_forward is not None:
            self.feed_forward.forward(x, ctx, y)
        kernels.add_scaled(h, y, self.mult)
        kernels.mark("norms")


class PostnormResidualBlock:
    """h += norm1(mixer(h));  h += norm2(feed_forward(h)): the sublayers read the stream itself (rounded to the
    activations' type where that is not float32) and the norm works on what they give.  Each sublayer stores its
    result into a float32 buffer of its own (parts that say `can_store_result` write it without a cleared buffer);
    one kernel then norms the buffer, adds it to the stream and leaves the rounded stream for the next reader.
    The rounded stream travels from layer to layer as an attribute of the stream tensor, so a layer's first
    sublayer does not round again what the layer before has rounded.  A layer may name no feed-forward."""
    padded_rows_ok = True               # as far as its parts are

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer = make_part(spec.part("mixer"))
        self.mixer_norm = make_part(spec.part("mixer_norm"))
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = make_part(spec.part("feed_forward"))
            self.feed_forward_norm = make_part(spec.part("feed_forward_norm"))

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm) if p is not None]

    def forward(self, h, ctx: StepContext) -> None:
        import torch
        act = ctx.runtime.act_dtype
        rounded = getattr(h, ROUNDED, None)
        if rounded is not None:
            delattr(h, ROUNDED)
        for part, norm in ((self.mixer, self.mixer_norm), (self.feed_forward, self.feed_forward_norm)):
            if part is None:
                continue
            if act == torch.float32:
                x = h
            else:
                x = rounded if rounded is not None else kernels.round_rows(h)
                kernels.mark("norms")
            store = getattr(part, "can_store_result", False)
            y = torch.empty_like(h) if store else torch.zeros_like(h)
            ctx.store_result = store
            try:
                part.forward(x, ctx, y)
            finally:
                ctx.store_result = False
            rounded = None if act == torch.float32 else torch.empty(h.shape, dtype=act, device=h.device)
            kernels.add_normed_copy(h, y, norm.weight, norm.eps, rounded)
            kernels.mark("norms")
        if rounded is not None:
            setattr(h, ROUNDED, rounded)


ROUNDED = "_tq_rounded_copy"      # attribute of the stream tensor: the copy a block left for the next block's reader
