"""Block arrangements.  `pre_norm` is the only one the reference runs on the
GPU (`model.py:262-264`, `engine/src/gpu_model.rs:518-520`):
x = x + mixer(norm(x)); x = x + ffn(norm(x)).  `parallel` has one norm that both
sublayers read: with n = norm(x), x = x + mixer(n) + ffn(n)."""
from __future__ import annotations

from .base import ARRANGEMENTS, Arrangement


class PreNormBlock(Arrangement):
    norm_names = ("mixer_norm", "feed_forward_norm")

    def __init__(self, spec, norms, mixer, feed_forward):
        # a layer without a feed-forward sublayer (a part with `absent`) has one norm only
        self.has_ffn = not getattr(feed_forward, "absent", False)
        if not self.has_ffn:
            self.norm_names = ("mixer_norm",)
        super().__init__(spec, norms, mixer, feed_forward)

    def forward(self, ctx, x, binding):
        h = self._norm(ctx, self.norms["mixer_norm"], self.mixer, x)
        if not self.has_ffn:
            self._announce(ctx, getattr(ctx, "norm_after_layer", None), x)
            self.mixer.forward(ctx, h, x, binding)
            return
        self._announce(ctx, (self.norms["feed_forward_norm"], self.feed_forward), x)
        self.mixer.forward(ctx, h, x, binding)
        h = self._norm(ctx, self.norms["feed_forward_norm"], self.feed_forward, x)
        self._announce(ctx, getattr(ctx, "norm_after_layer", None), x)
        self.feed_forward.forward(ctx, h, x)

    def entry_norm(self):
        """(norm, its consumer): the first reader of the rows this layer is given."""
        return self.norms["mixer_norm"], self.mixer

    @staticmethod
    def _announce(ctx, ahead, x):
        # the part that runs now writes x last before `ahead`'s norm reads it: its last product
        # may leave that norm's input (StepContext.announce_norm)
        announce = getattr(ctx, "announce_norm", None)
        if announce is None:
            return
        norm, consumer = ahead if ahead is not None else (None, None)
        # (a consumer with `takes_prenormed = False` fuses the norm of a few rows into its first
        # product but has no product that takes rows a product before it left ahead of their norm)
        if (norm is not None and getattr(consumer, "fuses_norm", False)
                and getattr(consumer, "takes_prenormed", True)
                and getattr(norm, "supports_ahead", False)):
            announce(norm, x)
        else:
            announce(None, None)

    @staticmethod
    def _norm(ctx, norm, consumer, x):
        # a consumer that can fuse the norm into its first product (`fuses_norm`)
        # may be handed rows that are not yet normalised, if the norm offers that
        if getattr(consumer, "fuses_norm", False) and getattr(norm, "supports_lazy", False):
            return norm.forward(ctx, x, lazy=True)
        return norm.forward(ctx, x)


class ParallelBlock(Arrangement):
    """One norm, two readers: n = norm(x); x += mixer(n); x += ffn(n).  Both sublayers add
    their results into the fp32 residual, so the layer's sum is a 32-bit sum; the order of
    the two additions is fixed.  A feed-forward part with `absent` leaves the mixer alone."""
    norm_names = ("norm",)

    def __init__(self, spec, norms, mixer, feed_forward):
        self.has_ffn = not getattr(feed_forward, "absent", False)
        super().__init__(spec, norms, mixer, feed_forward)

    def forward(self, ctx, x, binding):
        announce = getattr(ctx, "announce_norm", None)
        if announce is not None:
            announce(None, None)       # the rows' next norm reads them after BOTH sublayers
        n = self.norms["norm"].forward(ctx, x)
        self.mixer.forward(ctx, n, x, binding)
        if self.has_ffn:
            self.feed_forward.forward(ctx, n, x)


ARRANGEMENTS.register("pre_norm", PreNormBlock)
ARRANGEMENTS.register("parallel", ParallelBlock)
