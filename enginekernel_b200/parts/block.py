"""Pre-norm residual block: stream += mixer(norm(stream)); stream += ff(norm(stream)).
A layer without a feed-forward is the first half alone (and needs only ``pre_mixer``).

The add of a part's output is folded into the norm that follows it, so a block takes the
previous block's not-yet-added output (``pending``) and returns its own
(engine/ek_model.py:291-296, 312, 326-334).  Norms: ``pre_mixer``, ``pre_feed_forward``.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import register_part
from .base import Block, DeferredNorm
from .spec import TensorSpec


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    @classmethod
    def norm_names(cls, spec):
        return ["pre_mixer"]             # and "pre_feed_forward" when there is a feed-forward

    def __init__(self, spec, dtype, device, mixer, feed_forward, norms):
        super().__init__(spec, dtype, device, mixer, feed_forward, norms)
        if feed_forward is not None and "pre_feed_forward" not in norms:
            raise ValueError("block 'pre_norm' needs the norm 'pre_feed_forward' before its feed-forward")

    def first_norm(self):
        """The norm that takes this block's incoming ``pending``, if the part behind it can read
        a deferred norm; else None."""
        return self.norms["pre_mixer"] if self.mixer.takes_deferred_norm else None

    def forward(self, stream, pending, ctx, entry, writes_cache=True, next_norm=None):
        """``next_norm``: the norm that will take the returned ``pending`` (the next block's
        first), or None; with it the feed-forward may return a DeferredNorm."""
        if isinstance(pending, DeferredNorm):
            a = pending                          # made for pre_mixer by the block before
        else:
            a = self.norms["pre_mixer"].forward(stream, ctx, add=pending)
        if self.feed_forward is None:
            # the mixer's output is this block's pending; the block behind may take it deferred
            if self.mixer.defers_norm and next_norm is not None:
                return self.mixer.forward(a, ctx, entry, writes_cache, defer=(stream, next_norm))
            return self.mixer.forward(a, ctx, entry, writes_cache)
        if self.mixer.defers_norm and self.feed_forward.takes_deferred_norm:
            o = self.mixer.forward(a, ctx, entry, writes_cache,
                                   defer=(stream, self.norms["pre_feed_forward"]))
        else:
            o = self.mixer.forward(a, ctx, entry, writes_cache)
        m = o if isinstance(o, DeferredNorm) else self.norms["pre_feed_forward"].forward(stream, ctx, add=o)
        if self.feed_forward.defers_norm and next_norm is not None:
            return self.feed_forward.forward(m, ctx, defer=(stream, next_norm))
        return self.feed_forward.forward(m, ctx)


class ScaledSum:
    """What a ``parallel`` block leaves to be added to the stream: a * scale_a + b * scale_b (the
    scales 32-bit vectors of the stream's width or None; ``b`` None for a layer without feed-forward)."""
    __slots__ = ("a", "scale_a", "b", "scale_b")

    def __init__(self, a, scale_a, b=None, scale_b=None):
        self.a, self.scale_a, self.b, self.scale_b = a, scale_a, b, scale_b


@register_part("block", "parallel")
class ParallelBlock(Block):
    """One norm, two readers: with u = norm(stream), stream += s1 * mixer(u) + s2 * ff(u), where s1 and
    s2 are optional learned vectors of the stream's width (tensors ``mixer_scale``, ``feed_forward_scale``;
    a name left out of the weights means no scale).  A layer without a feed-forward is the first term
    alone.  The add - both terms multiplied by their scales and summed into the 32-bit stream - rides
    in the kernel of the next block's norm; the last block of a model does it in ``collapse``.  The
    norm must be gain * x * rsqrt(mean(x^2) + eps) over the row (``Norm.deferrable``).  Norm: ``pre_mixer``.
    """

    @classmethod
    def norm_names(cls, spec):
        return ["pre_mixer"]

    @classmethod
    def tensors(cls, spec):
        size = spec.params["hidden_size"]
        return [TensorSpec(spec.weights[n], (size,), "gain") for n in ("mixer_scale", "feed_forward_scale")
                if n in spec.weights]

    def __init__(self, spec, dtype, device, mixer, feed_forward, norms):
        super().__init__(spec, dtype, device, mixer, feed_forward, norms)
        if norms["pre_mixer"].deferrable() is None:
            raise ValueError("block 'parallel' needs a norm of the form gain * x * rsqrt(mean(x^2) + eps)")
        self.hidden = int(self.param("hidden_size"))
        self.scale_mixer = self.scale_ff = None

    def load(self, tensors):
        w = self.spec.weights
        if "mixer_scale" in w:
            self.scale_mixer = tensors[w["mixer_scale"]].to(torch.float32).contiguous()
        if "feed_forward_scale" in w and self.feed_forward is not None:
            self.scale_ff = tensors[w["feed_forward_scale"]].to(torch.float32).contiguous()

    def bytes_read_per_step(self, n_tokens):
        return sum(t.numel() * 4 for t in (self.scale_mixer, self.scale_ff) if t is not None)

    def _normed(self, stream, pending, ctx):
        norm = self.norms["pre_mixer"]
        if not isinstance(pending, ScaledSum):
            return norm.forward(stream, ctx, add=pending)
        gain, eps = norm.deferrable()
        y = ctx.workspace.get("normed", (ctx.n_tokens, self.hidden), self.dtype)
        kernels.rmsnorm_scaled_sum(y, stream, pending.a, gain, eps, scale_a=pending.scale_a, b=pending.b,
                                   scale_b=pending.scale_b, n_rows=ctx.n_tokens)
        return y

    def collapse(self, stream, pending, ctx):
        if isinstance(pending, ScaledSum):
            kernels.add_scaled(stream, pending.a, pending.scale_a, pending.b, pending.scale_b, n_rows=ctx.n_tokens)
            pending = None
        return stream, pending

    def forward(self, stream, pending, ctx, entry, writes_cache=True):
        u = self._normed(stream, pending, ctx)
        # (the two outputs live in different workspace buffers: "attn_proj" and the feed-forward's own)
        a = self.mixer.forward(u, ctx, entry, writes_cache)
        b = self.feed_forward.forward(u, ctx) if self.feed_forward is not None else None
        return ScaledSum(a, self.scale_mixer, b, self.scale_ff)
