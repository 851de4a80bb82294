"""Block arrangements.  ``pre_norm``: stream += mixer(norm(stream)); stream += ff(norm(stream)).
A layer without a feed-forward is the first half alone (and needs only ``pre_mixer``).  ``parallel``: one norm,
two readers.  ``sandwich``: a norm before and behind each sublayer.

The add of a part's output is folded into the norm that follows it, so a block takes the
previous block's not-yet-added output (``pending``) and returns its own
(engine/ek_model.py:291-296, 312, 326-334).  Norms: ``pre_mixer``, ``pre_feed_forward``.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..registry import register_part
from .base import Block, DeferredNorm, WeightedPair
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


class PostNormed:
    """What a ``sandwich`` block leaves to be added to the stream: gain * n(a * weight_a + b * weight_b + bias),
    the norm being the sublayer's own second norm (``norm``; ``b`` and ``bias`` may be absent)."""
    __slots__ = ("a", "weight_a", "b", "weight_b", "bias", "norm")

    def __init__(self, result, norm, bias=None):
        if isinstance(result, WeightedPair):
            self.a, self.weight_a, self.b, self.weight_b = result.a, result.weight_a, result.b, result.weight_b
        else:
            self.a, self.weight_a, self.b, self.weight_b = result, 1.0, None, 1.0
        self.bias, self.norm = bias, norm


@register_part("block", "sandwich")
class SandwichBlock(Block):
    """A norm before and a norm behind every sublayer: stream += post_mixer(mixer(pre_mixer(stream))), then
    stream += post_feed_forward(ff(pre_feed_forward(stream))).  A layer without a feed-forward is the
    first half alone.  The norm behind a sublayer, the add and the norm before the next sublayer are one
    kernel over the row (``rmsnorm_post_add``); the last block of a model, or a block before something
    else reads the stream, does the norm and the add in ``collapse``.  All norms must be of the form
    gain * x * rsqrt(mean(x^2) + eps).  A mixer may return a :class:`~.base.WeightedPair`, and a
    feed-forward that can leave its last bias to the consumer (``forward(..., leave_bias=True)`` and
    ``output_bias``) is asked to.  Norms: ``pre_mixer``, ``post_mixer``, ``pre_feed_forward``,
    ``post_feed_forward``."""

    @classmethod
    def norm_names(cls, spec):
        return ["pre_mixer", "post_mixer"]          # and the two of the feed-forward when there is one

    def __init__(self, spec, dtype, device, mixer, feed_forward, norms):
        super().__init__(spec, dtype, device, mixer, feed_forward, norms)
        needed = ["pre_mixer", "post_mixer"] + (["pre_feed_forward", "post_feed_forward"] if feed_forward is not None else [])
        for n in needed:
            if n not in norms:
                raise ValueError(f"block 'sandwich' needs the norm {n!r}")
            if norms[n].deferrable() is None:
                raise ValueError("block 'sandwich' needs norms of the form gain * x * rsqrt(mean(x^2) + eps)")
        self.hidden = int(self.param("hidden_size"))
        self._ff_leaves_bias = feed_forward is not None and hasattr(feed_forward, "output_bias")

    def _join(self, stream, pending, ctx, norm=None):
        """Adds ``pending`` to the stream; with ``norm`` also returns that norm of the sum."""
        t = ctx.n_tokens
        y = None if norm is None else ctx.workspace.get("normed", (t, self.hidden), self.dtype)
        if isinstance(pending, PostNormed):
            gain_post, eps_post = pending.norm.deferrable()
            gain, eps = norm.deferrable() if norm is not None else (None, 0.0)
            kernels.rmsnorm_post_add(y, stream, pending.a, gain_post, eps_post, gain, eps, weight_a=pending.weight_a,
                                     b=pending.b, weight_b=pending.weight_b, bias=pending.bias, n_rows=t)
            return y
        if norm is None:
            if pending is not None:
                kernels.add_residual(stream, pending, n_rows=t)
            return None
        return norm.forward(stream, ctx, add=pending)

    def collapse(self, stream, pending, ctx):
        if isinstance(pending, PostNormed):
            self._join(stream, pending, ctx)
            pending = None
        return stream, pending

    def forward(self, stream, pending, ctx, entry, writes_cache=True):
        a = self._join(stream, pending, ctx, self.norms["pre_mixer"])
        mixed = PostNormed(self.mixer.forward(a, ctx, entry, writes_cache), self.norms["post_mixer"])
        if self.feed_forward is None:
            return mixed
        h = self._join(stream, mixed, ctx, self.norms["pre_feed_forward"])
        if self._ff_leaves_bias:
            f = self.feed_forward.forward(h, ctx, leave_bias=True)
            return PostNormed(f, self.norms["post_feed_forward"], bias=self.feed_forward.output_bias)
        return PostNormed(self.feed_forward.forward(h, ctx), self.norms["post_feed_forward"])
