"""Arrangement of a layer's parts.  `PreNormBlock` is the reference's layer
(src/engine/cpu_backend.zig:258-325): norm -> mixer -> residual sum -> norm -> feed-forward
-> residual sum.  The residual stream is float32; the mixer and the feed-forward add onto
it in place.  A block says which caches it keeps (`cache_specs()`, here those of its mixer)
and is handed exactly those, so a block with two mixers, or with none, is a block like any other.
`PreNormBlock` may go without a feed-forward, and may end with one more part that reads and changes the residual
stream (`after`: a per-layer token input, for instance)."""
from __future__ import annotations

import torch

from .base import Part, register_part
from .parallel import mixer_cache_specs, mixer_caches


class PreNormBlock(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, mixer_norm, mixer, ffn_norm=None, feed_forward=None, after=None):
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("a feed-forward comes with its norm, or neither is given")
        self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward = mixer_norm, mixer, ffn_norm, feed_forward
        self.after = after          # forward(residual, ctx): one more sublayer behind the feed-forward

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward, self.after) if p is not None)

    def cache_specs(self):
        """The mixer's caches: one, or as many as it names."""
        return mixer_cache_specs(self.mixer)

    def forward(self, residual: torch.Tensor, ctx, caches, write_cache: bool = True) -> None:
        xb = torch.empty(residual.shape, dtype=ctx.precision.compute, device=residual.device)
        self.mixer_norm.forward(residual, xb)
        self.mixer.forward(xb, residual, ctx, mixer_caches(self.mixer, caches), write_cache)
        if self.feed_forward is not None:
            self.ffn_norm.forward(residual, xb)
            self.feed_forward.forward(xb, residual, ctx)
        if self.after is not None:
            self.after.forward(residual, ctx)


register_part("block", "pre_norm", PreNormBlock)


class SandwichNormBlock(Part):
    """A layer that norms both sides of each sublayer:
        x <- x + post_mixer_norm(mixer(mixer_norm(x)));   x <- x + post_ffn_norm(ffn(ffn_norm(x)))
    The sublayer writes its float32 result into a buffer (`accumulate=False`); the norm behind it is fused with
    the residual sum (`ops.rms_norm_add`).  Without a feed-forward (`feed_forward=None`) the second half is absent.
    The norms are RMSNorm parts; their eps may differ."""
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, mixer_norm, mixer, post_mixer_norm, ffn_norm=None, feed_forward=None, post_ffn_norm=None):
        if (feed_forward is None) != (ffn_norm is None) or (feed_forward is None) != (post_ffn_norm is None):
            raise ValueError("a feed-forward comes with both of its norms, or none of the three is given")
        self.mixer_norm, self.mixer, self.post_mixer_norm = mixer_norm, mixer, post_mixer_norm
        self.ffn_norm, self.feed_forward, self.post_ffn_norm = ffn_norm, feed_forward, post_ffn_norm

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.post_mixer_norm, self.ffn_norm, self.feed_forward,
                                 self.post_ffn_norm) if p is not None)

    def cache_specs(self):
        return [self.mixer.cache_spec()]

    def forward(self, residual: torch.Tensor, ctx, caches, write_cache: bool = True) -> None:
        from ..csrc import ops
        xb = torch.empty(residual.shape, dtype=ctx.precision.compute, device=residual.device)
        y = torch.empty_like(residual)
        self.mixer_norm.forward(residual, xb)
        self.mixer.forward(xb, y, ctx, caches[0], write_cache, accumulate=False)
        ops.rms_norm_add(y, self.post_mixer_norm.weight, self.post_mixer_norm.eps, residual)
        if self.feed_forward is not None:
            self.ffn_norm.forward(residual, xb)
            self.feed_forward.forward(xb, y, ctx, accumulate=False)
            ops.rms_norm_add(y, self.post_ffn_norm.weight, self.post_ffn_norm.eps, residual)


register_part("block", "sandwich_norm", SandwichNormBlock)


class PostNormBlock(Part):
    """A layer that norms only what its sublayers give back:
        x <- x + post_mixer_norm(mixer(x));   x <- x + post_ffn_norm(ffn(x))
    The sublayers read the residual stream itself.  In 32-bit that is the residual tensor; when serving, the
    bfloat16 copy that the products read is written by the kernel that last changed the residual (the norm + residual
    sum of the sublayer before, or the embedding) and handed on through `ctx.residual_narrow`.  Without a feed-forward
    the second half is absent."""
    graph_safe = True   # reads the batch from device tensors only
    keeps_narrow_residual = True

    def __init__(self, mixer, post_mixer_norm, feed_forward=None, post_ffn_norm=None):
        if (feed_forward is None) != (post_ffn_norm is None):
            raise ValueError("a feed-forward comes with its norm, or neither is given")
        self.mixer, self.post_mixer_norm = mixer, post_mixer_norm
        self.feed_forward, self.post_ffn_norm = feed_forward, post_ffn_norm

    def children(self):
        return tuple(p for p in (self.mixer, self.post_mixer_norm, self.feed_forward, self.post_ffn_norm) if p is not None)

    def cache_specs(self):
        return [self.mixer.cache_spec()]

    def forward(self, residual: torch.Tensor, ctx, caches, write_cache: bool = True) -> None:
        from ..csrc import ops
        narrow = ctx.precision.compute != torch.float32
        if not narrow:
            xb = residual                       # the sublayers read it and write elsewhere
        else:
            xb = getattr(ctx, "residual_narrow", None)
            if xb is None:                      # whoever changed the residual last left no copy
                xb = torch.empty(residual.shape, dtype=ctx.precision.compute, device=residual.device)
                xb.copy_(residual)
        y = torch.empty_like(residual)
        self.mixer.forward(xb, y, ctx, caches[0], write_cache, accumulate=False)
        ops.rms_norm_add(y, self.post_mixer_norm.weight, self.post_mixer_norm.eps, residual, xb if narrow else None)
        if self.feed_forward is not None:
            self.feed_forward.forward(xb, y, ctx, accumulate=False)
            ops.rms_norm_add(y, self.post_ffn_norm.weight, self.post_ffn_norm.eps, residual, xb if narrow else None)
        ctx.residual_narrow = xb if narrow else None


register_part("block", "post_norm", PostNormBlock)
