"""Arrangement of a mixer and a feed-forward in one layer.

"prenorm": x += mixer(norm(x)); x += feed_forward(norm(x)), the second only where the layer has a
feed-forward (cuongvng/bare-cuda-4gib engine/src/model.cpp:526-604).  Each add is carried out by the norm
that follows it, so a layer hands its last contribution on, not yet added, as `pending` - unless
the part's last kernel added it into the residual stream itself (`ctx.residual`), in which case the
part returns None.
"""

from __future__ import annotations

from .registry import build_part, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, layer_spec):
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.has_ffn = layer_spec.ffn is not None
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm) if self.has_ffn else None
        self.ffn = build_part("feed_forward", layer_spec.ffn) if self.has_ffn else None

    def parts(self):
        return [self.mixer_norm, self.mixer] + ([self.ffn_norm, self.ffn] if self.has_ffn else [])

    def cache_demands(self):
        """What this layer keeps per request: its mixer's paged cache and state."""
        return [(self.mixer.cache_request(), self.mixer.state_request())]

    def forward(self, ctx, call, residual, pending):
        n = ctx.n_tokens
        ctx.residual = residual      # a part may add its contribution here itself and return None
        after = getattr(ctx, "norm_after_layer", None)
        h = self.mixer_norm.forward(ctx, residual, pending, n, lazy=getattr(self.mixer, "takes_lazy_input", False))
        ctx.following_norm = self.ffn_norm if self.has_ffn else after     # the norm that reads the stream next
        mixed = self.mixer.forward(ctx, call, h)
        if not self.has_ffn:
            ctx.following_norm = None
            return mixed
        h = self.ffn_norm.forward(ctx, residual, mixed, n, lazy=getattr(self.ffn, "takes_lazy_input", False))
        ctx.following_norm = after
        out = self.ffn.forward(ctx, h)
        ctx.following_norm = None
        return out

    def entry_norm(self):
        """The norm that reads the residual stream first when this layer runs."""
        return self.mixer_norm


@register_block("sandwich")
class SandwichBlock:
    """x += norm_b(mixer(norm(x))), then (if the layer has a feed-forward) the same around it.  The
    norms behind the sublayers are `layer_spec.extras["post1"]` and `["post2"]`.  A sublayer's result is
    handed on un-normed and un-added; the norm that reads the stream next does both first."""

    def __init__(self, layer_spec):
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.post1 = build_part("norm", layer_spec.extras["post1"])
        self.has_ffn = layer_spec.ffn is not None
        if self.has_ffn:
            self.ffn_norm = build_part("norm", layer_spec.ffn_norm)
            self.ffn = build_part("feed_forward", layer_spec.ffn)
            self.post2 = build_part("norm", layer_spec.extras["post2"])

    def parts(self):
        out = [self.mixer_norm, self.mixer, self.post1]
        if self.has_ffn:
            out += [self.ffn_norm, self.ffn, self.post2]
        return out

    def cache_demands(self):
        many = getattr(self.mixer, "cache_demands", None)
        return many() if many else [(self.mixer.cache_request(), self.mixer.state_request())]

    def entry_norm(self):
        return self.mixer_norm

    def forward(self, ctx, call, residual, pending):
        n = ctx.n_tokens
        ctx.residual = None          # sublayers hand their result back: it is normed before it is added
        ctx.following_norm = None
        h = self.mixer_norm.forward(ctx, residual, pending, n)
        pending = self.post1.pending(self.mixer.forward(ctx, call, h))
        if self.has_ffn:
            h = self.ffn_norm.forward(ctx, residual, pending, n)
            pending = self.post2.pending(self.ffn.forward(ctx, h))
        return pending
