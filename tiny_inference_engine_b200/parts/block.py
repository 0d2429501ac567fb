"""Pre-norm arrangement of a layer: x += mixer(norm(x)); x += ffn(norm(x))
(src/model/qwen3.cpp:214-239). Each residual add is fused with the norm that follows it, so
the feed-forward's output is handed on as a pending delta that the next layer's first norm
(or the final norm) adds."""
from __future__ import annotations

from .base import Block, build_part, register_part


class PreNormBlock(Block):
    launches_only = True

    def __init__(self, layer_spec, dtype, prefix: str = ""):
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, dtype)
        self.mixer = build_part("mixer", layer_spec.mixer, dtype)
        self.has_ffn = layer_spec.ffn is not None          # a layer may be a mixer alone
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm, dtype) if self.has_ffn else None
        self.ffn = build_part("feed_forward", layer_spec.ffn, dtype) if self.has_ffn else None
        self.dtype = dtype
        self.parts = (self.mixer_norm, self.mixer) + ((self.ffn_norm, self.ffn) if self.has_ffn else ())

    def needs(self):
        n = {}
        for p in self.parts:
            n.update(p.needs())
        return n

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def forward(self, x, pending, ctx, cache, state):
        """`pending` and what the parts return may be tensors [T, D] or ops.SplitSum (a split product
        whose partial sums the next add+norm adds up itself)."""
        h = ctx.ws.rows("block.normed", x.shape[0], x.shape[1], self.dtype)
        self.mixer_norm.add_norm(x, as_delta(pending, self.mixer_norm, ctx, "block.delta"), h)
        mixed = self.mixer.forward(h, ctx, cache, state)
        if not self.has_ffn:
            return mixed
        self.ffn_norm.add_norm(x, as_delta(mixed, self.ffn_norm, ctx, "block.delta"), h)
        return self.ffn.forward(h, ctx)


def as_delta(delta, norm, ctx, name):
    """A SplitSum stays one for norms that add the splits themselves (`takes_split_sum`), else it is added up first."""
    from .. import ops
    if isinstance(delta, ops.SplitSum) and not getattr(norm, "takes_split_sum", False):
        return delta.materialize(ctx.ws.rows(name, delta.M, delta.N, ctx.ws_dtype))
    return delta


class SandwichNormBlock(Block):
    """A norm before and after each sublayer, and a factor on what joins the residual stream:

        x += mult * norm_b(mixer(norm_a(x)));   x += mult * norm_d(ffn(norm_c(x)))

    A layer may have no feed-forward (`LayerSpec.ffn` None): then it is the first line alone. A sublayer's output
    is handed on as an `ops.NormedDelta` (the raw output, the weight and eps of the norm it still has to pass, the
    factor, and a bias of the sublayer's last product where it has one: a mixer says so with an `output_bias`
    attribute, float32 [D]); the add+norm ahead of the next sublayer (or the model's final norm) finishes it, all in
    float32. params: `residual_mult`."""
    launches_only = False

    def __init__(self, layer_spec, dtype, prefix: str = ""):
        self.mult = float(layer_spec.block.params.get("residual_mult", 1.0))
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, dtype)
        self.mixer = build_part("mixer", layer_spec.mixer, dtype)
        self.mixer_post_norm = build_part("norm", layer_spec.mixer_post_norm, dtype)
        self.has_ffn = layer_spec.ffn is not None
        self.parts = (self.mixer_norm, self.mixer, self.mixer_post_norm)
        if self.has_ffn:
            self.ffn_norm = build_part("norm", layer_spec.ffn_norm, dtype)
            self.ffn = build_part("feed_forward", layer_spec.ffn, dtype)
            self.ffn_post_norm = build_part("norm", layer_spec.ffn_post_norm, dtype)
            self.parts += (self.ffn_norm, self.ffn, self.ffn_post_norm)
        self.dtype = dtype

    def needs(self):
        n = {}
        for p in self.parts:
            n.update(p.needs())
        return n

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def _normed(self, delta, norm, bias=None):
        from .. import ops
        return ops.NormedDelta(delta, norm.weight, norm.eps, self.mult, bias)

    def forward(self, x, pending, ctx, cache, state):
        h = ctx.ws.rows("block.normed", x.shape[0], x.shape[1], self.dtype)
        self.mixer_norm.add_norm(x, as_delta(pending, self.mixer_norm, ctx, "block.delta"), h)
        mixed = self._normed(self.mixer.forward(h, ctx, cache, state), self.mixer_post_norm,
                             getattr(self.mixer, "output_bias", None))
        if not self.has_ffn:
            return mixed
        self.ffn_norm.add_norm(x, mixed, h)
        return self._normed(self.ffn.forward(h, ctx), self.ffn_post_norm)


register_part("block", "prenorm", PreNormBlock, replace=True)
register_part("block", "sandwich_norm", SandwichNormBlock, replace=True)
