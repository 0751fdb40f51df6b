"""Arrangement of a layer's parts: pre-norm with two residual adds,

    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))

(model/qwen3_graph.go:76-100). The residual stream h is float32. Each add is left
pending and handed to the next norm, which does it in its own kernel.
"""
from __future__ import annotations

from ..config.spec import LayerSpec
from ..registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .base import Part

DEFAULT_NAMES = {
    "mixer_norm": "input_layernorm.weight",
    "ffn_norm": "post_attention_layernorm.weight",
    "mixer": "self_attn.",
    "feed_forward": "mlp.",
}


class PreNormResidual(Part):
    def __init__(self, spec: LayerSpec, hidden: int, device=None):
        names = dict(DEFAULT_NAMES)
        names.update(dict(spec.names))
        p = spec.prefix
        self.norm1 = NORMS.get(spec.norm.kind)(spec.norm, hidden, p + names["mixer_norm"])
        self.norm2 = NORMS.get(spec.norm.kind)(spec.norm, hidden, p + names["ffn_norm"])
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, hidden, p + names["mixer"], device)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
            spec.feed_forward, hidden, p + names["feed_forward"], device)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def weight_specs(self):
        out = []
        for part in self.parts():
            out += part.weight_specs()
        return out

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def forward(self, h, pending, ctx, cache):
        n = self.norm1.forward(h, pending, ctx.act_dtype)
        a = self.mixer.forward(n, ctx, cache)
        n = self.norm2.forward(h, a, ctx.act_dtype)
        return h, self.feed_forward.forward(n, ctx)


BLOCKS.register("prenorm_residual", PreNormResidual)
