"""Arrangement of a layer's parts: pre-norm with two residual adds,

    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))

(model/qwen3_graph.go:76-100). The residual stream h is float32. Each add is left
pending and handed to the next norm, which does it in its own kernel.
"""
from __future__ import annotations

import inspect

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
        # a part whose forward takes `residual` may add its result to the stream itself
        # every part reaches the device through the package's kernels only: its products may
        # be collected into chains (see kernels/ops.py begin_chain)
        self.chain_safe = all(getattr(part, "chain_safe", False)
                              for part in (self.mixer, self.feed_forward)) and \
            hasattr(self.norm1, "lazy") and hasattr(self.norm2, "lazy")
        self._mixer_adds = "residual" in inspect.signature(self.mixer.forward).parameters
        self._ffn_adds = "residual" in inspect.signature(self.feed_forward.forward).parameters

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

    def _normed(self, norm, part, h, pending, ctx):
        if getattr(part, "takes_normed_rows", False) and hasattr(norm, "lazy"):
            return norm.lazy(h, pending, ctx.act_dtype)
        return norm.forward(h, pending, ctx.act_dtype)

    def forward(self, h, pending, ctx, cache):
        n = self._normed(self.norm1, self.mixer, h, pending, ctx)
        if self._mixer_adds:
            a = self.mixer.forward(n, ctx, cache, residual=h)
        else:
            a = self.mixer.forward(n, ctx, cache)
        n = self._normed(self.norm2, self.feed_forward, h, a, ctx)
        if self._ffn_adds:
            return h, self.feed_forward.forward(n, ctx, residual=h)
        return h, self.feed_forward.forward(n, ctx)


BLOCKS.register("prenorm_residual", PreNormResidual)
