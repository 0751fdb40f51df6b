"""Arrangement of a layer's parts: pre-norm with two residual adds,

    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))

(model/qwen3_graph.go:76-100). The residual stream h is float32. Each add is left
pending and handed to the next norm, which does it in its own kernel. The two norms'
checkpoint names come from the layer spec's `tensors` table (roles mixer_norm, ffn_norm).
"""
from __future__ import annotations

import inspect

from ..config.spec import LayerSpec, tensor_names
from ..registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .base import Part, offered


class PreNormResidual(Part):
    def __init__(self, spec: LayerSpec, hidden: int, device=None):
        p = spec.prefix
        names = tensor_names(spec.tensors, p, ["mixer_norm", "ffn_norm"], "pre-norm block")
        self.norm1 = NORMS.get(spec.norm.kind)(spec.norm, hidden, names["mixer_norm"])
        self.norm2 = NORMS.get(spec.norm.kind)(spec.norm, hidden, names["ffn_norm"])
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, hidden, p, device)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
            spec.feed_forward, hidden, p, device)
        # a part whose forward takes `residual` may add its result to the stream itself
        self._mixer_adds = "residual" in inspect.signature(self.mixer.forward).parameters
        self._ffn_adds = "residual" in inspect.signature(self.feed_forward.forward).parameters
        # a part with `lazy_rows` set takes its input as ops.NormedRows (a norm it may fold
        # into its first product), if the norm knows how to hand that on
        self._lazy1 = getattr(self.mixer, "lazy_rows", False) and \
            "lazy" in inspect.signature(self.norm1.forward).parameters
        self._lazy2 = getattr(self.feed_forward, "lazy_rows", False) and \
            "lazy" in inspect.signature(self.norm2.forward).parameters

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

    def libraries(self, dtype, page_size):
        out = []
        for part in self.parts():
            out += offered(part, "libraries")(dtype, page_size)
        return out

    def prepare_capture(self, ctx, cache):
        for part in self.parts():
            offered(part, "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, writes_cache=True):
        return sum(offered(part, "flops")(extents, first_positions, writes_cache)
                   for part in self.parts())

    def cache_bytes_read(self, context_len, width):
        return offered(self.mixer, "cache_bytes_read")(context_len, width)

    def forward(self, h, pending, ctx, cache):
        n = self.norm1.forward(h, pending, ctx.act_dtype, lazy=True) if self._lazy1 else \
            self.norm1.forward(h, pending, ctx.act_dtype)
        if self._mixer_adds:
            a = self.mixer.forward(n, ctx, cache, residual=h)
        else:
            a = self.mixer.forward(n, ctx, cache)
        n = self.norm2.forward(h, a, ctx.act_dtype, lazy=True) if self._lazy2 else \
            self.norm2.forward(h, a, ctx.act_dtype)
        if self._ffn_adds:
            return h, self.feed_forward.forward(n, ctx, residual=h)
        return h, self.feed_forward.forward(n, ctx)


BLOCKS.register("prenorm_residual", PreNormResidual)
