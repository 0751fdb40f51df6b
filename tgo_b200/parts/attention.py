"""Grouped-query causal attention over the paged cache.

q, k, v projections (one joined matrix product) -> per-head RMSNorm of q and k over
head_dim, before the rotation -> rotation -> k and v stored in the cache -> softmax(q K^T
scale) V over the keys the query may see -> output projection. No bias anywhere
(nn/attention.go:131-265; order of norm and rotation: specs/004-model-graph.md:149-160).
Query head h reads kv head floor(h / (H / Hkv)) (internal/oracle/attention.go:6-95).

Every size, the window, the scale and the position encoding are parameters. A call that
reads another call's cache computes q only.
"""
from __future__ import annotations

import math

import torch

from ..config.spec import MixerSpec
from ..kernels import ops
from ..registry import MIXERS, POSITIONS
from ..weights.binder import WeightSpec
from .base import CacheNeed, LayerCache, Part


class GQAAttention(Part):
    takes_normed_rows = True      # its first step is a matrix product: the norm may fold in
    chain_safe = True             # touches device data through kernels/ops.py only

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.prefix = prefix
        self.H, self.Hkv, self.dh = spec.num_heads, spec.num_kv_heads, spec.head_dim
        if self.H <= 0 or self.Hkv <= 0 or self.H % self.Hkv:
            raise ValueError(f"attention: {self.H} query heads do not group over {self.Hkv}")
        self.qk_norm = spec.qk_norm
        self.eps = float(spec.norm_eps)
        self.window = spec.window
        # 1/sqrt(head_dim) in float64, rounded once to float32 by the kernel argument
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(self.dh)
        pos_spec = spec.position
        self.position = (POSITIONS.get(pos_spec.kind)(pos_spec, self.dh, device)
                         if pos_spec is not None else None)
        self.w_qkv = self.w_q = self.w_o = None
        self.q_gain = self.k_gain = None

    # ---- declarations
    def weight_specs(self):
        p, d = self.prefix, self.hidden
        out = [WeightSpec(p + "q_proj.weight", (self.H * self.dh, d)),
               WeightSpec(p + "k_proj.weight", (self.Hkv * self.dh, d)),
               WeightSpec(p + "v_proj.weight", (self.Hkv * self.dh, d)),
               WeightSpec(p + "o_proj.weight", (d, self.H * self.dh))]
        if self.qk_norm:
            out += [WeightSpec(p + "q_norm.weight", (self.dh,), "gain"),
                    WeightSpec(p + "k_norm.weight", (self.dh,), "gain")]
        return out

    def cache_need(self):
        if self.window is None:
            return CacheNeed("full", None, self.Hkv, self.dh)
        return CacheNeed("window", int(self.window), self.Hkv, self.dh)

    def state_need(self):
        return None

    def bind(self, weights):
        p = self.prefix
        wq = weights.pop(p + "q_proj.weight")
        wk = weights.pop(p + "k_proj.weight")
        wv = weights.pop(p + "v_proj.weight")
        self.w_qkv = torch.cat([wq, wk, wv], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.H * self.dh]
        self.w_o = weights.pop(p + "o_proj.weight").contiguous()
        if self.qk_norm:
            self.q_gain = weights.pop(p + "q_norm.weight").contiguous()
            self.k_gain = weights.pop(p + "k_norm.weight").contiguous()

    # ---- compute
    def forward(self, x: torch.Tensor, ctx, cache: LayerCache, residual=None):
        """With `residual` (the float32 stream) the result may be added to it, and None is
        then returned; otherwise the result is returned for the caller to add."""
        H, Hkv, dh = self.H, self.Hkv, self.dh
        qw, kw = H * dh, Hkv * dh
        if cache.writable:
            qkv = ops.linear(x, self.w_qkv)
            q, k, v = qkv[:, :qw], qkv[:, qw:qw + kw], qkv[:, qw + kw:]
        else:
            q, k, v = ops.linear(x, self.w_q), None, None
        fused = self.position is None or getattr(self.position, "fusable", False)
        rope, rot = self.position.rotary(ctx) if (fused and self.position is not None) \
            else (None, 0)
        if fused:
            ops.qk_norm_rope_cache(q, k, v, H, Hkv, dh, self.q_gain, self.k_gain, self.eps,
                                   rope, rot, cache.slots if k is not None else None,
                                   cache.k if k is not None else None,
                                   cache.v if k is not None else None, cache.page_size)
        else:
            # a position encoding this kernel does not know: norm, then the encoding's own
            # code (which may use anything: products still pending must have run), then the store
            ops.flush_chain()
            if self.qk_norm:
                ops.qk_norm_rope_cache(q, k, None, H, Hkv, dh, self.q_gain, self.k_gain,
                                       self.eps, None, 0, None, None, None, 0)
            self.position.apply(q, k, ctx, H, Hkv, dh)
            if k is not None:
                ops.qk_norm_rope_cache(q, k, v, H, Hkv, dh, None, None, 0.0, None, 0,
                                       cache.slots, cache.k, cache.v, cache.page_size)
        a = torch.empty((x.shape[0], qw), dtype=q.dtype, device=q.device)
        ops.paged_attention(q, a, H, Hkv, dh, cache, ctx, self.scale, self.window or 0)
        return ops.linear(a, self.w_o, residual=residual)


MIXERS.register("gqa_attention", GQAAttention)
