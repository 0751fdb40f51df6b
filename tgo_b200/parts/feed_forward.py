"""Dense SiLU-gated feed-forward: (SiLU(x Wg^T) * (x Wu^T)) Wd^T, no bias
(nn/blocks.go:57-66). The gate and up matrices are joined at bind time so that one
matrix product makes both, and one kernel applies the gate."""
from __future__ import annotations

import torch

from ..config.spec import FeedForwardSpec
from ..kernels import ops
from ..registry import FEED_FORWARDS
from ..weights.binder import WeightSpec
from .base import Part


class SwiGLU(Part):
    def __init__(self, spec: FeedForwardSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.inter = spec.intermediate_size
        self.prefix = prefix
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self):
        p = self.prefix
        return [WeightSpec(p + "gate_proj.weight", (self.inter, self.hidden)),
                WeightSpec(p + "up_proj.weight", (self.inter, self.hidden)),
                WeightSpec(p + "down_proj.weight", (self.hidden, self.inter))]

    def bind(self, weights):
        p = self.prefix
        self.w_gate_up = torch.cat([weights.pop(p + "gate_proj.weight"),
                                    weights.pop(p + "up_proj.weight")], dim=0).contiguous()
        self.w_down = weights.pop(p + "down_proj.weight").contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        gu = ops.linear(x, self.w_gate_up)
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        ops.swiglu(gu, act)
        return ops.linear(act, self.w_down)


FEED_FORWARDS.register("swiglu", SwiGLU)
