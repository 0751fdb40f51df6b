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
        self.interleaved = False

    def weight_specs(self):
        p = self.prefix
        return [WeightSpec(p + "gate_proj.weight", (self.inter, self.hidden)),
                WeightSpec(p + "up_proj.weight", (self.inter, self.hidden)),
                WeightSpec(p + "down_proj.weight", (self.hidden, self.inter))]

    takes_normed_rows = True      # its first step is a matrix product: the norm may fold in
    chain_safe = True             # touches device data through kernels/ops.py only

    def bind(self, weights):
        p = self.prefix
        gate, up = weights.pop(p + "gate_proj.weight"), weights.pop(p + "up_proj.weight")
        f, d = self.inter, self.hidden
        # eight gate rows, then the eight matching up rows, and so on: one 16-row tile of the
        # weight-streaming product then holds a gate column and its up column together
        self.interleaved = f % 8 == 0
        if self.interleaved:
            self.w_gate_up = torch.stack([gate.view(f // 8, 8, d), up.view(f // 8, 8, d)],
                                         dim=1).reshape(2 * f, d).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights.pop(p + "down_proj.weight").contiguous()

    def forward(self, x: torch.Tensor, ctx, residual=None):
        """With `residual` (the float32 stream) the result may be added to it, and None is
        then returned; otherwise the result is returned for the caller to add."""
        act = ops.gated_linear(x, self.w_gate_up, self.interleaved)
        return ops.linear(act, self.w_down, residual=residual)


FEED_FORWARDS.register("swiglu", SwiGLU)
