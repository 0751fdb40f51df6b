"""Dense SiLU-gated feed-forward: (SiLU(x Wg^T) * (x Wu^T)) Wd^T, no bias
(nn/blocks.go:57-66). The gate and up matrices are joined at bind time so that one
matrix product makes both, and one kernel applies the gate. The checkpoint names of the
three matrices come from the spec's `tensors` table (roles gate, up or gate_up for a
matrix that is shipped joined, gate rows first; down)."""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import FeedForwardSpec, tensor_names
from ..kernels import ops
from ..registry import FEED_FORWARDS
from ..weights.binder import WeightSpec
from .base import Part


class SwiGLU(Part):
    def __init__(self, spec: FeedForwardSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.inter = spec.intermediate_size
        self.joined = "gate_up" in dict(spec.tensors)
        roles = (["gate_up"] if self.joined else ["gate", "up"]) + ["down"]
        self.names = tensor_names(spec.tensors, prefix, roles, "feed-forward")
        self.w_gate_up = None
        self.w_down = None
        self.interleaved = False

    def weight_specs(self):
        n = self.names
        if self.joined:
            first = [WeightSpec(n["gate_up"], (2 * self.inter, self.hidden))]
        else:
            first = [WeightSpec(n["gate"], (self.inter, self.hidden)),
                     WeightSpec(n["up"], (self.inter, self.hidden))]
        return first + [WeightSpec(n["down"], (self.hidden, self.inter))]

    def bind(self, weights):
        n = self.names
        f, d = self.inter, self.hidden
        if self.joined:
            both = weights.pop(n["gate_up"])
            gate, up = both[:f], both[f:]
        else:
            gate, up = weights.pop(n["gate"]), weights.pop(n["up"])
        # eight gate rows, then the eight matching up rows, and so on: one 16-row tile of the
        # weight-streaming product then holds a gate column and its up column together
        self.interleaved = f % 8 == 0
        if self.interleaved:
            self.w_gate_up = torch.stack([gate.reshape(f // 8, 8, d), up.reshape(f // 8, 8, d)],
                                         dim=1).reshape(2 * f, d).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = weights.pop(n["down"]).contiguous()

    def libraries(self, dtype, page_size) -> List[str]:
        return ["sgemm"] if dtype == torch.float32 else ["gemm_skinny"]

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        return 2.0 * sum(extents) * self.hidden * 3 * self.inter

    lazy_rows = True        # x may come as ops.NormedRows; the gate/up product folds the norm in

    def forward(self, x, ctx, residual=None):
        """With `residual` (the float32 stream) the result may be added to it, and None is
        then returned; otherwise the result is returned for the caller to add."""
        act = ops.gated_linear(x, self.w_gate_up, self.interleaved)
        return ops.linear(act, self.w_down, residual=residual)


FEED_FORWARDS.register("swiglu", SwiGLU)
