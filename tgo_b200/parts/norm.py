"""RMSNorm over the last axis, with the residual add (and the row selection before the
head) fused into the same kernel, or, for the few rows of a decode step, left to the product
that consumes them: y = (x * rsqrt(mean x^2 + eps)) * gain, eps inside
the root, sums in float32 (nn/blocks.go:53-55; internal/oracle/oracle.go:31-67)."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import NormSpec
from ..kernels import ops
from ..registry import NORMS
from ..weights.binder import WeightSpec
from .base import Part


class RMSNorm(Part):
    def __init__(self, spec: NormSpec, width: int, name: str):
        self.eps = float(spec.eps)
        self.width = width
        self.name = name
        self.gain: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.name, (self.width,), "gain")]

    def bind(self, weights):
        self.gain = weights[self.name].contiguous()

    def libraries(self, dtype, page_size):
        return ["elementwise"]

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None, lazy: bool = False):
        """With `lazy` (the consumer takes `ops.NormedRows`), a few bfloat16 rows with nothing
        to add are handed on uncomputed: the product that reads them norms them itself."""
        if lazy and delta is None and rows is None and out_dtype == torch.bfloat16 and \
                h.is_cuda and h.shape[0] <= ops.SKINNY_MAX_ROWS:
            return ops.NormedRows(h, self.gain, self.eps, out_dtype)
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.width), dtype=out_dtype, device=h.device)
        ops.add_rmsnorm(h, delta, self.gain, self.eps, out, rows)
        return out


NORMS.register("rmsnorm", RMSNorm)
