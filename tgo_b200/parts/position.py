"""Rotary position encoding with half-split pairing: channel i of a head is paired with
channel i + rot/2 and the pair is rotated by position * theta^(-2i/rot)
(internal/oracle/rope.go:83-146; nn/attention.go:203-211). The reference reaches the same
pairing by permuting channels at load and running an interleaved kernel
(weights/convert.go:88-125); here the weights stay as the checkpoint has them and the
kernel pairs across the half."""
from __future__ import annotations

import torch

from ..config.spec import PositionSpec
from ..kernels import ops
from ..registry import POSITIONS
from .base import Part


class RopeHalfSplit(Part):
    fusable = True      # rotary() describes it fully; the mixer's kernel does the rotation

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        rot = spec.rotary_dim or head_dim
        if rot % 2 or rot <= 0 or rot > head_dim:
            raise ValueError(f"rotary_dim {rot} must be even and within head_dim {head_dim}")
        self.rotary_dim = rot
        self.theta = float(spec.theta)
        i = torch.arange(rot // 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-2.0 * i / rot)).to(device)

        self._key = ("rope_table", rot, self.theta)

    def table(self, ctx):
        """Cosines and sines of this step's positions, made once per step and shared by
        every layer with the same rotary_dim and theta."""
        got = ctx.aux.get(self._key)
        if got is None:
            got = ops.rope_table(ctx.positions, self.inv_freq)
            ctx.aux[self._key] = got
        return got

    def rotary(self, ctx):
        """(table, rotary_dim): lets a mixer do the rotation inside its own kernel."""
        return self.table(ctx), self.rotary_dim

    def apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim):
        """Rotate q [T, H*dh] and k [T, Hkv*dh] in place."""
        ops.qk_norm_rope_cache(q, k, None, num_heads, num_kv_heads, head_dim, None, None, 0.0,
                               self.table(ctx), self.rotary_dim, None, None, None, 0)


class NoPosition(Part):
    """Positions do not enter the mixer."""
    fusable = True

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        pass

    def rotary(self, ctx):
        return None, 0

    def apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim):
        pass


POSITIONS.register("rope_half_split", RopeHalfSplit)
POSITIONS.register("none", NoPosition)
