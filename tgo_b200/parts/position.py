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

    def rotary(self):
        """(inv_freq, rotary_dim): lets a mixer fuse the rotation into its own kernel."""
        return self.inv_freq, self.rotary_dim

    def apply(self, q, k, positions, num_heads, num_kv_heads, head_dim):
        """Rotate q [T, H*dh] and k [T, Hkv*dh] in place."""
        ops.qk_norm_rope_cache(q, k, None, num_heads, num_kv_heads, head_dim, None, None, 0.0,
                               positions, self.inv_freq, self.rotary_dim, None, None, None, 0)


class NoPosition(Part):
    """Positions do not enter the mixer."""
    fusable = True

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        pass

    def rotary(self):
        return None, 0

    def apply(self, q, k, positions, num_heads, num_kv_heads, head_dim):
        pass


POSITIONS.register("rope_half_split", RopeHalfSplit)
POSITIONS.register("none", NoPosition)
