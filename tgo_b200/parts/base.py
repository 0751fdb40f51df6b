"""What every part of a layer has in common, and what a step hands to it.

A part is built from its spec record and the sizes around it, says which tensors
it needs (`weight_specs`), takes them (`bind`) and then computes (`forward`).
No part knows which model it is in: it sees its own spec, the hidden width, the
tensor-name prefix it was given, and a StepContext.

Interfaces (duck-typed; `Part` only supplies the defaults):

  norm            forward(h, delta, out_dtype, rows=None) -> normed rows
                  h is the float32 residual stream [T, d]; delta, if given, is added
                  to it first (and stays added); rows selects rows instead of all.
  position        `apply(q, k, ctx, num_heads, num_kv_heads, head_dim)` in place; and, if the
                  class sets `fusable = True`, `rotary(ctx)` -> (table [T, rotary_dim] of
                  cosines then sines, or None; rotary_dim), which lets the mixer do a
                  half-split rotation inside its own kernel instead of calling `apply`.
  mixer           cache_need() -> CacheNeed or None; state_need() -> StateNeed or None;
                  forward(x, ctx, cache) -> [T, d] in the activation dtype. A forward that
                  also takes `residual=None` may add its result into that float32 tensor
                  itself and return None (or return the result as usual).
  feed-forward    forward(x, ctx) -> [T, d]; `residual` as for the mixer.
  block           forward(h, pending, ctx, cache) -> (h, pending): `pending` is a delta
                  not yet added to h, so the add can be fused into the next norm.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..weights.binder import WeightSpec


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values a mixer keeps per token: every one of them, or a window."""
    kind: str                     # "full" | "window"
    window: Optional[int]
    num_kv_heads: int
    head_dim: int


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state a mixer keeps per request, float32, zero when a request starts."""
    shape: Tuple[int, ...]


@dataclass
class LayerCache:
    """What a layer call may touch of the cache during one step."""
    k: Optional[torch.Tensor] = None            # [pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    page_size: int = 0
    block_tables: Optional[torch.Tensor] = None  # int32 [B, max_blocks] of this layer's group
    slots: Optional[torch.Tensor] = None         # int32 [T], row of the storage per token
    writable: bool = True                        # False: the cache belongs to another call
    state: Optional[torch.Tensor] = None         # [num_slots, *StateNeed.shape] float32
    group: int = -1


@dataclass
class StepContext:
    """One step's batch as the parts see it. All tensors live on the device.

    Requests lie end to end in the token axis: request b owns tokens
    q_start[b] .. q_start[b+1]-1, at positions context_lens[b] - extent .. context_lens[b]-1.
    """
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor          # int32 [T]
    positions: torch.Tensor          # int32 [T]
    seq_ids: torch.Tensor            # int32 [T]  which request of the batch
    q_start: torch.Tensor            # int32 [B+1]
    context_lens: torch.Tensor       # int32 [B]  tokens in the cache after this step
    state_slots: torch.Tensor        # int32 [B]
    logit_rows: torch.Tensor         # int32 [n]  token rows whose logits are wanted
    act_dtype: torch.dtype
    # host-side copies, for kernel selection and tiling
    extents: List[int] = field(default_factory=list)
    first_positions: List[int] = field(default_factory=list)
    max_extent: int = 0
    max_context: int = 0
    decode_only: bool = False        # every request brings exactly one token
    aux: Dict[str, object] = field(default_factory=dict)   # per-step device tensors made once


class Part:
    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        pass
