"""What every part of a layer has in common, and what a step hands to it.

A part is built from its spec record and the sizes around it, says which tensors
it needs (`weight_specs`), takes them (`bind`) and then computes (`forward`).
No part knows which model it is in: it sees its own spec, the hidden width, the
tensor-name prefix it was given, and a StepContext.

Interfaces (duck-typed; `Part` only supplies the defaults):

  norm            forward(h, delta, out_dtype, rows=None) -> normed rows
                  h is the float32 residual stream [T, d]; delta, if given, is added
                  to it first (and stays added); rows selects rows instead of all.
                  A forward that also takes `lazy=False` may, when asked, hand on rows it
                  has not computed (`ops.NormedRows`: the stream, the gain and eps) for the
                  consumer's first product to make while it reads them.
  position        `apply(q, k, ctx, num_heads, num_kv_heads, head_dim)` in place; and, if the
                  class sets `fusable = True`, `rotary(ctx)` -> (table [T, rotary_dim] of
                  cosines then sines, or None; rotary_dim), which lets the mixer do a
                  half-split rotation inside its own kernel instead of calling `apply`.
  mixer           cache_need() -> CacheNeed or None; state_need() -> StateNeed or None;
                  forward(x, ctx, cache) -> [T, d] in the activation dtype. A forward that
                  also takes `residual=None` may add its result into that float32 tensor
                  itself and return None (or return the result as usual).
  feed-forward    forward(x, ctx) -> [T, d]; `residual` as for the mixer.
                  A mixer or feed-forward whose class sets `lazy_rows = True` accepts x as
                  `ops.NormedRows` (it passes x to `ops.linear` / `ops.gated_linear`, or asks
                  `ops.rows_of(x)` for the tensor); without it a part always gets a tensor.
  block           forward(h, pending, ctx, cache) -> (h, pending): `pending` is a delta
                  not yet added to h, so the add can be fused into the next norm.

A part's constructor gets (its spec, the hidden width, the layer's tensor-name prefix, the
device); the checkpoint names of its weights are in its spec's `tensors` table, which the
architecture's config reader writes: no part carries a checkpoint's names in its code.

What a part may also offer, each with a default in `Part` (a part from outside the package
that offers none of them still runs):

  libraries(dtype, page_size) -> names of the kernel libraries (kernels/build.py) it will
                  call, so that an engine compiles them side by side before its first step;
  prepare_capture(ctx, cache) -> make, outside a CUDA-graph capture, whatever its forward
                  would otherwise make on the host during the step (lists derived from the
                  step's shape), leaving it in ctx.aux under a key that starts with "tiles";
  flops(extents, first_positions, writes_cache) -> floating-point operations of one forward
                  over requests bringing `extents` tokens from `first_positions` on;
  cache_bytes_read(context_len, width) -> bytes of cache one decoded token at that context
                  length reads (mixers that own a cache).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..weights.binder import WeightSpec


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per token in the paged cache: `planes` tensors (keys and values
    are two) of one row of `row_shape` each, for every token or for a window of them. The
    books only see kind and window; the storage gives every call of the group
    [planes, pages, page layout], where a row of two or more axes is laid out with its
    first axis outermost ([heads, page_size, head_dim]: one head's rows of a page lie
    together) and a row of one axis as [page_size, width]."""
    kind: str                     # "full" | "window"
    window: Optional[int]
    planes: int
    row_shape: Tuple[int, ...]

    @staticmethod
    def keys_and_values(window: Optional[int], num_kv_heads: int, head_dim: int) -> "CacheNeed":
        kind = "full" if window is None else "window"
        return CacheNeed(kind, None if window is None else int(window), 2,
                         (int(num_kv_heads), int(head_dim)))


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state a mixer keeps per request, float32, zero when a request starts."""
    shape: Tuple[int, ...]


@dataclass
class LayerCache:
    """What a layer call may touch of the cache during one step."""
    planes: Optional[torch.Tensor] = None       # [planes, pages, *page layout] of this call
    page_size: int = 0
    block_tables: Optional[torch.Tensor] = None  # int32 [B, max_blocks] of this layer's group
    slots: Optional[torch.Tensor] = None         # int32 [T], row of the storage per token
    writable: bool = True                        # False: the cache belongs to another call
    state: Optional[torch.Tensor] = None         # [num_slots, *StateNeed.shape] float32
    group: int = -1

    @property
    def k(self) -> Optional[torch.Tensor]:
        """Plane 0: for keys and values, the keys [pages, kv_heads, page_size, head_dim]."""
        return None if self.planes is None else self.planes[0]

    @property
    def v(self) -> Optional[torch.Tensor]:
        return None if self.planes is None else self.planes[1]


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

    def libraries(self, dtype: torch.dtype, page_size: int) -> List[str]:
        return []

    def prepare_capture(self, ctx: StepContext, cache: Optional[LayerCache]) -> None:
        pass

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        return 0.0

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        return 0.0


def offered(part, name: str):
    """A part's optional method, or Part's default when it has none (duck-typed parts from
    outside the package need not derive from Part)."""
    fn = getattr(part, name, None)
    if fn is not None:
        return fn
    return getattr(_DEFAULTS, name)


_DEFAULTS = Part()
