"""A model as the engine runs it: embedding, blocks in their run order, final norm, head.

Built from a ModelSpec alone. The run order is data: a list of calls, each naming a layer
(twice, if the spec says so) and either owning a cache or reading an earlier call's
(model/qwen3_graph.go:32-128 is the reference's fixed loop for the dense case).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..cache.pages import GroupLayout
from ..cache.storage import CacheStorage
from ..config.spec import ModelSpec
from ..kernels import ops
from ..parts.base import LayerCache, StepContext
from ..registry import BLOCKS, NORMS
from ..weights.binder import WeightSpec


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"model: compute dtype {dtype}; float32 or bfloat16")
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks = [BLOCKS.get(ls.block)(ls, spec.hidden_size, self.device)
                       for ls in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, spec.hidden_size,
                                                          spec.final_norm_name)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self._layout()

    # ------------------------------------------------------------------- weights
    def weight_specs(self) -> List[WeightSpec]:
        s = self.spec
        out = [WeightSpec(s.embedding_name, (s.vocab_size, s.hidden_size), "table")]
        for b in self.blocks:
            out += b.weight_specs()
        out.append(WeightSpec(s.final_norm_name, (s.hidden_size,), "gain"))
        if s.head_name is not None:
            out.append(WeightSpec(s.head_name, (s.vocab_size, s.hidden_size), "matrix"))
        return out

    def tied_alias(self):
        """(name a tied checkpoint may ship anyway, name it must equal)."""
        if self.spec.head_name is None and self.spec.tied_head_alias:
            return (self.spec.tied_head_alias, self.spec.embedding_name)
        return None

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = weights[s.embedding_name].contiguous()
        self.head = self.embedding if s.head_name is None else weights[s.head_name].contiguous()
        for b in self.blocks:
            b.bind(weights)
        self.final_norm.bind(weights)

    def weight_bytes(self) -> int:
        """Bytes of every matrix a decode step reads once (the embedding table is read by
        row and is not counted unless it is also the head)."""
        seen, total = set(), 0
        tensors = [self.head]
        for b in self.blocks:
            for part in b.parts():
                tensors += [v for v in vars(part).values() if isinstance(v, torch.Tensor)]
        for t in tensors:
            if t is None or t.dtype not in (torch.float32, torch.bfloat16):
                continue
            key = t.untyped_storage().data_ptr()
            if key in seen:
                continue
            seen.add(key)
            total += t.untyped_storage().nbytes()
        return total

    # --------------------------------------------------------------------- cache
    def _layout(self) -> None:
        """Group the cache-owning calls by what they need."""
        self.groups: List[GroupLayout] = []
        self.call_group: Dict[int, int] = {}
        self.state_shapes: Dict[int, tuple] = {}
        by_key = {}
        for ci, call in enumerate(self.spec.run_order):
            if call.cache_from is not None:
                continue
            mixer = self.blocks[call.layer].mixer
            need = mixer.cache_need() if hasattr(mixer, "cache_need") else None
            if need is not None:
                key = (need.kind, need.window, need.num_kv_heads, need.head_dim)
                if key not in by_key:
                    by_key[key] = len(self.groups)
                    self.groups.append(GroupLayout(need.kind, need.window, need.num_kv_heads,
                                                   need.head_dim, []))
                self.groups[by_key[key]].calls.append(ci)
                self.call_group[ci] = by_key[key]
            st = mixer.state_need() if hasattr(mixer, "state_need") else None
            if st is not None:
                self.state_shapes[ci] = tuple(st.shape)

    def cache_bytes_per_token(self) -> int:
        """Bytes of keys and values one token adds over all full groups."""
        width = 4 if self.dtype == torch.float32 else 2
        return sum(2 * len(g.calls) * g.num_kv_heads * g.head_dim * width for g in self.groups)

    # ------------------------------------------------------------------- forward
    def layer_cache(self, ci: int, ctx: StepContext, storage: CacheStorage,
                    group_tables, group_slots) -> LayerCache:
        call = self.spec.run_order[ci]
        owner = ci if call.cache_from is None else call.cache_from
        lc = LayerCache(writable=call.cache_from is None, page_size=storage.page_size)
        if owner in storage.where:
            lc.k, lc.v, g = storage.layer(owner)
            lc.group = g
            lc.block_tables = group_tables[g]
            lc.slots = group_slots[g]
        if owner in storage.state:
            lc.state = storage.state[owner]
        return lc

    def forward(self, ctx: StepContext, storage: CacheStorage, group_tables,
                group_slots) -> torch.Tensor:
        """Run the step's tokens through every call; logits (float32) at ctx.logit_rows."""
        s = self.spec
        h = torch.empty((ctx.num_tokens, s.hidden_size), dtype=torch.float32, device=self.device)
        ops.embed(self.embedding, ctx.token_ids, h)
        pending = None
        # a decode step of a few rows: the products of consecutive parts (and layers) are
        # collected and run as chains in one persistent kernel each, if every block keeps to
        # the kernels of this package
        chained = ctx.decode_only and self.dtype == torch.bfloat16 and \
            all(getattr(b, "chain_safe", False) for b in self.blocks) and \
            ops.begin_chain(ctx.num_tokens)
        try:
            for ci, call in enumerate(s.run_order):
                cache = self.layer_cache(ci, ctx, storage, group_tables, group_slots)
                h, pending = self.blocks[call.layer].forward(h, pending, ctx, cache)
        finally:
            if chained:
                ops.end_chain()
        n_want = ctx.logit_rows.numel()
        if n_want == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=self.device)
        n = self.final_norm.forward(h, pending, ctx.act_dtype, rows=ctx.logit_rows)
        return ops.linear(n, self.head, out_dtype=torch.float32)
