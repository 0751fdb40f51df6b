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
from ..parts.base import LayerCache, StepContext, offered
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
            for part in (b.parts() if hasattr(b, "parts") else [b]):
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
                key = (need.kind, need.window, need.planes, tuple(need.row_shape))
                if key not in by_key:
                    by_key[key] = len(self.groups)
                    self.groups.append(GroupLayout(need.kind, need.window, need.planes,
                                                   need.row_shape, []))
                self.groups[by_key[key]].calls.append(ci)
                self.call_group[ci] = by_key[key]
            st = mixer.state_need() if hasattr(mixer, "state_need") else None
            if st is not None:
                self.state_shapes[ci] = tuple(st.shape)

    def cache_bytes_per_token(self) -> int:
        """Bytes one token adds to the cache over all groups."""
        width = 4 if self.dtype == torch.float32 else 2
        return sum(g.planes * len(g.calls) * g.row_elements * width for g in self.groups)

    # ------------------------------------------------------- what the parts report
    def libraries(self, page_size: int) -> List[str]:
        """Kernel libraries the model's parts say they will call, without repeats."""
        names = ["elementwise", "sgemm" if self.dtype == torch.float32 else "gemm_skinny"]
        for b in self.blocks:
            names += offered(b, "libraries")(self.dtype, page_size)
        names += offered(self.final_norm, "libraries")(self.dtype, page_size)
        return list(dict.fromkeys(names))

    def prepare_capture(self, ctx: StepContext, storage: CacheStorage, group_tables,
                        group_slots) -> None:
        """Before a CUDA-graph capture of this step: every part makes what its forward would
        otherwise make on the host."""
        for ci, call in enumerate(self.spec.run_order):
            cache = self.layer_cache(ci, ctx, storage, group_tables, group_slots)
            offered(self.blocks[call.layer], "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, n_logit_rows: int = 1) -> float:
        """Floating-point operations of one step, as the parts count their own, plus the
        head's product."""
        total = 0.0
        for call in self.spec.run_order:
            total += offered(self.blocks[call.layer], "flops")(extents, first_positions,
                                                               call.cache_from is None)
        return total + 2.0 * n_logit_rows * self.spec.hidden_size * self.spec.vocab_size

    def cache_bytes_read(self, context_len: float) -> float:
        """Bytes of cache one decoded token of a request at this context length reads."""
        width = 4 if self.dtype == torch.float32 else 2
        return sum(offered(self.blocks[call.layer], "cache_bytes_read")(context_len, width)
                   for call in self.spec.run_order)

    # ------------------------------------------------------------------- forward
    def layer_cache(self, ci: int, ctx: StepContext, storage: CacheStorage,
                    group_tables, group_slots) -> LayerCache:
        call = self.spec.run_order[ci]
        owner = ci if call.cache_from is None else call.cache_from
        lc = LayerCache(writable=call.cache_from is None, page_size=storage.page_size)
        if owner in storage.where:
            lc.planes, g = storage.layer(owner)
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
        for ci, call in enumerate(s.run_order):
            cache = self.layer_cache(ci, ctx, storage, group_tables, group_slots)
            h, pending = self.blocks[call.layer].forward(h, pending, ctx, cache)
        n_want = ctx.logit_rows.numel()
        if n_want == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=self.device)
        n = self.final_norm.forward(h, pending, ctx.act_dtype, rows=ctx.logit_rows)
        return ops.linear(n, self.head, out_dtype=torch.float32)
