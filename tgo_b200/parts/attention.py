"""Grouped-query causal attention over the paged cache.

q, k, v products (one joined matrix product) -> per-head RMSNorm of q and k over
head_dim, before the rotation -> rotation -> k and v stored in the cache -> softmax(q K^T
scale) V over the keys the query may see -> output product. No bias anywhere
(nn/attention.go:131-265; order of norm and rotation: specs/004-model-graph.md:149-160).
Query head h reads kv head floor(h / (H / Hkv)) (internal/oracle/attention.go:6-95).

Every size, the window, the scale and the position encoding are parameters. A call that
reads another call's cache computes q only. The checkpoint names of the weights come from
the spec's `tensors` table (roles q, k, v or qkv for a joined matrix, o, q_norm, k_norm).

Which attention kernel runs is this part's business too (`paged_attention` below): by storage
type, head size, group size, page size and what the step holds.
"""
from __future__ import annotations

import math
from typing import List

import torch

from ..config.spec import MixerSpec, tensor_names
from ..kernels import ops
from ..registry import MIXERS, POSITIONS
from ..weights.binder import WeightSpec
from .base import CacheNeed, LayerCache, Part

USE_TC_ATTENTION = True          # prompt portions with head size 128 on the tcgen05 kernel
SPLIT_MIXED_STEPS = True         # single tokens of a mixed step go through the decode kernel
TC_TILE_ROWS = 128               # query rows (token x head of the group) of a tcgen05 tile


# ---------------------------------------------------------------- per-step lists and plans


def step_tiles(ctx, tokens_per_tile: int):
    """Tile arrays of a step (first token and token count of each tile; a tile holds tokens
    of one request), made once per step and tile size and kept in ctx.aux."""
    key = ("tiles", tokens_per_tile)
    got = ctx.aux.get(key)
    if got is None:
        tok0, ntok, base = [], [], 0
        for n in ctx.extents:
            for o in range(0, n, tokens_per_tile):
                tok0.append(base + o)
                ntok.append(min(tokens_per_tile, n - o))
            base += n
        dev = torch.tensor([tok0, ntok], dtype=torch.int32).to(ctx.token_ids.device,
                                                               non_blocking=True)
        got = (dev[0], dev[1])
        ctx.aux[key] = got
    return got


def step_tiles_and_singles(ctx, tokens_per_tile: int):
    """For a step that holds prompt portions and single tokens: tile arrays of the entries
    with more than one token, and the list of the tokens that are alone in their entry."""
    key = ("tiles", tokens_per_tile, "split")
    got = ctx.aux.get(key)
    if got is None:
        tok0, ntok, singles, base = [], [], [], 0
        for n in ctx.extents:
            if n == 1:
                singles.append(base)
            else:
                for o in range(0, n, tokens_per_tile):
                    tok0.append(base + o)
                    ntok.append(min(tokens_per_tile, n - o))
            base += n
        dev = torch.tensor(tok0 + ntok + singles, dtype=torch.int32).to(ctx.token_ids.device,
                                                                         non_blocking=True)
        k = len(tok0)
        got = (dev[:k], dev[k:2 * k], dev[2 * k:], len(singles))
        ctx.aux[key] = got
    return got


def splits_for(pairs: int, reach: int, window: int, num_sms: int, ctas_per_sm: int = 3) -> int:
    """How many CTAs share one (request, kv head) pair's keys in a decode step: the count
    that is cheapest by a small model fitted on B200 (8 kv heads, contexts of 1024 and 4096,
    batches 8 to 128): the CTAs run in rounds of as many as the GPU holds, a CTA costs 1 unit
    per 64-key tile and 5 to start, joining the splits costs 10 once. So a few requests are
    cut until they fill the GPU once (batch 8: 7 ways), 32 or 64 requests of 1024 keys are
    not cut (the start is paid once), and 64 requests of 4096 keys are cut in 3 or 4, because
    the second, nearly empty round of whole requests would cost a whole request's time."""
    tiles = max(1, (reach + 63) // 64 + (1 if window > 0 else 0))
    pairs = max(1, pairs)
    wave = num_sms * ctas_per_sm
    best, best_cost = 1, None
    for s in range(1, max(1, min(tiles // 2, 64)) + 1):
        rounds = -(-pairs * s // wave)
        cost = rounds * (tiles / s * 1.0 + 5.0) + (10.0 if s > 1 else 0.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def decode_splits(ctx, num_kv_heads: int, window: int, device) -> int:
    reach = min(ctx.max_context, window) if window > 0 else ctx.max_context
    return splits_for(ctx.num_seqs * num_kv_heads, reach, window, ops.num_sms(device))


def tc_kernel_takes(q_dtype, head_dim: int, group: int, page_size: int) -> bool:
    return USE_TC_ATTENTION and q_dtype == torch.bfloat16 and head_dim == 128 and \
        ops.attention_tc_supports(head_dim, group, page_size)


def paged_attention(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, cache, ctx, scale: float, window: int) -> None:
    """Attention of every token of the step over its request's cached keys and values.

    float32, or a head size or group the tensor-core kernels have no instance for: the
    generic kernel (a warp per token and head, keys in a fixed order). bfloat16 decode
    steps: the split-key decode kernel (pages by TMA at head size 128). bfloat16 steps with
    prompt portions: the tcgen05 kernel at head size 128 (single tokens beside the portions
    go through the decode kernel), the mma.sync tile kernel at the other head sizes."""
    group = num_heads // num_kv_heads
    ps = cache.page_size
    args = (q, out, num_heads, num_kv_heads, head_dim, cache.k, cache.v, ps, cache.block_tables,
            ctx.positions, ctx.seq_ids)
    if q.dtype != torch.bfloat16 or not ops.flash_supports(head_dim, group):
        ops.attention_generic(q, out, num_heads, num_kv_heads, head_dim, cache.k, cache.v, ps,
                              cache.block_tables, ctx.seq_ids, ctx.positions, scale, window)
        return
    if ctx.decode_only:
        ops.attention_flash(*args, None, None, scale, window,
                            n_splits=decode_splits(ctx, num_kv_heads, window, q.device))
        return
    contiguous = cache.k.is_contiguous() and cache.v.is_contiguous()
    if contiguous and tc_kernel_takes(q.dtype, head_dim, group, ps):
        per_tile = TC_TILE_ROWS // group
        if SPLIT_MIXED_STEPS and 1 in ctx.extents and \
                ops.attention_decode_tma_supports(head_dim, group, ps):
            # prompt portions beside single tokens: the portions through the tile kernel, the
            # single tokens through the decode kernel (a tile of 128 rows for one token's few
            # heads would walk that request's whole context almost empty)
            tok0, ntok, singles, n_single = step_tiles_and_singles(ctx, per_tile)
            if tok0.numel():
                ops.attention_tc_prefill(*args, tok0, ntok, scale, window)
            reach = min(ctx.max_context, window) if window > 0 else ctx.max_context
            ops.attention_flash(*args, None, None, scale, window,
                                n_splits=splits_for(n_single * num_kv_heads, reach, window,
                                                    ops.num_sms(q.device)),
                                tok_list=singles)
            return
        tok0, ntok = step_tiles(ctx, per_tile)
        ops.attention_tc_prefill(*args, tok0, ntok, scale, window)
        return
    tok0, ntok = step_tiles(ctx, ops.flash_tile_rows() // group)
    ops.attention_flash(*args, tok0, ntok, scale, window)


# -------------------------------------------------------------------------------- the part


class GQAAttention(Part):
    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.H, self.Hkv, self.dh = spec.num_heads, spec.num_kv_heads, spec.head_dim
        if self.H <= 0 or self.Hkv <= 0 or self.H % self.Hkv:
            raise ValueError(f"attention: {self.H} query heads do not group over {self.Hkv}")
        self.qk_norm = spec.qk_norm
        self.eps = float(spec.norm_eps)
        self.window = spec.window
        # 1/sqrt(head_dim) in float64, rounded once to float32 by the kernel argument
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(self.dh)
        pos_spec = spec.position
        self.position = (POSITIONS.get(pos_spec.kind)(pos_spec, self.dh, device)
                         if pos_spec is not None else None)
        self.joined = "qkv" in dict(spec.tensors)        # the checkpoint ships one q/k/v matrix
        roles = (["qkv"] if self.joined else ["q", "k", "v"]) + ["o"] + \
            (["q_norm", "k_norm"] if self.qk_norm else [])
        self.names = tensor_names(spec.tensors, prefix, roles, "attention")
        self.w_qkv = self.w_q = self.w_o = None
        self.q_gain = self.k_gain = None

    # ---- declarations
    def weight_specs(self):
        n, d = self.names, self.hidden
        qw, kw = self.H * self.dh, self.Hkv * self.dh
        if self.joined:
            out = [WeightSpec(n["qkv"], (qw + 2 * kw, d))]
        else:
            out = [WeightSpec(n["q"], (qw, d)), WeightSpec(n["k"], (kw, d)),
                   WeightSpec(n["v"], (kw, d))]
        out.append(WeightSpec(n["o"], (d, qw)))
        if self.qk_norm:
            out += [WeightSpec(n["q_norm"], (self.dh,), "gain"),
                    WeightSpec(n["k_norm"], (self.dh,), "gain")]
        return out

    def cache_need(self):
        return CacheNeed.keys_and_values(self.window, self.Hkv, self.dh)

    def state_need(self):
        return None

    def bind(self, weights):
        n = self.names
        if self.joined:
            self.w_qkv = weights.pop(n["qkv"]).contiguous()
        else:
            self.w_qkv = torch.cat([weights.pop(n["q"]), weights.pop(n["k"]),
                                    weights.pop(n["v"])], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.H * self.dh]
        self.w_o = weights.pop(n["o"]).contiguous()
        if self.qk_norm:
            self.q_gain = weights.pop(n["q_norm"]).contiguous()
            self.k_gain = weights.pop(n["k_norm"]).contiguous()

    # ---- what the engine may ask
    def libraries(self, dtype, page_size) -> List[str]:
        if dtype == torch.float32:
            return ["sgemm", "attention_generic"]
        names = ["gemm_skinny", "attention_flash"]
        if self.dh == 128:
            names += ["attention_tc", "attention_decode_tma"]
        return names

    def prepare_capture(self, ctx, cache) -> None:
        """The tile lists of a step with prompt portions are made on the host: before a
        capture, make them for the tile size the step's kernel will ask for."""
        if ctx.decode_only or cache is None:
            return
        group = self.H // self.Hkv
        if ctx.act_dtype != torch.bfloat16 or not ops.flash_supports(self.dh, group):
            return
        if tc_kernel_takes(ctx.act_dtype, self.dh, group, cache.page_size):
            if SPLIT_MIXED_STEPS and 1 in ctx.extents and \
                    ops.attention_decode_tma_supports(self.dh, group, cache.page_size):
                step_tiles_and_singles(ctx, TC_TILE_ROWS // group)
            else:
                step_tiles(ctx, TC_TILE_ROWS // group)
        else:
            step_tiles(ctx, ops.flash_tile_rows() // group)

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        """2 per multiply-add: the q (k, v) and o products, and q.K and w.V over the keys
        each token may read."""
        n = sum(extents)
        qw = self.H * self.dh
        kv = 2 * self.Hkv * self.dh if writes_cache else 0
        total = 2.0 * n * self.hidden * (qw + kv) + 2.0 * n * qw * self.hidden
        keys = 0
        for first, extent in zip(first_positions, extents):
            if self.window:
                keys += sum(min(first + t + 1, self.window) for t in range(extent))
            else:
                keys += extent * first + extent * (extent + 1) // 2
        return total + 4.0 * qw * keys

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        reach = min(context_len, self.window) if self.window else context_len
        return 2.0 * self.Hkv * self.dh * width * reach

    # ---- compute
    lazy_rows = True        # x may come as ops.NormedRows; its first product folds the norm in

    def forward(self, x, ctx, cache: LayerCache, residual=None):
        """With `residual` (the float32 stream) the result may be added to it, and None is
        then returned; otherwise the result is returned for the caller to add."""
        H, Hkv, dh = self.H, self.Hkv, self.dh
        qw, kw = H * dh, Hkv * dh
        if cache.writable:
            qkv = ops.linear(x, self.w_qkv)           # x may be ops.NormedRows: folded in there
            q, k, v = qkv[:, :qw], qkv[:, qw:qw + kw], qkv[:, qw + kw:]
        else:
            q, k, v = ops.linear(x, self.w_q), None, None
        fused = self.position is None or getattr(self.position, "fusable", False)
        rope, rot = self.position.rotary(ctx) if (fused and self.position is not None) \
            else (None, 0)
        if fused and k is not None and ctx.decode_only and ops.decode_attention_fuses(
                q, dh, H // Hkv, cache.page_size, cache.k, cache.v, rot if rope is not None else 0):
            # a decode step at head size 128: the attention kernel norms, rotates and stores
            a = torch.empty((x.shape[0], qw), dtype=q.dtype, device=q.device)
            ops.attention_decode_fused(
                q, k, v, a, H, Hkv, dh, self.q_gain, self.k_gain, self.eps, rope, cache.slots,
                cache.k, cache.v, cache.page_size, cache.block_tables, ctx.positions, ctx.seq_ids,
                self.scale, self.window or 0,
                n_splits=decode_splits(ctx, Hkv, self.window or 0, q.device))
            return ops.linear(a, self.w_o, residual=residual)
        if fused:
            ops.qk_norm_rope_cache(q, k, v, H, Hkv, dh, self.q_gain, self.k_gain, self.eps,
                                   rope, rot, cache.slots if k is not None else None,
                                   cache.k if k is not None else None,
                                   cache.v if k is not None else None, cache.page_size)
        else:
            # a position encoding this kernel does not know: norm, then the encoding's own
            # code, then the store
            if self.qk_norm:
                ops.qk_norm_rope_cache(q, k, None, H, Hkv, dh, self.q_gain, self.k_gain,
                                       self.eps, None, 0, None, None, None, 0)
            self.position.apply(q, k, ctx, H, Hkv, dh)
            if k is not None:
                ops.qk_norm_rope_cache(q, k, v, H, Hkv, dh, None, None, 0.0, None, 0,
                                       cache.slots, cache.k, cache.v, cache.page_size)
        a = torch.empty((x.shape[0], qw), dtype=q.dtype, device=q.device)
        paged_attention(q, a, H, Hkv, dh, cache, ctx, self.scale, self.window or 0)
        return ops.linear(a, self.w_o, residual=residual)


MIXERS.register("gqa_attention", GQAAttention)
