"""Python face of the CUDA kernels: each function checks its tensors, then calls the
extern "C" entry point of the same name on the current CUDA stream.

Tensors are torch tensors on a CUDA device; nothing here computes with torch, and
nothing falls back to it. A refused size raises with the kernel's name in the message.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
E_BAD_ARG = 1000

c_int, c_ll, c_float, c_void = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 storage, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void(0) if t is None else c_void(t.data_ptr())


def _stream():
    return c_void(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on a CUDA device only; got a tensor on "
                              f"{t.device}. There is no CPU path.")


LAUNCHES = [0]        # kernels of this package launched so far (graph replays add theirs)


def _check(status: int, name: str, detail: str = "") -> None:
    if status == 0:
        LAUNCHES[0] += 1
        return
    if status == E_BAD_ARG:
        raise KernelError(f"{name}: refused these sizes or types {detail}")
    raise KernelError(f"{name}: CUDA error {status} at launch {detail}")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] widened to float32. ids int32 [T]; out float32 [T, d]."""
    _need_cuda(table, ids, out)
    T, d = out.shape
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous()
    lib = load_library("elementwise")
    _check(lib.tgo_embed(_ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out),
                         c_int(T), c_int(d), c_int(table.shape[0]), _stream()), "embed")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """h += delta (if given, and rows is None), out = rmsnorm(h) * gain.
    With `rows` (int32 [n]): out[i] = rmsnorm(h[rows[i]] + delta[rows[i]]) * gain, h untouched."""
    _need_cuda(h, delta, gain, out, rows)
    n, d = out.shape
    assert h.dtype == torch.float32 and gain.dtype == torch.float32 and h.is_contiguous()
    assert gain.numel() == d and out.is_contiguous() and h.shape[1] == d
    if delta is not None:
        assert delta.shape == h.shape and delta.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n
    else:
        assert h.shape[0] == n
    lib = load_library("elementwise")
    _check(lib.tgo_add_rmsnorm(_ptr(h), _ptr(delta),
                               c_int(dtype_code(delta.dtype) if delta is not None else 0),
                               _ptr(gain), c_float(eps), _ptr(out), c_int(dtype_code(out.dtype)),
                               _ptr(rows), c_int(n), c_int(d), _stream()), "add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    """h += delta, h float32."""
    _need_cuda(h, delta)
    assert h.dtype == torch.float32 and h.is_contiguous() and delta.is_contiguous()
    assert h.shape == delta.shape
    lib = load_library("elementwise")
    _check(lib.tgo_residual_add(_ptr(h), _ptr(delta), c_int(dtype_code(delta.dtype)),
                                c_ll(h.numel()), _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, f + j]."""
    _need_cuda(gate_up, out)
    T, f = out.shape
    assert gate_up.shape == (T, 2 * f) and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.dtype == out.dtype
    lib = load_library("elementwise")
    _check(lib.tgo_swiglu(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T),
                          c_int(f), _stream()), "swiglu", f"(T={T}, f={f})")


def qk_norm_rope_cache(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                       num_heads: int, num_kv_heads: int, head_dim: int,
                       q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                       positions: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                       rotary_dim: int, slots: Optional[torch.Tensor],
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       page_size: int) -> None:
    """Per-head RMSNorm of q and k (if gains are given), half-split rotation (if inv_freq
    is given), q written back in place, k and v stored at `slots` of the paged cache
    [page, kv_head, offset, head_dim]. q, k, v are 2-D views whose rows may be strided
    (columns of one fused projection output)."""
    _need_cuda(q, k, v, q_gain, k_gain, positions, inv_freq, slots, k_cache, v_cache)
    T = q.shape[0]
    for t in (q, k, v):
        if t is not None:
            assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary_dim // 2
        assert positions is not None and positions.dtype == torch.int32
    if k_cache is not None:
        assert k_cache.dtype == q.dtype and v_cache.dtype == q.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert slots.dtype == torch.int32 and slots.numel() == T
    lib = load_library("elementwise")
    _check(lib.tgo_qk_norm_rope_cache(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0) if k is not None else 0),
        _ptr(v), c_ll(v.stride(0) if v is not None else 0), c_int(dtype_code(q.dtype)), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(q_gain), _ptr(k_gain),
        c_float(eps), _ptr(positions), _ptr(inv_freq), c_int(rotary_dim if inv_freq is not None
                                                              else 0),
        _ptr(slots), _ptr(k_cache), _ptr(v_cache), c_int(page_size), _stream()),
        "qk_norm_rope_cache", f"(head_dim={head_dim}, rotary_dim={rotary_dim})")


def attention_generic(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                      block_tables: torch.Tensor, seq_ids: torch.Tensor, positions: torch.Tensor,
                      scale: float, window: int) -> None:
    """Paged causal attention, one warp per (token, head). q is a 2-D view [T, >= H*dh]
    with unit column stride; out likewise. window 0 = every earlier key."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, seq_ids, positions)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype
    assert block_tables.dtype == torch.int32 and block_tables.dim() == 2
    assert block_tables.is_contiguous() and seq_ids.dtype == torch.int32
    assert positions.dtype == torch.int32
    lib = load_library("attention_generic")
    _check(lib.tgo_attention_generic(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), c_int(dtype_code(q.dtype)),
        c_int(T), c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(k_cache),
        _ptr(v_cache), c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(seq_ids), _ptr(positions), c_float(scale), c_int(window), _stream()),
        "attention_generic", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")


def sgemm_tn(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = x[M,K] . w[N,K]^T, all float32, plain FMA."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert x.dtype == w.dtype == out.dtype == torch.float32
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    lib = load_library("sgemm")
    _check(lib.tgo_sgemm_tn(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), _stream()),
           "sgemm_tn", f"(M={M}, N={N}, K={K})")


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x . w^T with w stored [out, in].

    float32: this package's plain-FMA kernel. bfloat16: the library matrix product
    (cuBLASLt through torch.mm) with float32 accumulation; out_dtype float32 keeps the
    accumulator's width (used for the logits).
    """
    _need_cuda(x, w)
    M, N = x.shape[0], w.shape[0]
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        sgemm_tn(x, w, out)
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: x is {x.dtype} and w is {w.dtype}")
    if out_dtype == torch.bfloat16:
        if out is None:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out=out)
    if out is None:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t(), out_dtype=torch.float32, out=out)


def paged_attention(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, cache, ctx, scale: float, window: int) -> None:
    """Attention of every token of the step over its request's cached keys and values.
    Picks the kernel by storage type, head size and what the step holds."""
    attention_generic(q, out, num_heads, num_kv_heads, head_dim, cache.k, cache.v,
                      cache.page_size, cache.block_tables, ctx.seq_ids, ctx.positions, scale,
                      window)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r, ties to the lowest id."""
    _need_cuda(logits, out)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert out.dtype == torch.int32 and out.numel() == n
    lib = load_library("sampling")
    _check(lib.tgo_argmax(_ptr(logits), c_ll(logits.stride(0)), c_int(n), c_int(V), _ptr(out),
                          _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, draws: torch.Tensor, out: torch.Tensor) -> None:
    """Per row: temperature 0 -> argmax; else the softmax of logits / temperature, cut to the
    top_k largest (0: no cut) and to the top_p nucleus (0: no cut), walked in ascending id
    order to draws[r] * total."""
    _need_cuda(logits, temperature, top_k, top_p, draws, out)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert draws.dtype == torch.float32 and top_k.dtype == torch.int32 and out.dtype == torch.int32
    assert temperature.numel() == top_k.numel() == top_p.numel() == draws.numel() == n
    lib = load_library("sampling")
    _check(lib.tgo_sample(_ptr(logits), c_ll(logits.stride(0)), c_int(n), c_int(V),
                          _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(draws), _ptr(out),
                          _stream()), "sample")


def logits_adjust(row: torch.Tensor, bias_ids: Optional[torch.Tensor],
                  bias: Optional[torch.Tensor], ids: Optional[torch.Tensor],
                  counts: Optional[torch.Tensor], repetition: float, presence: float,
                  frequency: float) -> None:
    """Edit one row of logits in place: add the biases, then apply the penalties to the
    distinct history tokens `ids` with their `counts`."""
    _need_cuda(row, bias_ids, bias, ids, counts)
    assert row.dtype == torch.float32 and row.dim() == 1 and row.is_contiguous()
    nb = 0 if bias_ids is None else bias_ids.numel()
    ni = 0 if ids is None else ids.numel()
    lib = load_library("sampling")
    _check(lib.tgo_logits_adjust(_ptr(row), _ptr(bias_ids), _ptr(bias), c_int(nb), _ptr(ids),
                                 _ptr(counts), c_int(ni), c_float(repetition), c_float(presence),
                                 c_float(frequency), c_int(row.numel()), _stream()),
           "logits_adjust")
