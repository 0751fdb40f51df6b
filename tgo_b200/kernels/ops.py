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


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[t, j] = silu(gate_j) * up_j; gate_up holds the gate columns then the up columns,
    or, `interleaved`, eight gate columns and the eight matching up columns in turn."""
    _need_cuda(gate_up, out)
    T, f = out.shape
    assert gate_up.shape == (T, 2 * f) and gate_up.is_contiguous() and out.is_contiguous()
    assert gate_up.dtype == out.dtype
    lib = load_library("elementwise")
    _check(lib.tgo_swiglu(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(T),
                          c_int(f), c_int(1 if interleaved else 0), _stream()), "swiglu",
           f"(T={T}, f={f})")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[T, 2 * half] float32: cos then sin of position * inv_freq, evaluated in float64."""
    _need_cuda(positions, inv_freq)
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float64
    T, half = positions.numel(), inv_freq.numel()
    table = torch.empty((T, 2 * half), dtype=torch.float32, device=positions.device)
    lib = load_library("elementwise")
    _check(lib.tgo_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(table), c_int(T),
                              c_int(half), _stream()), "rope_table")
    return table


def qk_norm_rope_cache(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                       num_heads: int, num_kv_heads: int, head_dim: int,
                       q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                       rope: Optional[torch.Tensor], rotary_dim: int,
                       slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], page_size: int) -> None:
    """Per-head RMSNorm of q and k (if gains are given), half-split rotation (if `rope`, a
    table from rope_table, is given), q written back in place, k and v stored at `slots` of
    the paged cache [page, kv_head, offset, head_dim]. q, k, v are 2-D views whose rows may
    be strided (columns of one joined projection output)."""
    _need_cuda(q, k, v, q_gain, k_gain, rope, slots, k_cache, v_cache)
    T = q.shape[0]
    for t in (q, k, v):
        if t is not None:
            assert t.stride(1) == 1 and t.dtype == q.dtype and t.shape[0] == T
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, rotary_dim)
        assert rope.is_contiguous()
    if k_cache is not None:
        assert k_cache.dtype == q.dtype and v_cache.dtype == q.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert slots.dtype == torch.int32 and slots.numel() == T
    lib = load_library("elementwise")
    _check(lib.tgo_qk_norm_rope_cache(
        _ptr(q), c_ll(q.stride(0)), _ptr(k), c_ll(k.stride(0) if k is not None else 0),
        _ptr(v), c_ll(v.stride(0) if v is not None else 0), c_int(dtype_code(q.dtype)), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(q_gain), _ptr(k_gain),
        c_float(eps), _ptr(rope), c_int(rotary_dim if rope is not None else 0),
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


SKINNY_MAX_ROWS = 8

def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
                gated: bool = False) -> None:
    """out = x . w^T for at most 64 rows, bfloat16 [M, K] by bfloat16 [N, K], the
    weight-streaming kernel. out: bfloat16 or float32 [M, N]; with `accumulate` (float32) the
    product is added to it; with `gated`, w is a gate/up matrix with rows interleaved in
    eights and out is silu(gate) * up, bfloat16 [M, N / 2]."""
    _need_cuda(x, w, out)
    M, N, K = x.shape[0], w.shape[0], w.shape[1]
    assert w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    assert x.shape[1] == K and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2) and N % 16 == 0
        omode = 3
    elif accumulate:
        assert out.dtype == torch.float32 and out.shape == (M, N)
        omode = 2
    else:
        assert out.dtype in (torch.bfloat16, torch.float32) and out.shape == (M, N)
        omode = 0 if out.dtype == torch.bfloat16 else 1
    lib = load_library("gemm_skinny")
    _check(lib.tgo_gemm_skinny(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                               c_int(omode), _stream()), "gemm_skinny", f"(M={M}, N={N}, K={K})")


class NormedRows:
    """RMSNorm(h) * gain for a few rows of the float32 stream, not computed yet: a
    weight-streaming product that takes it makes the rows while it stages them (one kernel
    fewer between two products of a decode step); anything else asks for `rows()`. Carries
    the shape, dtype and device of the rows it stands for."""

    def __init__(self, h: torch.Tensor, gain: torch.Tensor, eps: float, dtype: torch.dtype):
        self.h, self.gain, self.eps, self.dtype = h, gain, eps, dtype
        self.shape, self.device = h.shape, h.device
        self._rows: Optional[torch.Tensor] = None

    def rows(self) -> torch.Tensor:
        if self._rows is None:
            self._rows = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            add_rmsnorm(self.h, None, self.gain, self.eps, self._rows)
        return self._rows


def rows_of(x) -> torch.Tensor:
    """x itself, or the rows a NormedRows stands for."""
    return x.rows() if isinstance(x, NormedRows) else x


_folds = {}


def folds_norm(M: int, N: int, K: int) -> bool:
    """Whether the weight-streaming product of these sizes can take its rows as NormedRows."""
    key = (M, N, K)
    if key not in _folds:
        _folds[key] = bool(load_library("gemm_skinny").tgo_gemm_skinny_folds_norm(
            c_int(M), c_int(N), c_int(K)))
    return _folds[key]


def gemm_skinny_normed(x: NormedRows, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """gemm_skinny with RMSNorm(x.h) * x.gain as its rows (at most 8), the norm folded into
    the product: out bfloat16 or float32 [M, N], or, `gated`, silu(gate) * up [M, N / 2]."""
    _need_cuda(x.h, x.gain, w, out)
    M, N, K = x.shape[0], w.shape[0], w.shape[1]
    assert x.h.dtype == torch.float32 and x.h.is_contiguous() and x.h.shape[1] == K
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and out.is_contiguous()
    assert x.gain.dtype == torch.float32 and x.gain.numel() == K
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2) and N % 16 == 0
        omode = 3
    else:
        assert out.dtype in (torch.bfloat16, torch.float32) and out.shape == (M, N)
        omode = 0 if out.dtype == torch.bfloat16 else 1
    lib = load_library("gemm_skinny")
    _check(lib.tgo_gemm_skinny_normed(_ptr(x.h), _ptr(x.gain), c_float(x.eps), _ptr(w), _ptr(out),
                                      c_int(M), c_int(N), c_int(K), c_int(omode), _stream()),
           "gemm_skinny_normed", f"(M={M}, N={N}, K={K})")


def _skinny_ok(x, w) -> bool:
    dt = x.dtype
    return dt == torch.bfloat16 and w.dtype == torch.bfloat16 and \
        x.shape[0] <= SKINNY_MAX_ROWS and w.shape[1] % 8 == 0


# Which kernel multiplies, by the number of rows (measured on B200 with the 8B shapes,
# `python bench.py --only products`):
#   1..8      gemm_skinny (weight streaming, mma.sync)        8-16 % faster than the library
#   9..1024   the library product (cuBLASLt through torch.mm)  the tcgen05 kernel is behind it on
#             q/k/v, o and down here (at 1024 rows 43 / 32 / 101 us against 37 / 26 / 75: too few
#             tiles for 148 SMs)
#   1025..    gemm_tc (tcgen05 + TMEM + TMA)                   at 2048 rows q/k/v 81 us (library 71),
#             o 48 (49), down 145 (144), gate/up with the gate 286 (library and gate kernel 319)
TC_MIN_ROWS = 1025
TC_MIN_ROWS_GATED = 1024   # the gate/up product with the gate in its epilogue: from here on it beats
                           # the library product followed by the gate kernel (149.6 against 154.8 us
                           # at 1024 rows of the 8B shape, 286 against 319 at 2048)
USE_TC = True            # False: the library product for every size above 8 rows


def product_regime(rows: int) -> int:
    """Which of the three product kernels a bfloat16 product of this many rows takes
    (0 weight streaming, 1 the library, 2 tcgen05): an engine warms each one up once before
    it captures a graph that holds it."""
    return 0 if rows <= SKINNY_MAX_ROWS else 1 if rows < TC_MIN_ROWS else 2


def _tc_ok(x, w, min_rows: Optional[int] = None) -> bool:
    return USE_TC and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and \
        x.shape[0] >= (TC_MIN_ROWS if min_rows is None else min_rows) and w.shape[1] % 8 == 0 and \
        x.is_contiguous() and w.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def _dense(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    M, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
        sgemm_tn(x, w, y)
        return y
    if _tc_ok(x, w):
        y = torch.empty((M, N), dtype=out_dtype, device=x.device)
        gemm_tc(x, w, y)
        return y
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        return torch.mm(x, w.t()) if out_dtype == torch.bfloat16 else \
            torch.mm(x, w.t(), out_dtype=torch.float32)
    raise KernelError(f"linear: x is {x.dtype} and w is {w.dtype}")


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           residual: Optional[torch.Tensor] = None):
    """y = x . w^T with w stored [out, in]. residual: a float32 [M, N] tensor the product
    belongs to: either it is added there and None is returned, or the product is returned
    for the caller to add (the block hands it to the next norm).

    float32: this package's plain-FMA kernel. bfloat16 with few rows (a decode step): this
    package's weight-streaming kernel, which does the residual add in its epilogue.
    bfloat16 with many rows (TC_MIN_ROWS): this package's tcgen05 kernel (TMA-fed,
    accumulators in tensor memory); between them the library product. out_dtype float32
    keeps the accumulator's width (the logits).
    """
    out_dtype = out_dtype or x.dtype
    if isinstance(x, NormedRows):
        M, N = x.shape[0], w.shape[0]
        if residual is None and _skinny_ok(x, w) and folds_norm(M, N, w.shape[1]):
            out = torch.empty((M, N), dtype=out_dtype, device=x.device)
            gemm_skinny_normed(x, w, out)
            return out
        x = x.rows()
    if _skinny_ok(x, w):
        M, N = x.shape[0], w.shape[0]
        if residual is not None:
            gemm_skinny(x, w, residual, accumulate=True)
            return None
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        gemm_skinny(x, w, out)
        return out
    if residual is not None and x.dtype == torch.bfloat16:
        # more than a few rows: the library has no add into a float32 stream, and from the
        # tcgen05 product's epilogue a read-modify-write of the stream is slow (each thread
        # owns a row); hand the product back and let the next norm, which reads the stream
        # anyway, add it
        return _dense(x, w, out_dtype)
    y = _dense(x, w, out_dtype)
    if residual is not None:
        residual_add(residual, y)
        return None
    return y


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) as [M, f] in x's dtype. w_gate_up is [2f, K]: the gate
    rows then the up rows, or (`interleaved`) eight gate rows and the eight matching up rows
    in turn, which lets the bfloat16 kernels apply the gate in their epilogue."""
    M, f = x.shape[0], w_gate_up.shape[0] // 2
    if isinstance(x, NormedRows):
        if interleaved and _skinny_ok(x, w_gate_up) and folds_norm(M, 2 * f, w_gate_up.shape[1]):
            out = torch.empty((M, f), dtype=torch.bfloat16, device=x.device)
            gemm_skinny_normed(x, w_gate_up, out, gated=True)
            return out
        x = x.rows()
    if interleaved and _skinny_ok(x, w_gate_up):
        out = torch.empty((M, f), dtype=torch.bfloat16, device=x.device)
        gemm_skinny(x, w_gate_up, out, gated=True)
        return out
    if interleaved and _tc_ok(x, w_gate_up, min(TC_MIN_ROWS, TC_MIN_ROWS_GATED)) and f % 8 == 0:
        out = torch.empty((M, f), dtype=torch.bfloat16, device=x.device)
        gemm_tc(x, w_gate_up, out, gated=True)
        return out
    gu = _dense(x, w_gate_up, x.dtype)
    out = torch.empty((M, f), dtype=x.dtype, device=x.device)
    swiglu(gu, out, interleaved)
    return out


_num_sms = {}


def num_sms(device) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    key = torch.device(device).index or 0
    if key not in _num_sms:
        _num_sms[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return _num_sms[key]


def flash_supports(head_dim: int, group: int) -> bool:
    """Whether the tensor-core attention kernel has an instance for this head size and
    group (others go to the generic kernel)."""
    return bool(load_library("attention_flash").tgo_attention_flash_supports(
        c_int(head_dim), c_int(group)))


USE_TMA_DECODE = True       # decode attention with head size 128: cache pages by TMA


def attention_decode_tma_supports(head_dim: int, group: int, page_size: int) -> bool:
    if head_dim != 128:                  # do not build the library for models that cannot use it
        return False
    return bool(load_library("attention_decode_tma").tgo_attention_decode_tma_supports(
        c_int(head_dim), c_int(group), c_int(page_size)))


def attention_decode_tma_error() -> int:
    """1 if a wait of the TMA-fed decode attention kernel ever ran out, else 0. Synchronises."""
    value = ctypes.c_int(0)
    _check(load_library("attention_decode_tma").tgo_attention_decode_tma_error(ctypes.byref(value)),
           "attention_decode_tma_error")
    return int(value.value)


FUSE_DECODE_QK = True        # decode steps at head size 128: q/k-norm, rotation and cache write
                             # inside the attention kernel instead of in a kernel before it


def decode_attention_fuses(q: torch.Tensor, head_dim: int, group: int, page_size: int,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, rotary_dim: int) -> bool:
    """Whether attention_decode_fused takes this layer: bfloat16, the TMA decode kernel's
    shapes, and a rotation of the whole head or none."""
    return FUSE_DECODE_QK and USE_TMA_DECODE and q.dtype == torch.bfloat16 and \
        rotary_dim in (0, head_dim) and k_cache.dim() == 4 and k_cache.is_contiguous() and \
        v_cache.is_contiguous() and k_cache.dtype == torch.bfloat16 and \
        attention_decode_tma_supports(head_dim, group, page_size)


def attention_decode_fused(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                           num_heads: int, num_kv_heads: int, head_dim: int,
                           q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                           rope: Optional[torch.Tensor], slots: torch.Tensor, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, page_size: int, block_tables: torch.Tensor,
                           positions: torch.Tensor, seq_ids: torch.Tensor, scale: float, window: int,
                           n_splits: int = 1) -> None:
    """A decode step's qk_norm_rope_cache and attention_flash in one kernel (head size 128):
    q, k, v are the raw rows of the step's tokens, one a request; q and k are normed (gains, or
    None) and rotated (`rope` [T, 128] from rope_table, or None) as qk_norm_rope_cache does,
    bit for bit, k and v are stored at `slots` of the cache, and every token attends over its
    request's keys including its own. q is left as it came."""
    _need_cuda(q, k, v, out, q_gain, k_gain, rope, slots, k_cache, v_cache, block_tables, positions,
               seq_ids)
    T = q.shape[0]
    assert q.dtype == k.dtype == v.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and out.stride(1) == 1
    assert k.shape[0] == v.shape[0] == T and slots.dtype == torch.int32 and slots.numel() == T
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.shape == (T, head_dim) and rope.is_contiguous()
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((T, num_heads, n_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, num_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    _check(load_library("attention_decode_tma").tgo_attention_decode_tma_fused(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(k_cache.shape[0]), c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(positions), _ptr(seq_ids), c_int(T), c_int(num_heads), c_int(num_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(n_splits), _ptr(part_o), _ptr(part_ml),
        _ptr(k), c_ll(k.stride(0)), _ptr(v), c_ll(v.stride(0)), _ptr(q_gain), _ptr(k_gain),
        c_float(eps), _ptr(rope), _ptr(slots), _stream()),
        "attention_decode_tma_fused", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")
    if n_splits > 1:
        _check(load_library("attention_flash").tgo_attention_flash_combine(
            _ptr(part_o), _ptr(part_ml), _ptr(out), c_ll(out.stride(0)), c_int(T), c_int(num_heads),
            c_int(head_dim), c_int(n_splits), _stream()), "attention_flash_combine")


def attention_flash(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                    block_tables: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
                    tile_tok0: Optional[torch.Tensor], tile_ntok: Optional[torch.Tensor],
                    scale: float, window: int, n_splits: int = 1,
                    tok_list: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention on the tensor cores (bfloat16). With tile arrays (int32,
    first token and token count of each tile, tokens of one request, at most
    flash_tile_rows() // group of them) any step; without them every token is a tile of its
    own (decode), and n_splits > 1 cuts each request's keys over that many CTAs and joins
    them. tok_list (int32, decode with head size 128 only): the tokens of the step to take,
    instead of all."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, positions, seq_ids, tile_tok0, tile_ntok,
               tok_list)
    T = q.shape[0] if tok_list is None else tok_list.numel()
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert k_cache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    n_tiles = T if tile_tok0 is None else tile_tok0.numel()
    tma = tile_tok0 is None and USE_TMA_DECODE and k_cache.dim() == 4 and k_cache.is_contiguous() and \
        v_cache.is_contiguous() and attention_decode_tma_supports(
            head_dim, num_heads // num_kv_heads, page_size)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((T, num_heads, n_splits, head_dim), dtype=torch.float32,
                             device=q.device)
        part_ml = torch.empty((T, num_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    lib = load_library("attention_flash")
    if tma:
        # decode with the pages brought in by TMA
        _check(load_library("attention_decode_tma").tgo_attention_decode_tma(
            _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
            c_int(k_cache.shape[0]), c_int(page_size), _ptr(block_tables),
            c_int(block_tables.shape[1]), _ptr(positions), _ptr(seq_ids), c_int(T), c_int(num_heads),
            c_int(num_kv_heads), c_int(head_dim), c_float(scale), c_int(window), c_int(n_splits),
            _ptr(part_o), _ptr(part_ml), _ptr(tok_list), _stream()),
            "attention_decode_tma", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")
        if n_splits > 1:
            _check(lib.tgo_attention_flash_combine_listed(
                _ptr(part_o), _ptr(part_ml), _ptr(out), c_ll(out.stride(0)), c_int(T),
                c_int(num_heads), c_int(head_dim), c_int(n_splits), _ptr(tok_list), _stream()),
                "attention_flash_combine")
        return
    assert tok_list is None, "a token list is taken by the TMA decode kernel only"
    _check(lib.tgo_attention_flash(
        _ptr(q), c_ll(q.stride(0)), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]), _ptr(positions),
        _ptr(seq_ids), _ptr(tile_tok0), _ptr(tile_ntok), c_int(n_tiles), c_int(num_heads),
        c_int(num_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
        c_int(n_splits), _ptr(part_o), _ptr(part_ml), _stream()),
        "attention_flash", f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads})")
    if n_splits > 1:
        _check(lib.tgo_attention_flash_combine(
            _ptr(part_o), _ptr(part_ml), _ptr(out), c_ll(out.stride(0)), c_int(T),
            c_int(num_heads), c_int(head_dim), c_int(n_splits), _stream()),
            "attention_flash_combine")


def attention_tc_supports(head_dim: int, group: int, page_size: int) -> bool:
    return bool(load_library("attention_tc").tgo_attention_tc_supports(c_int(head_dim), c_int(group),
                                                                       c_int(page_size)))


def attention_tc_error() -> int:
    """The code a wait of the tcgen05 attention kernel left when it ran out (1 producer,
    2 issuer, 3 softmax), or 0. Synchronises with the device."""
    value = ctypes.c_int(0)
    _check(load_library("attention_tc").tgo_attention_tc_error(ctypes.byref(value)), "attention_tc_error")
    return int(value.value)


def attention_tc_prefill(q: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                         block_tables: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
                         tile_tok0: torch.Tensor, tile_ntok: torch.Tensor, scale: float,
                         window: int) -> None:
    """Paged causal attention of prompt portions on the tcgen05 tensor cores (bfloat16, head
    size 128): tiles of 128 // group consecutive tokens of one request (tile_tok0, tile_ntok,
    int32); K and V pages [n_pages, kv_heads, page_size, 128] come in by TMA."""
    _need_cuda(q, out, k_cache, v_cache, block_tables, positions, seq_ids, tile_tok0, tile_ntok)
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_cache.shape == v_cache.shape and k_cache.shape[1:] == (num_kv_heads, page_size, head_dim)
    assert block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    lib = load_library("attention_tc")
    _check(lib.tgo_attention_tc_prefill(
        _ptr(q), c_ll(q.stride(0)), c_int(q.shape[0]), _ptr(out), c_ll(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_int(k_cache.shape[0]), c_int(page_size), _ptr(block_tables), c_int(block_tables.shape[1]),
        _ptr(positions), _ptr(seq_ids), _ptr(tile_tok0), _ptr(tile_ntok), c_int(tile_tok0.numel()),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
        _stream()), "attention_tc_prefill",
        f"(head_dim={head_dim}, heads={num_heads}/{num_kv_heads}, page_size={page_size})")


def flash_tile_rows() -> int:
    """Query rows (token x head of the group) one prefill tile of the attention kernel holds."""
    return int(load_library("attention_flash").tgo_attention_flash_tile_rows())


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r, ties to the lowest id."""
    _need_cuda(logits, out)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert out.dtype == torch.int32 and out.numel() == n
    lib = load_library("sampling")
    part_v = torch.empty((n, 32), dtype=torch.float32, device=logits.device)
    part_i = torch.empty((n, 32), dtype=torch.int32, device=logits.device)
    _check(lib.tgo_argmax(_ptr(logits), c_ll(logits.stride(0)), c_int(n), c_int(V), _ptr(out),
                          _ptr(part_v), _ptr(part_i), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, draws: torch.Tensor, out: torch.Tensor,
           report: Optional[torch.Tensor] = None, logprob: Optional[torch.Tensor] = None,
           top_ids: Optional[torch.Tensor] = None, top_logprobs: Optional[torch.Tensor] = None
           ) -> None:
    """Per row: temperature 0 -> argmax; else the softmax of logits / temperature, cut to the
    top_k largest (0: no cut) and to the top_p nucleus (0: no cut), walked in ascending id
    order to draws[r] * total.

    With `report` (int32 per row; negative: nothing for this row), a row also writes ln of
    the drawn token's share of the distribution it was drawn from into logprob[r], and its
    report[r] most likely tokens, descending, into top_ids[r] and top_logprobs[r] (both
    [rows, at most 128]; a token the policy left no chance has -inf)."""
    _need_cuda(logits, temperature, top_k, top_p, draws, out, report, logprob, top_ids,
               top_logprobs)
    n, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert draws.dtype == torch.float32 and top_k.dtype == torch.int32 and out.dtype == torch.int32
    assert temperature.numel() == top_k.numel() == top_p.numel() == draws.numel() == n
    width = 0
    if report is not None:
        assert report.dtype == torch.int32 and report.numel() == n
        assert logprob is not None and logprob.dtype == torch.float32 and logprob.numel() == n
        if top_ids is not None:
            width = top_ids.shape[1]
            assert top_ids.dtype == torch.int32 and top_logprobs.dtype == torch.float32
            assert top_ids.shape == top_logprobs.shape == (n, width)
            assert top_ids.is_contiguous() and top_logprobs.is_contiguous()
    lib = load_library("sampling")
    _check(lib.tgo_sample(_ptr(logits), c_ll(logits.stride(0)), c_int(n), c_int(V),
                          _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(draws), _ptr(out),
                          _ptr(report), _ptr(logprob), _ptr(top_ids), _ptr(top_logprobs),
                          c_int(width), _stream()), "sample")


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


_tc_err = {}


def gemm_tc_error_flag(device) -> torch.Tensor:
    """The int32 flag a tensor-core product sets if one of its waits ran out (0: none;
    1 producer, 2 issuer, 3 epilogue). One per device, made at first use."""
    key = torch.device(device).index or 0
    if key not in _tc_err:
        _tc_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_err[key]


_tc_tail = {}


def _tc_tail_buffers(device):
    """Per device: the float32 workspace and the zeroed flags through which the CTAs of a
    product's last round hand each other their parts of a tile (made at first use, outside
    any stream capture: the engine's first steps run uncaptured). One product at a time
    per device may use them."""
    key = torch.device(device).index or 0
    if key not in _tc_tail:
        lib = load_library("gemm_tc")
        lib.tgo_gemm_tc_tail_floats.restype = ctypes.c_longlong
        with torch.cuda.device(device):
            n, f = int(lib.tgo_gemm_tc_tail_floats()), int(lib.tgo_gemm_tc_tail_flags())
        _tc_tail[key] = (torch.empty(n, dtype=torch.float32, device=device),
                         torch.zeros(f, dtype=torch.int32, device=device))
    return _tc_tail[key]


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
            gated: bool = False) -> None:
    """out[M, N] = x[M, K] . w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, float32
    accumulation in tensor memory, TMA-fed); for many rows. out: bfloat16 or float32, or
    float32 that the product is added to. gated: w is a gate/up matrix with rows interleaved
    in eights and out is silu(gate) * up, bfloat16 [M, N / 2]. One thread at a time launches
    these (the forced tile and the last plan below are process-wide, the workspace of the
    last round's cut is one per device)."""
    _need_cuda(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    assert out.shape == ((M, N // 2) if gated else (M, N))
    if gated:
        assert out.dtype == torch.bfloat16 and N % 16 == 0
        omode = 4
    elif accumulate:
        assert out.dtype == torch.float32
        omode = 2
    else:
        omode = 0 if out.dtype == torch.bfloat16 else 1
        assert out.dtype in (torch.bfloat16, torch.float32)
    lib = load_library("gemm_tc")
    tail_ws, tail_flags = _tc_tail_buffers(x.device)
    _check(lib.tgo_gemm_tc(_ptr(x), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int(omode),
                           _ptr(tail_ws), _ptr(tail_flags), _ptr(gemm_tc_error_flag(x.device)),
                           _stream()), "gemm_tc", f"(M={M}, N={N}, K={K})")


def gemm_tc_force_tile(rows: int = 0, width: int = 0, cut_last_round: bool = True) -> None:
    """For tests and tuning: `gemm_tc` runs tiles of rows x width (rows 128
    or 256; width a multiple of 16 up to 256) instead of choosing; 0 gives the choice back.
    cut_last_round False: the tiles of the last round are not cut along K."""
    lib = load_library("gemm_tc")
    _check(lib.tgo_gemm_tc_force_tile(c_int(rows), c_int(width), c_int(0 if cut_last_round else 1)),
           "gemm_tc_force_tile", f"(rows={rows}, width={width})")


def gemm_tc_last_plan() -> tuple:
    """(rows, width, parts) of the last `gemm_tc`: its tile and into how many
    parts along K the tiles of its last round were cut (1: not cut)."""
    lib = load_library("gemm_tc")
    r, w, c = c_int(0), c_int(0), c_int(0)
    lib.tgo_gemm_tc_last_plan(ctypes.byref(r), ctypes.byref(w), ctypes.byref(c))
    return r.value, w.value, c.value


def kernel_wait_errors() -> dict:
    """Which kernels of this package gave up a wait (on an mbarrier or a grid barrier) since
    the process began: {kernel: code}, empty when none did. Their results are then not to be
    trusted. Looks only at libraries that are loaded; synchronises with the device."""
    from .build import _loaded
    out = {}
    if "attention_tc" in _loaded:
        code = attention_tc_error()
        if code:
            out["attention_tc"] = code
    if "attention_decode_tma" in _loaded:
        code = attention_decode_tma_error()
        if code:
            out["attention_decode_tma"] = code
    for key, flag in _tc_err.items():
        code = int(flag.item())
        if code:
            out[f"gemm_tc (device {key})"] = code
    return out
