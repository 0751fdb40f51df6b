"""Stand-ins for the CUDA kernels, written with torch on the CPU, for tests only.

The engine has no CPU path. To check the host side of the engine on a machine without
a GPU (batch building, block tables, page reuse, the scheduler's loop), the `-m "not gpu"`
tests swap the functions of `tgo_b200.kernels.ops` for these through `install(monkeypatch)`.
They mirror the kernels' contracts (in-place writes, strided views, the cache layout
[page, kv_head, offset, head_dim]) and nothing of this file is importable from the
package itself.
"""
from __future__ import annotations

import math

import torch


def embed(table, ids, out):
    out.copy_(table[ids.long()].float())


def add_rmsnorm(h, delta, gain, eps, out, rows=None):
    if rows is None:
        if delta is not None:
            h += delta.float()
        x = h
    else:
        x = h[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    scale = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    out.copy_(((x * scale) * gain).to(out.dtype))


def residual_add(h, delta):
    h += delta.float()


def _gate(gate_up, f, interleaved):
    if interleaved:
        v = gate_up.reshape(gate_up.shape[0], f // 8, 2, 8)
        return v[:, :, 0].reshape(-1, f).float(), v[:, :, 1].reshape(-1, f).float()
    return gate_up[:, :f].float(), gate_up[:, f:].float()


def swiglu(gate_up, out, interleaved=False):
    g, u = _gate(gate_up, out.shape[1], interleaved)
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def rope_table(positions, inv_freq):
    ang = positions.double()[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=1).float()


def qk_norm_rope_cache(q, k, v, num_heads, num_kv_heads, head_dim, q_gain, k_gain, eps, rope,
                       rotary_dim, slots, k_cache, v_cache, page_size):
    T = q.shape[0]

    def treat(x, heads, gain):
        y = x.reshape(T, heads, head_dim).float()
        if gain is not None:
            y = (y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps)) * gain
        if rope is not None:
            half = rotary_dim // 2
            cos, sin = rope[:, None, :half], rope[:, None, half:]
            lo, hi = y[..., :half].clone(), y[..., half:rotary_dim].clone()
            y[..., :half] = lo * cos - hi * sin
            y[..., half:rotary_dim] = lo * sin + hi * cos
        return y

    q.copy_(treat(q, num_heads, q_gain).reshape(T, -1).to(q.dtype))
    if k is not None:
        kk = treat(k, num_kv_heads, k_gain)
        if k_cache is None:
            k.copy_(kk.reshape(T, -1).to(k.dtype))
    if k_cache is not None:
        vv = v.reshape(T, num_kv_heads, head_dim)
        for t in range(T):
            s = int(slots[t])
            if s < 0:
                continue
            page, off = s // page_size, s % page_size
            k_cache[page, :, off, :] = kk[t].to(k_cache.dtype)
            v_cache[page, :, off, :] = vv[t]


def attention_generic(q, out, num_heads, num_kv_heads, head_dim, k_cache, v_cache, page_size,
                      block_tables, seq_ids, positions, scale, window):
    T = q.shape[0]
    group = num_heads // num_kv_heads
    scale = float(torch.tensor(scale, dtype=torch.float32))
    for t in range(T):
        p, b = int(positions[t]), int(seq_ids[t])
        lo = max(0, p - window + 1) if window > 0 else 0
        idx = torch.arange(lo, p + 1)
        pages = block_tables[b].long()[idx // page_size]
        offs = idx % page_size
        for h in range(num_heads):
            g = h // group
            K = k_cache[pages, g, offs, :].float()
            V = v_cache[pages, g, offs, :].float()
            qv = q[t, h * head_dim:(h + 1) * head_dim].float()
            s = (K @ qv) * scale
            w = torch.softmax(s, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (w @ V).to(out.dtype)


def paged_attention(q, out, num_heads, num_kv_heads, head_dim, cache, ctx, scale, window):
    attention_generic(q, out, num_heads, num_kv_heads, head_dim, cache.k, cache.v,
                      cache.page_size, cache.block_tables, ctx.seq_ids, ctx.positions, scale,
                      window)


def linear(x, w, out_dtype=None, residual=None):
    y = x.float() @ w.float().t()
    if residual is not None:
        residual += y
        return None
    return y.to(out_dtype or x.dtype)


def gated_linear(x, w_gate_up, interleaved):
    gu = (x.float() @ w_gate_up.float().t()).to(x.dtype)
    out = torch.empty((x.shape[0], w_gate_up.shape[0] // 2), dtype=x.dtype)
    swiglu(gu, out, interleaved)
    return out


def sgemm_tn(x, w, out):
    out.copy_(x @ w.t())


def argmax(logits, out):
    import plain_qwen3 as plain
    for r in range(logits.shape[0]):
        out[r] = plain.argmax_lowest(logits[r].numpy())


def sample(logits, temperature, top_k, top_p, draws, out, report=None, logprob=None,
           top_ids=None, top_logprobs=None):
    import plain_qwen3 as plain
    for r in range(logits.shape[0]):
        ids, w, total = plain.policy_distribution(
            logits[r].numpy(), temperature=float(temperature[r]), top_k=int(top_k[r]),
            top_p=float(top_p[r]))
        out[r] = plain.walk(ids, w, total, float(draws[r]))
        if report is not None and int(report[r]) >= 0:
            lp, top = plain.token_logprobs(ids, w, total, int(out[r]), int(report[r]),
                                           logits.shape[1])
            logprob[r] = lp
            for j, (i, v) in enumerate(top):
                top_ids[r, j] = i
                top_logprobs[r, j] = v


def logits_adjust(row, bias_ids, bias, ids, counts, repetition, presence, frequency):
    if bias_ids is not None:
        for i, b in zip(bias_ids.tolist(), bias.tolist()):
            row[i] += b
    if ids is not None:
        for i, c in zip(ids.tolist(), counts.tolist()):
            x = float(row[i])
            if repetition not in (0.0, 1.0):
                x = x / repetition if x > 0 else x * repetition
            x -= presence + frequency * c
            row[i] = x


NAMES = ["rope_table", "argmax", "sample", "logits_adjust", "embed", "add_rmsnorm", "residual_add", "swiglu", "qk_norm_rope_cache",
         "attention_generic", "linear", "gated_linear", "sgemm_tn"]


def install(monkeypatch):
    from tgo_b200.kernels import ops
    from tgo_b200.parts import attention
    here = globals()
    for name in NAMES:
        monkeypatch.setattr(ops, name, here[name])
    monkeypatch.setattr(attention, "paged_attention", paged_attention)
