"""Plain, slow Qwen3-dense forward pass in float64 NumPy: the yardstick of the tests.

It rests on the formulas of latere-ai/tgo (the reference cannot be compiled on a
machine without a Go toolchain and without its external `accel` module, so no
output of the reference's own code is committed beside this file). Every function
cites the reference file and lines whose formula it restates.

Whole sequences only, no cache, no batching, one function per part. It shares no
code with `tgo_b200/`: it has its own safetensors reader, its own config reading
and its own sampler.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

# --------------------------------------------------------------------------- io


_ST_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64,
              "I32": np.int32, "BF16": None}


def read_safetensors(path):
    """name -> float64/int array. Layout: 8-byte little-endian header length, JSON
    header {name: {dtype, shape, data_offsets}}, then the planes.
    (safetensors/safetensors.go:114-193 describes the same container.)"""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        lo, hi = ent["data_offsets"]
        plane = raw[base + lo:base + hi]
        if ent["dtype"] == "BF16":
            u16 = np.frombuffer(plane, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(plane, dtype=_ST_DTYPES[ent["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(ent["shape"])
    return out


def write_safetensors(path, arrays, bfloat16=True):
    """Write {name: float array} in the layout `read_safetensors` describes, as BF16 (values
    rounded to the nearest, ties to even) or F32. Written here from the format's description,
    sharing nothing with the product's writer."""
    header, planes, at = {}, [], 0
    for name in sorted(arrays):
        a = np.ascontiguousarray(arrays[name], dtype=np.float32)
        if bfloat16:
            bits = a.view(np.uint32).astype(np.uint64)
            plane = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype("<u2").tobytes()
        else:
            plane = a.astype("<f4").tobytes()
        header[name] = {"dtype": "BF16" if bfloat16 else "F32", "shape": list(a.shape),
                        "data_offsets": [at, at + len(plane)]}
        planes.append(plane)
        at += len(plane)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)) + blob + b"".join(planes))


def load_model_dir(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, weights


# ------------------------------------------------------------------------ parts


def embedding(table, ids):
    """h[t,:] = E[ids[t],:] (model/qwen3_graph.go:48-61; internal/oracle/oracle.go:168-183)."""
    ids = np.asarray(ids)
    assert ids.min() >= 0 and ids.max() < table.shape[0]
    return table[ids].astype(np.float64)


def rmsnorm(x, gain, eps):
    """y_i = x_i * rsqrt(mean_j x_j^2 + eps) * g_i, eps inside the root, over the
    last axis (nn/blocks.go:53-55; internal/oracle/oracle.go:31-67)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return (x / np.sqrt(ms + eps)) * gain


def linear(x, w):
    """y = x . W^T with W stored [out, in], no bias (nn/blocks.go:22-46;
    internal/oracle/oracle.go:78)."""
    return x @ w.T


def rope_half_split(x, positions, theta, rotary_dim=None):
    """Rotate channel pairs (i, i + rot/2) of each head by pos * theta^(-2i/rot).
    x is [T, heads, dh]. Channels past rotary_dim are left alone.
    (internal/oracle/rope.go:83-146; nn/attention.go:203-211; the half-split
    pairing is the model's own, which the reference reaches by permuting
    channels at load: weights/convert.go:88-125.)"""
    T, _, dh = x.shape
    rot = dh if rotary_dim is None else rotary_dim
    half = rot // 2
    i = np.arange(half, dtype=np.float64)
    inv = theta ** (-2.0 * i / rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]      # [T, half]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    lo, hi = x[..., :half], x[..., half:rot]
    out = x.copy()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:rot] = lo * sin + hi * cos
    return out


def causal_gqa_attention(q, k, v, scale, window=None, round_weights=None):
    """q [T,H,dh], k/v [T,Hkv,dh] of one whole sequence. Query row t of head h
    reads kv head floor(h / (H/Hkv)) over keys 0..t (those with t - j < window if
    a window is given); softmax with the maximum subtracted; masking is by
    shortening the key range (internal/oracle/attention.go:6-95;
    nn/attention.go:234-264). round_weights: see forward_rounded."""
    T, H, dh = q.shape
    hkv = k.shape[1]
    group = H // hkv
    out = np.zeros_like(q)
    for t in range(T):
        lo = 0 if window is None else max(0, t - window + 1)
        for h in range(H):
            g = h // group
            s = (k[lo:t + 1, g, :] @ q[t, h, :]) * scale
            w = np.exp(s - s.max())
            if round_weights is None:
                w = w / w.sum()
            else:           # the weights that multiply the values are rounded, their sum is not
                w = round_weights(w) / w.sum()
            out[t, h, :] = w @ v[lo:t + 1, g, :]
    return out


def silu(x):
    """x / (1 + exp(-x)) (internal/oracle/oracle.go:101-110)."""
    return x / (1.0 + np.exp(-x))


def swiglu_mlp(x, w_gate, w_up, w_down):
    """(SiLU(x Wg^T) * (x Wu^T)) Wd^T (nn/blocks.go:57-66; internal/oracle/oracle.go:120-129)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def attention_block(x, positions, w, prefix, cfg, window=None):
    """q/k/v projections, per-head RMSNorm of q and k over head_dim (before the
    rotation), rotation, attention, output projection (nn/attention.go:131-265;
    ordering: specs/004-model-graph.md:149-160)."""
    H = cfg["num_attention_heads"]
    hkv = cfg.get("num_key_value_heads", H)
    dh = cfg.get("head_dim", cfg["hidden_size"] // H)
    eps = cfg["rms_norm_eps"]
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"]).reshape(T, H, dh)
    k = linear(x, w[prefix + "k_proj.weight"]).reshape(T, hkv, dh)
    v = linear(x, w[prefix + "v_proj.weight"]).reshape(T, hkv, dh)
    q = rmsnorm(q, w[prefix + "q_norm.weight"], eps)
    k = rmsnorm(k, w[prefix + "k_norm.weight"], eps)
    q = rope_half_split(q, positions, cfg["rope_theta"])
    k = rope_half_split(k, positions, cfg["rope_theta"])
    a = causal_gqa_attention(q, k, v, 1.0 / math.sqrt(dh), window)
    return linear(a.reshape(T, H * dh), w[prefix + "o_proj.weight"])


def layer_windows(cfg):
    """Window of every layer (None = all keys), from `layer_types` and
    `sliding_window`. The reference refuses windows (model/config.go:258-271);
    the engine under test accepts the explicit per-layer list."""
    L = cfg["num_hidden_layers"]
    kinds = cfg.get("layer_types")
    if not kinds:
        return [None] * L
    return [cfg["sliding_window"] if kd == "sliding_attention" else None for kd in kinds]


def forward(cfg, w, token_ids):
    """Logits [T, V] of one whole sequence (model/qwen3_graph.go:32-128)."""
    eps = cfg["rms_norm_eps"]
    T = len(token_ids)
    positions = np.arange(T)
    h = embedding(w["model.embed_tokens.weight"], token_ids)
    windows = layer_windows(cfg)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        n = rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        h = h + attention_block(n, positions, w, p + "self_attn.", cfg, windows[l])
        n = rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
    n = rmsnorm(h, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(n, head)


# ------------------------------------------------- the same model with rounded activations


def round_bfloat16(x):
    """Every value rounded to the nearest bfloat16 (8 significant bits, ties to even), as
    float64."""
    bits = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64)


def forward_rounded(cfg, w, token_ids, rnd=round_bfloat16):
    """`forward`, with every activation that an engine computing in bfloat16 stores in
    bfloat16 rounded by `rnd`: the norms' outputs, q, k and v before and after the q/k norm
    and rotation, the softmax weights that multiply the values, the attention's output, each
    product's output before it joins the (unrounded) residual sum, gate, up and their gated
    product. Softmax sums, norms, angles and the residual sum stay exact. The difference from
    `forward` is what rounding alone does to this model's logits on this input: the tests
    hold a bfloat16 engine's error against it."""
    eps = cfg["rms_norm_eps"]
    H = cfg["num_attention_heads"]
    hkv = cfg.get("num_key_value_heads", H)
    dh = cfg.get("head_dim", cfg["hidden_size"] // H)
    T = len(token_ids)
    positions = np.arange(T)
    h = embedding(w["model.embed_tokens.weight"], token_ids)
    windows = layer_windows(cfg)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        a = p + "self_attn."
        n = rnd(rmsnorm(h, w[p + "input_layernorm.weight"], eps))
        q = rnd(linear(n, w[a + "q_proj.weight"])).reshape(T, H, dh)
        k = rnd(linear(n, w[a + "k_proj.weight"])).reshape(T, hkv, dh)
        v = rnd(linear(n, w[a + "v_proj.weight"])).reshape(T, hkv, dh)
        q = rnd(rope_half_split(rmsnorm(q, w[a + "q_norm.weight"], eps), positions, cfg["rope_theta"]))
        k = rnd(rope_half_split(rmsnorm(k, w[a + "k_norm.weight"], eps), positions, cfg["rope_theta"]))
        att = rnd(causal_gqa_attention(q, k, v, 1.0 / math.sqrt(dh), windows[l], round_weights=rnd))
        h = h + rnd(linear(att.reshape(T, H * dh), w[a + "o_proj.weight"]))
        n = rnd(rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps))
        gate = rnd(linear(n, w[p + "mlp.gate_proj.weight"]))
        up = rnd(linear(n, w[p + "mlp.up_proj.weight"]))
        h = h + rnd(linear(rnd(silu(gate) * up), w[p + "mlp.down_proj.weight"]))
    n = rnd(rmsnorm(h, w["model.norm.weight"], eps))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(n, head)


# --------------------------------------------------------------------- sampling


def argmax_lowest(logits):
    """Largest logit, ties to the lowest id (sample/stages.go:196-206)."""
    best, at = logits[0], 0
    for i in range(1, len(logits)):
        if logits[i] > best:
            best, at = logits[i], i
    return at


def penalize(logits, history, rep=1.0, presence=0.0, frequency=0.0, window=0):
    """Repetition (divide a positive logit, multiply a non-positive one, once per
    token that appears), presence (once) and frequency (per occurrence)
    penalties over the last `window` tokens of history, 0 = all
    (sample/stages.go:152-190)."""
    logits = np.array(logits, dtype=np.float32)
    use_rep = rep not in (0.0, 1.0)
    use_add = presence != 0 or frequency != 0
    if not (use_rep or use_add):
        return logits
    hist = list(history)
    if window > 0 and len(hist) > window:
        hist = hist[-window:]
    counts = {}
    for t in hist:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        if use_rep:
            logits[t] = logits[t] / np.float32(rep) if logits[t] > 0 else logits[t] * np.float32(rep)
        if use_add:
            logits[t] = logits[t] - (np.float32(presence) + np.float32(frequency) * np.float32(c))
    return logits


def policy_distribution(logits, history=(), temperature=0.0, top_k=0, top_p=0.0,
                        rep=1.0, presence=0.0, frequency=0.0, window=0, bias=None,
                        exact_totals=False):
    """(ids ascending, float32 weights, float32 total) the draw is taken against:
    bias -> penalties -> (T == 0: argmax) -> /T -> top-k on the weights by
    (value, lower id) -> top-p prefix that reaches p of the total -> ascending ids
    (sample/stages.go:74-146, 216-241, 251-324). The totals are single ascending float32
    sums as there; with exact_totals they are float64 sums rounded once, for comparing an
    implementation that sums in another order (over 150k terms the single float32 sum is
    itself 1e-4 off, enough to move the nucleus's edge by a token)."""
    logits = np.array(logits, dtype=np.float32)
    for i, b in (bias or {}).items():
        logits[i] += np.float32(b)
    logits = penalize(logits, history, rep, presence, frequency, window)
    if temperature == 0:
        return [argmax_lowest(logits)], np.ones(1, np.float32), np.float32(1)
    logits = logits / np.float32(temperature)
    m = logits[argmax_lowest(logits)]
    allw = np.exp((logits - m).astype(np.float64)).astype(np.float32)
    def sum32(xs):
        if exact_totals:
            return np.float32(np.sum(np.asarray(xs, np.float64)))
        total = np.float32(0)
        for x in xs:
            total = np.float32(total + x)
        return total
    if top_k <= 0 and top_p <= 0:
        return list(range(len(allw))), allw, sum32(allw)
    n = min(top_k if top_k > 0 else 128, len(allw))
    order = sorted(range(len(allw)), key=lambda i: (-allw[i], i))[:n]
    wts = [allw[i] for i in order]
    total = sum32(wts) if top_k > 0 else sum32(allw)
    if top_p > 0:
        target = np.float32(total * np.float32(top_p))
        acc, cnt = np.float32(0), 0
        while cnt < len(order) and acc < target:
            acc = np.float32(acc + wts[cnt])
            cnt += 1
        order, wts, total = order[:cnt], wts[:cnt], acc
    pairs = sorted(zip(order, wts))
    return [p[0] for p in pairs], np.array([p[1] for p in pairs], np.float32), total


def walk(ids, weights, total, u):
    """First id, in ascending order, whose cumulative weight exceeds u * total;
    the last kept id if rounding never gets there (sample/stages.go:27-55)."""
    target = np.float32(np.float32(u) * total)
    acc = np.float32(0)
    last = ids[0]
    for i, x in zip(ids, weights):
        acc = np.float32(acc + x)
        if acc > target:
            return i
        last = i
    return last


def token_logprobs(ids, weights, total, token, n_top, vocab):
    """(ln p(token), [(id, ln p)] for the n_top most likely tokens) of the distribution
    policy_distribution returned: a kept token's share is its float32 weight over the
    float32 total, every other token has probability zero and so -inf; the alternatives
    descend by (probability, lower id), so once the kept tokens are used up the lowest
    unkept ids follow (decode.go:263-318, sample/sample.go:155-176)."""
    share = {i: np.float32(np.float32(x) / np.float32(total)) for i, x in zip(ids, weights)}

    def ln(i):
        q = float(share.get(i, 0.0))
        return float(np.log(q)) if q > 0 else -np.inf
    n = min(n_top, vocab)
    order = sorted(share, key=lambda i: (-share[i], i))[:n]
    i = 0
    while len(order) < n:
        if i not in share:
            order.append(i)
        i += 1
    return ln(token), [(i, ln(i)) for i in order]


def greedy_generate(cfg, w, prompt, n_new):
    """Whole-sequence recomputation for every new token; argmax with the lowest-id
    tie rule on the last row."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, seq)[-1]
        tok = argmax_lowest(logits.astype(np.float32))
        out.append(tok)
        seq.append(tok)
    return out
