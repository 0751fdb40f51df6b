"""Tiny configurations, random model folders and trace builders shared by the tests.

Two configurations of the one architecture that differ in every size and option:

            layers hidden heads kv  head_dim  q width  inter vocab  theta  eps    tied  window  page
  TINY_A      2     64     4    2    16        64      128   256   1e4    1e-6   yes   none     16
  TINY_B      3     96     6    2    32       192      224   384   1e6    1e-5   no    24 (layer 1)  8

In A the q width equals the hidden size and layers equal kv heads, so a confusion of
those two pairs passes there; B is the configuration that tells them apart.

A third, TINY_C, has the head size (128) that the tcgen05 attention kernel takes, a window
layer, and prompts long enough for the tcgen05 product, so that replay in bfloat16 goes
through those kernels too:

  TINY_C      2    160     4    2   128       512      272   320   5e5    1e-5   no    40 (layer 0)  16
"""
from __future__ import annotations

import json
import math
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TINY_A = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
              vocab_size=256, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
              max_position_embeddings=128, attention_bias=False, sliding_window=None,
              use_sliding_window=False)
TINY_A_RUN = dict(seed=0, sigma=0.02, page_size=16)

TINY_B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=96, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=224,
              vocab_size=384, rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False,
              max_position_embeddings=256, attention_bias=False, sliding_window=24,
              layer_types=["full_attention", "sliding_attention", "full_attention"])
TINY_B_RUN = dict(seed=1, sigma=0.03, page_size=8)

TINY_C = dict(architectures=["Qwen3ForCausalLM"], hidden_size=160, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=272,
              vocab_size=320, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=False,
              max_position_embeddings=512, attention_bias=False, sliding_window=40,
              layer_types=["sliding_attention", "full_attention"])
TINY_C_RUN = dict(seed=2, sigma=0.03, page_size=16)

TINIES = {"A": (TINY_A, TINY_A_RUN), "B": (TINY_B, TINY_B_RUN), "C": (TINY_C, TINY_C_RUN)}


def make_model_dir(path, config, seed, sigma, gain_sigma=0.1):
    from tgo_b200.weights.random_init import write_random_model
    write_random_model(str(path), config, seed=seed, sigma=sigma, gain_sigma=gain_sigma)
    return str(path)


def random_requests(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, n).tolist() for i, n in enumerate(lengths)}


def round_up(n, m):
    return (n + m - 1) // m * m


# ------------------------------------------------------------------------ traces
# A trace is a list of steps as trace_run reads them. `keys_of(trace)` gives, per step,
# the (request id, absolute position) of every wanted row, in file order.


def keys_of(trace):
    held = {}
    out = {}
    for st in trace:
        ks = []
        for e in st["entries"]:
            base = held.get(e["id"], 0)
            ks += [(e["id"], base + w) for w in e["want"]]
            held[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            held.pop(rid, None)
        if ks:
            out[st["step"]] = ks
    return out


def max_tokens_of(trace, quantum=64):
    """The most tokens live requests hold at any time, each rounded up to `quantum`."""
    held, peak = {}, 0
    for st in trace:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(round_up(n, quantum) for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def trace_whole(requests):
    """Each request alone, whole, every position wanted."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
             "end": [rid]} for i, (rid, toks) in enumerate(requests.items())]


def trace_tail(requests, tail=32):
    """Most of each request in one step, then the last `tail` tokens one by one."""
    trace, step = [], 0
    for rid, toks in requests.items():
        head = max(0, len(toks) - tail)
        if head:
            trace.append({"step": step, "entries": [
                {"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
            step += 1
        for i in range(head, len(toks)):
            trace.append({"step": step, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            step += 1
    return trace


def trace_portions(requests, sizes=(7, 2, 5, 3, 2, 16, 9, 4, 2, 31, 64)):
    """Each request alone, in portions of changing size, down to two tokens."""
    trace, step = [], 0
    for rid, toks in requests.items():
        o, k = 0, 0
        while o < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - o)
            if len(toks) - o - n == 1:      # never leave a single token over: portions >= 2
                n += 1
            k += 1
            trace.append({"step": step, "entries": [
                {"id": rid, "tokens": toks[o:o + n], "want": list(range(n))}],
                "end": [rid] if o + n == len(toks) else []})
            o += n
            step += 1
    return trace


def trace_mixed(requests, seed=0, max_live=4, tail=32):
    """Up to `max_live` live requests: prompt portions of some beside single (decoded)
    tokens of others; a request may sit a step out; a finished request ends and the next
    one starts, so its pages are used again."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live = {}
    trace, step = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, end = [], []
        rids = list(live)
        for rid in rids:
            toks, o = live[rid]
            if len(rids) > 1 and rng.random() < 0.2:
                continue
            left = len(toks) - o
            if left <= tail:
                n = 1
            else:
                n = int(min(rng.integers(2, 20), left - tail))
                if n < 2:
                    n = min(2, left)
            entries.append({"id": rid, "tokens": toks[o:o + n], "want": list(range(n))})
            live[rid][1] = o + n
            if o + n == len(toks):
                end.append(rid)
        if not entries:
            continue
        for rid in end:
            del live[rid]
        trace.append({"step": step, "entries": entries, "end": end})
        step += 1
    return trace


# ----------------------------------------------------------------------- running


def run_trace_engine(engine, trace):
    """Drive an Engine in-process; {(id, position): logits row (numpy float32)}."""
    from tgo_b200.engine.step import StepEntry
    keys = keys_of(trace)
    out = {}
    for st in trace:
        entries = []
        for e in st["entries"]:
            if e["id"] not in engine.cache.requests:
                engine.admit(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = engine.step(entries)
        if st["step"] in keys:
            arr = logits.float().cpu().numpy()
            assert arr.shape[0] == len(keys[st["step"]])
            for row, k in zip(arr, keys[st["step"]]):
                out[k] = row
        for rid in st["end"]:
            engine.finish(rid)
        engine.cache.check_invariants()
    return out


def run_trace_program(model_dir, dtype, trace, out_dir, vocab, max_tokens=None, extra=()):
    """Drive bin/trace_run as a subprocess, waiting for `done <step>` after each line."""
    os.makedirs(out_dir, exist_ok=True)
    n = max_tokens or max_tokens_of(trace)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(n)] + list(extra)
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for st in trace:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"trace_run said {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    out = {}
    for step, ks in keys_of(trace).items():
        arr = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(ks), vocab)
        for row, k in zip(arr, ks):
            out[k] = row
    return out


def plain_logits(model_dir, requests):
    import plain_qwen3 as plain
    cfg, w = plain.load_model_dir(model_dir)
    return {rid: plain.forward(cfg, w, toks) for rid, toks in requests.items()}


def tolerance(config, dtype, scale):
    """Allowed absolute difference between engine logits and the float64 yardstick.

    float32: the reference's derived bound for a float32 graph against its float64 oracle,
    8 * (2L+1) * sqrt(d) * 2^-24 * 10 (model/graph_rig_test.go:538-549), times the logits'
    magnitude. bfloat16: activations are rounded to 8 significant bits about six times a
    layer (norm output, q/k/v, attention output, projection output, gate, feed-forward
    output) and the errors add like a random walk: 4 * sqrt(6L + 2) * 2^-9.
    """
    L, d = config["num_hidden_layers"], config["hidden_size"]
    if dtype == "float32":
        return 8 * (2 * L + 1) * math.sqrt(d) * 2.0 ** -24 * 10 * max(scale, 1.0)
    return 4 * math.sqrt(6 * L + 2) * 2.0 ** -9 * max(scale, 1.0)


def compare(got, want, config, dtype):
    """got: {(id, pos): row}; want: {id: [T, V]}. Returns the worst (error, key)."""
    worst, where = 0.0, None
    scale = max(float(np.abs(v).max()) for v in want.values())
    for (rid, pos), row in sorted(got.items()):
        err = float(np.abs(row.astype(np.float64) - want[rid][pos]).max())
        if not np.isfinite(err):
            return float("inf"), (rid, pos), tolerance(config, dtype, scale)
        if err > worst:
            worst, where = err, (rid, pos)
    return worst, where, tolerance(config, dtype, scale)


def repeated_layers_reference(pc, pw, tokens):
    """Plain logits of TINY_A's weights run as calls [0, 1, 0, 1] where the last call reads
    the cache of call 1 instead of writing its own (keys and values of call 1, queries of
    its own input)."""
    import plain_qwen3 as plain
    eps, T = pc["rms_norm_eps"], len(tokens)
    pos = np.arange(T)
    h = plain.embedding(pw["model.embed_tokens.weight"], tokens)
    kv1 = None
    for call, layer in enumerate([0, 1, 0, 1]):
        p = f"model.layers.{layer}."
        n = plain.rmsnorm(h, pw[p + "input_layernorm.weight"], eps)
        H, hkv, dh = 4, 2, 16
        q = plain.rmsnorm(plain.linear(n, pw[p + "self_attn.q_proj.weight"]).reshape(T, H, dh),
                          pw[p + "self_attn.q_norm.weight"], eps)
        q = plain.rope_half_split(q, pos, pc["rope_theta"])
        if call == 3:
            k, v = kv1
        else:
            k = plain.rmsnorm(plain.linear(n, pw[p + "self_attn.k_proj.weight"]).reshape(T, hkv, dh),
                              pw[p + "self_attn.k_norm.weight"], eps)
            k = plain.rope_half_split(k, pos, pc["rope_theta"])
            v = plain.linear(n, pw[p + "self_attn.v_proj.weight"]).reshape(T, hkv, dh)
            if call == 1:
                kv1 = (k, v)
        a = plain.causal_gqa_attention(q, k, v, 0.25).reshape(T, H * dh)
        h = h + plain.linear(a, pw[p + "self_attn.o_proj.weight"])
        n = plain.rmsnorm(h, pw[p + "post_attention_layernorm.weight"], eps)
        h = h + plain.swiglu_mlp(n, pw[p + "mlp.gate_proj.weight"], pw[p + "mlp.up_proj.weight"],
                                 pw[p + "mlp.down_proj.weight"])
    return plain.linear(plain.rmsnorm(h, pw["model.norm.weight"], eps),
                        pw["model.embed_tokens.weight"])
