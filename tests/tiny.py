"""Tiny configurations, random model folders and trace builders shared by the tests.

Two configurations of the one architecture that differ in every size and option:

            layers hidden heads kv  head_dim  q width  inter vocab  theta  eps    tied  window  page
  TINY_A      2     64     4    2    16        64      128   256   1e4    1e-6   yes   none     16
  TINY_B      3     96     6    2    32       192      224   384   1e6    1e-5   no    24 (layer 1)  8

In A the q width equals the hidden size and layers equal kv heads, so a confusion of
those two pairs passes there; B is the configuration that tells them apart.

A third, TINY_C, has the head size (128) that the tcgen05 attention kernel and the TMA-fed
decode kernel take, and a window layer, so that replay in bfloat16 goes through those
kernels too. (The tcgen05 product starts above 1024 rows: tests/test_schedules_gpu.py runs
Tiny C with a 1200-token request, and with the threshold lowered to 65 rows.)

  TINY_C      2    160     4    2   128       512      272   320   5e5    1e-5   no    40 (layer 0)  16

A fourth, TINY_D, is wide instead of tiny where the decode kernels ask for it: hidden size,
q width and intermediate size of 2048, so that at 1 to 8 rows every product of a layer and
the vocabulary product take the persistent form of the weight-streaming kernel, with the two
norms folded into the q/k/v and gate/up products (tests/test_schedules_gpu.py).

  TINY_D      2   2048    16    4   128      2048     2048   512   1e6    1e-6   no    none          16
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

TINY_D = dict(architectures=["Qwen3ForCausalLM"], hidden_size=2048, num_hidden_layers=2,
              num_attention_heads=16, num_key_value_heads=4, head_dim=128, intermediate_size=2048,
              vocab_size=512, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False,
              max_position_embeddings=512, attention_bias=False, sliding_window=None,
              use_sliding_window=False)
TINY_D_RUN = dict(seed=4, sigma=0.02, page_size=16)


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


def held_pages(engine):
    """Per group, {page: request id} over the live requests' block tables."""
    out = [dict() for _ in engine.cache.groups]
    for rid, req in engine.cache.requests.items():
        for g in range(len(out)):
            for p in req.held(g):
                out[g][p] = rid
    return out


def poison_unheld(engine):
    """NaN into every page no live request holds: pages never handed out, pages of finished
    requests, pages a window has passed."""
    for g, held in enumerate(held_pages(engine)):
        n = engine.cache.pools[g].num_pages
        engine.storage.poison_pages(g, [p for p in range(1, n + 1) if p not in held])


def run_trace_engine(engine, trace, poison=False, owners=None):
    """Drive an Engine in-process; {(id, position): logits row (numpy float32)}.
    poison: before the first step, and after every step and every end of a request, every
    page that no live request holds is filled with NaN. owners: a list (one dict per cache
    group) that collects {page: set of request ids that ever held it}."""
    from tgo_b200.engine.step import StepEntry
    keys = keys_of(trace)
    out = {}
    if poison:
        poison_unheld(engine)
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
        if owners is not None:
            for g, held in enumerate(held_pages(engine)):
                for p, rid in held.items():
                    owners[g].setdefault(p, set()).add(rid)
        for rid in st["end"]:
            engine.finish(rid)
        if poison:
            poison_unheld(engine)
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


def plain_logits_rounded(model_dir, requests):
    """The plain implementation with bfloat16-rounded activations: the scale of the bound
    for a bfloat16 engine (see `tolerance`)."""
    import plain_qwen3 as plain
    cfg, w = plain.load_model_dir(model_dir)
    return {rid: plain.forward_rounded(cfg, w, toks) for rid, toks in requests.items()}


def tolerance(config, dtype, reference, rounded=None):
    """Allowed absolute difference between engine logits and the float64 yardstick.
    `reference`: the yardstick's logits (an array or several).

    float32: the reference's derived bound for a float32 graph against its float64 oracle,
    8 * (2L+1) * sqrt(d) * 2^-24 * 10 (model/graph_rig_test.go:538-549), times the largest
    logit (at least 1).

    bfloat16: `rounded` holds the logits of the plain implementation run with every
    activation rounded to bfloat16 where a bfloat16 engine stores one
    (plain_qwen3.forward_rounded), for the same inputs as `reference`. Its largest
    difference from `reference` is what rounding alone does to this model on these inputs;
    an engine may differ from the yardstick by twice that (its sums run in another order, it
    rounds a few more intermediate values, and the largest of some 10^5 errors varies from
    one draw to the next). The bound therefore follows the model: it is small where the
    model damps rounding errors and larger where large weights amplify them, and it has no
    floor."""
    L, d = config["num_hidden_layers"], config["hidden_size"]
    arrays = reference if isinstance(reference, (list, tuple)) else [reference]
    if dtype == "float32":
        top = max(float(np.abs(np.asarray(a)).max()) for a in arrays)
        return 8 * (2 * L + 1) * math.sqrt(d) * 2.0 ** -24 * 10 * max(top, 1.0)
    if rounded is None:
        raise ValueError("tolerance: the bfloat16 bound needs the rounded plain logits")
    others = rounded if isinstance(rounded, (list, tuple)) else [rounded]
    return 2.0 * max(float(np.abs(np.asarray(r, dtype=np.float64) - a).max())
                     for r, a in zip(others, arrays))


def note(what, worst, allowed):
    """With TGO_TOLERANCE_LOG=<file>: append how much of its bound a comparison used."""
    path = os.environ.get("TGO_TOLERANCE_LOG")
    if path:
        with open(path, "a") as f:
            f.write(f"{what}\t{worst:.4e}\t{allowed:.4e}\t{worst / allowed if allowed else 0:.3f}\n")


def compare(got, want, config, dtype, what="", rounded=None):
    """got: {(id, pos): row}; want: {id: [T, V]}; rounded: {id: [T, V]} of the rounded plain
    implementation (bfloat16 only). Returns the worst (error, key) and the allowed error."""
    worst, where = 0.0, None
    ids = list(want)
    allowed = tolerance(config, dtype, [want[i] for i in ids],
                        None if dtype == "float32" else [rounded[i] for i in ids])
    for (rid, pos), row in sorted(got.items()):
        err = float(np.abs(row.astype(np.float64) - want[rid][pos]).max())
        if not np.isfinite(err):
            return float("inf"), (rid, pos), allowed
        if err > worst:
            worst, where = err, (rid, pos)
    note(what or f"compare/{dtype}/L{config['num_hidden_layers']}", worst, allowed)
    return worst, where, allowed


def repeated_layers_reference(pc, pw, tokens, rnd=None):
    """Plain logits of TINY_A's weights run as calls [0, 1, 0, 1] where the last call reads
    the cache of call 1 instead of writing its own (keys and values of call 1, queries of
    its own input). rnd: round the activations a bfloat16 engine stores (see
    plain_qwen3.forward_rounded)."""
    import plain_qwen3 as plain
    rnd = rnd or (lambda x: x)
    eps, T = pc["rms_norm_eps"], len(tokens)
    pos = np.arange(T)
    h = plain.embedding(pw["model.embed_tokens.weight"], tokens)
    kv1 = None
    for call, layer in enumerate([0, 1, 0, 1]):
        p = f"model.layers.{layer}."
        n = rnd(plain.rmsnorm(h, pw[p + "input_layernorm.weight"], eps))
        H, hkv, dh = 4, 2, 16
        q = plain.rmsnorm(rnd(plain.linear(n, pw[p + "self_attn.q_proj.weight"])).reshape(T, H, dh),
                          pw[p + "self_attn.q_norm.weight"], eps)
        q = rnd(plain.rope_half_split(q, pos, pc["rope_theta"]))
        if call == 3:
            k, v = kv1
        else:
            k = plain.rmsnorm(rnd(plain.linear(n, pw[p + "self_attn.k_proj.weight"])).reshape(T, hkv, dh),
                              pw[p + "self_attn.k_norm.weight"], eps)
            k = rnd(plain.rope_half_split(k, pos, pc["rope_theta"]))
            v = rnd(plain.linear(n, pw[p + "self_attn.v_proj.weight"])).reshape(T, hkv, dh)
            if call == 1:
                kv1 = (k, v)
        a = rnd(plain.causal_gqa_attention(q, k, v, 0.25, round_weights=rnd)).reshape(T, H * dh)
        h = h + rnd(plain.linear(a, pw[p + "self_attn.o_proj.weight"]))
        n = rnd(plain.rmsnorm(h, pw[p + "post_attention_layernorm.weight"], eps))
        gate = rnd(plain.linear(n, pw[p + "mlp.gate_proj.weight"]))
        up = rnd(plain.linear(n, pw[p + "mlp.up_proj.weight"]))
        h = h + rnd(plain.linear(rnd(plain.silu(gate) * up), pw[p + "mlp.down_proj.weight"]))
    return plain.linear(rnd(plain.rmsnorm(h, pw["model.norm.weight"], eps)),
                        pw["model.embed_tokens.weight"])
