"""Timing of the two workloads the reference's `tgo bench` reports (cmd/tgo/bench.go:
168-246: warm up, reset, measure; prefill of a synthetic prompt, then decode steps), on
the device with CUDA events, plus the arithmetic for roofline fractions.

Prompts are seeded uniform-random token ids. A decode step of a model larger than the L2
cache reads its weights from HBM every time, so no flush is needed between steps; for
small models `flush_l2` writes a buffer larger than L2 between timed steps.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .step import Engine, StepEntry

L2_BYTES = 126 * 1024 * 1024


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def model_flops(model, n_tokens: int, first_position: int = 0, n_logit_rows: int = 1) -> float:
    """Floating-point operations of one step that runs `n_tokens` tokens of one request
    starting at `first_position`: what every part of every call counts for itself (2 per
    multiply-add of its matrix products, and of q.K and w.V over the keys each token may
    read), plus the head's product. A part that counts nothing adds nothing."""
    return model.flops([n_tokens], [first_position], n_logit_rows)


def decode_bytes(model, context_lens) -> float:
    """Bytes a decode step has to read: every weight it uses once, and what every mixer says
    it reads of the live requests' cache (attention: keys and values, a window layer at most
    its window)."""
    return model.weight_bytes() + sum(model.cache_bytes_read(c) for c in context_lens)


def load_peaks(path: Optional[str] = None) -> Dict[str, object]:
    """Measured peaks of this pool if the driver wrote them, else the stated fallback."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = path or os.path.join(here, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
           "source": "fallback"}
    try:
        with open(path) as f:
            raw = json.load(f)

        def find(d, key):
            if isinstance(d, dict):
                if key in d and isinstance(d[key], (int, float)):
                    return float(d[key])
                for v in d.values():
                    r = find(v, key)
                    if r is not None:
                        return r
            return None
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            v = find(raw, key)
            if v:
                out[key] = v
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class L2Flusher:
    def __init__(self, device):
        self.buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.fill_(1)


def random_prompts(vocab: int, n: int, length: int, seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n, length), generator=g).tolist()


def measure_prefill(loaded, tokens: int, warmup: int = 3, steps: int = 3, seed: int = 0,
                    page_size: int = 16) -> dict:
    """One request of `tokens` prompt tokens in one step, logits of its last token."""
    model = loaded.model
    eng = Engine(model, page_size=page_size, max_tokens=round_up(tokens, 64), num_slots=1)
    prompt = random_prompts(model.spec.vocab_size, 1, tokens, seed)[0]
    flush = L2Flusher(model.device)
    times = []
    for i in range(warmup + steps):
        eng.admit("p")
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([StepEntry("p", prompt, [tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        eng.finish("p")
        if i >= warmup:
            times.append(a.elapsed_time(b))
    ms = sum(times) / len(times)
    flops = model_flops(model, tokens)
    return {"tokens": tokens, "ms": ms, "tokens_per_s": tokens / ms * 1e3, "flops": flops,
            "tflops": flops / ms / 1e9, "steps": steps}


def measure_decode(loaded, batch: int, prompt_len: int, tokens: int, warmup: int = 8,
                   seed: int = 0, page_size: int = 16, prefill_budget: int = 8192,
                   flush_l2: bool = False) -> dict:
    """`batch` requests with `prompt_len`-token prompts decode `tokens` steps greedily.
    Each step: copy the step's inputs to the device, run the step, pick the argmax on the
    device, read the ids back (they are the next step's inputs). Timed as a whole with
    CUDA events around the `tokens` steps, and per step for the percentiles."""
    model = loaded.model
    V = model.spec.vocab_size
    per_req = round_up(prompt_len + warmup + tokens + 1, 64)
    eng = Engine(model, page_size=page_size, max_tokens=batch * per_req, num_slots=batch)
    prompts = random_prompts(V, batch, prompt_len, seed)
    ids = [f"d{i}" for i in range(batch)]
    for r in ids:
        eng.admit(r, prompt_len + warmup + tokens + 1)
    out_ids = torch.empty(batch, dtype=torch.int32, device=model.device)
    feed = [0] * batch
    # prompts, several requests a step within the token budget
    i = 0
    while i < batch:
        group, used = [], 0
        while i < batch and (not group or used + prompt_len <= prefill_budget):
            group.append(i)
            used += prompt_len
            i += 1
        logits = eng.step([StepEntry(ids[j], prompts[j], [prompt_len - 1]) for j in group])
        tmp = torch.empty(len(group), dtype=torch.int32, device=model.device)
        ops.argmax(logits, tmp)
        for j, t in zip(group, tmp.tolist()):
            feed[j] = t
    flush = L2Flusher(model.device) if flush_l2 else None
    step_ms, events = [], []
    launches0 = 0
    for s in range(warmup + tokens):
        if s == warmup:
            torch.cuda.synchronize()
            launches0 = ops.LAUNCHES[0]
            start = torch.cuda.Event(enable_timing=True)
            start.record()
        if flush is not None:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        logits = eng.step([StepEntry(ids[j], [feed[j]], [0]) for j in range(batch)])
        ops.argmax(logits, out_ids)
        b.record()
        feed = out_ids.tolist()
        if s >= warmup:
            events.append((a, b))
    end = torch.cuda.Event(enable_timing=True)
    end.record()
    torch.cuda.synchronize()
    total_ms = start.elapsed_time(end)
    step_ms = sorted(a.elapsed_time(b) for a, b in events)
    launches = ops.LAUNCHES[0] - launches0
    ctx = [eng.length(r) for r in ids]
    mean_ctx = [c - tokens / 2 for c in ctx]
    nbytes = decode_bytes(model, mean_ctx)
    ms_per_step = total_ms / tokens
    dev_ms = sum(step_ms) / len(step_ms)

    def rank(p):
        return step_ms[min(len(step_ms) - 1, max(0, int(p * len(step_ms) + 0.999999) - 1))]
    for r in ids:
        eng.finish(r)
    return {"batch": batch, "prompt_tokens": prompt_len, "tokens": tokens,
            "ms_per_step": ms_per_step, "device_ms_per_step": dev_ms,
            "tokens_per_s": batch * 1e3 / ms_per_step, "p50_ms": rank(0.5), "p90_ms": rank(0.9),
            "p99_ms": rank(0.99), "bytes_per_step": nbytes,
            "gbs": nbytes / (ms_per_step * 1e-3) / 1e9, "gpu_launches": launches,
            "h2d_bytes_per_step": 0, "final_context": ctx[0]}


def measure_products(config: dict, rows_list, repeats: int = 20) -> List[dict]:
    """The four matrix products of one layer of `config` (q/k/v, o, gate/up with the gate
    applied, down) at each row count, timed warm with CUDA events: this package's kernel for
    that row count (`ops.linear` / `ops.gated_linear`, whichever kernel they pick), the
    tcgen05 kernel forced, and the library product (for gate/up: plus this package's gate
    kernel, which the library product needs after it). Weights and inputs are seeded random."""
    d, f = config["hidden_size"], config["intermediate_size"]
    H, Hkv = config["num_attention_heads"], config.get("num_key_value_heads", config["num_attention_heads"])
    dh = config.get("head_dim", d // H)
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1)
    shapes = [("qkv", (H + 2 * Hkv) * dh, d, False), ("o", d, H * dh, False),
              ("gate_up", 2 * f, d, True), ("down", d, f, False)]

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(repeats):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / repeats * 1e3
    out = []
    for name, N, K, gated in shapes:
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        for M in rows_list:
            x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
            y = torch.empty(M, N // 2 if gated else N, dtype=torch.bfloat16, device=dev)
            rec = {"product": name, "rows": M, "N": N, "K": K, "gflop": 2.0 * M * N * K / 1e9}
            rec["ours_us"] = timed((lambda: ops.gated_linear(x, w, True)) if gated else (lambda: ops.linear(x, w)))
            if M > ops.SKINNY_MAX_ROWS * 8:
                rec["tcgen05_us"] = timed(lambda: ops.gemm_tc(x, w, y, gated=gated))
                rec["tile"] = "x".join(str(v) for v in ops.gemm_tc_last_plan())

            def library():
                gu = torch.mm(x, w.t())
                if gated:
                    ops.swiglu(gu, y, True)
            rec["library_us"] = timed(library)
            out.append(rec)
    return out
