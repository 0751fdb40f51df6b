#!/usr/bin/env python3
"""Headline measurement: decode tokens a second of a Qwen3-8B-shaped model with random
bfloat16 weights at batch 8 (1,024-token prompts), on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step. Prints one JSON line: `value` is decoded tokens a second timed
on the device over exactly K steps; `e2e` is the same through the Python entry point
(scheduler, sampling, host tokens in and out); `prefill` a 2,048-token prompt; `roofline`
the bytes a decode step must read over its time against the measured copy bandwidth;
`points` decoding at batch 1 and 64.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# configs[2] of the baseline record: the Qwen3-8B shape
CONFIG_8B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=36,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                 intermediate_size=12288, vocab_size=151936, rms_norm_eps=1e-6,
                 rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=40960,
                 attention_bias=False, sliding_window=None, use_sliding_window=False)
# configs[3] and configs[4]: the 14B and 32B shapes (--shape 14b / 32b; the contract line is
# the 8B one)
CONFIG_14B = dict(CONFIG_8B, hidden_size=5120, num_hidden_layers=40, num_attention_heads=40,
                  intermediate_size=17408)
CONFIG_32B = dict(CONFIG_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64,
                  intermediate_size=25600)
SHAPES = {"8b": (CONFIG_8B, 8), "14b": (CONFIG_14B, 14), "32b": (CONFIG_32B, 32)}
SEED = 8
PROMPT = 1024
CONTEXT_CAP = 8192
PAGE = 16
PREFILL_TOKENS = 2048


class ClockSampler:
    """nvidia-smi in the background during the timed region (reads only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(index), "-lms", "200"], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm():
    """The reference is a Go program (go.mod wants Go 1.27, and its device layer is an
    external Go module); there is no Go toolchain here and pip cannot install it."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "latere-ai/tgo is Go (no setup.py/pyproject; needs Go 1.27 and the "
                      "external golang.design/x/accel module, neither present offline); "
                      "pip install of the reference checkout fails"}))
    return 0


def e2e_decode(model, batch, steps, warmup):
    """Decode tokens a second through the public entry point: new_scheduler, admit, then
    Runner steps (plan, pack inputs in pinned memory, copy, run, sample on the device,
    read the ids back, feed). Timed with the host clock around exactly `steps` steps."""
    import torch

    from tgo_b200.engine.measure import random_prompts, round_up
    from tgo_b200.engine.scheduler import Request, Runner
    from tgo_b200.sampling.policy import Policy
    from tgo_b200.sampling.sampler import sample_rows
    total = warmup + steps + 2
    sched = model.new_scheduler(batch, chunk=PREFILL_TOKENS, reserve=total,
                                pool_tokens=batch * round_up(PROMPT + total, 64), page_size=PAGE,
                                max_batched_tokens=8192)
    runner = Runner(sched, sample_rows)
    prompts = random_prompts(model.spec.vocab_size, batch, PROMPT, SEED + 1)
    reqs = [Request(p, Policy(max_tokens=total), request_id=i) for i, p in enumerate(prompts)]
    for r in reqs:
        runner.submit(r)
    while min(len(r.output) for r in reqs) < warmup + 1:
        runner.run_step()
    torch.cuda.synchronize()
    before = sum(len(r.output) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(steps):
        runner.run_step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = sum(len(r.output) for r in reqs) - before
    h2d = sched.engine.h2d_bytes_last
    for slot in list(runner.by_slot):
        sched.finish(slot)
    return {"value": made / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * batch, "ms_per_step": dt / steps * 1e3}


def serve_workload(model, config, shape):
    """The continuous-batching workload of the baseline record's 14B configuration, through
    the library's generate: 32 requests, prompt lengths uniform in [128, 4096], outputs uniform
    in [64, 512], prompt portions of 512 tokens, pages of 16, up to 8192 tokens a request.
    Run twice over one scheduler, as a server would hold it (the first run also compiles
    kernels and captures the decode graphs); the second is reported."""
    import time

    import numpy as np
    import torch

    from tgo_b200.sampling.policy import Policy
    rng = np.random.default_rng(14)
    n = 32
    plens, olens = rng.integers(128, 4097, n), rng.integers(64, 513, n)
    prompts = [rng.integers(0, config["vocab_size"], int(p)).tolist() for p in plens]
    policies = [Policy(max_tokens=int(o)) for o in olens]
    # prompt portions of 512 tokens as the record says; a step carries up to 1024 tokens (two
    # portions, or one and the decoding requests' tokens): measured 5.59 s against 5.88 s with
    # steps of 512, and 5.56 s with 1536
    scheduler = model.new_scheduler(n, chunk=512, reserve=int(olens.max()), pool_tokens=n * CONTEXT_CAP,
                                    page_size=PAGE, max_batched_tokens=1024)
    for _ in range(2):
        torch.cuda.synchronize()
        t0 = time.time()
        outs = model.generate(prompts, policies, scheduler=scheduler)
        torch.cuda.synchronize()
        seconds = time.time() - t0
    generated = sum(len(o) for o in outs)
    print(json.dumps({"only": "serve", "shape": shape, "layers": config["num_hidden_layers"],
                      "requests": n, "prompt_tokens": int(plens.sum()), "generated_tokens": generated,
                      "seconds": round(seconds, 3),
                      "generated_tokens_per_s": round(generated / seconds, 1),
                      "tokens_per_s": round((generated + int(plens.sum())) / seconds, 1)}))
    return 0


def exactness_check(config, seed, shape):
    """Logits at real layer sizes under different ways of cutting the work. Three requests
    (1500, 300 and 65 prompt tokens, then 8 given tokens each; 1500 rows in a step take the
    tcgen05 product) run (a) each alone, the prompt
    in one step and the rest token by token; (b) together, at most two live at a time in a
    pool that holds just those two, the prompts in portions of changing size (down to two
    tokens) beside the single tokens of the others, the third request in pages the second
    gave back. Both in true float32 and in bfloat16, with the same seeded weights. Compared:
    float32 (b) with float32 (a); bfloat16 (a) and (b) with float32 (a), against the bound
    the tests use for bfloat16 (activations rounded to 8 bits about six times a layer, a
    random walk: 4 * sqrt(6 L + 2) * 2^-9 times the largest logit)."""
    import math

    import numpy as np
    import torch

    import tgo_b200
    from tgo_b200.engine.measure import round_up
    from tgo_b200.engine.step import Engine, StepEntry
    V, L = config["vocab_size"], config["num_hidden_layers"]
    rng = np.random.default_rng(5)
    lens, extra, tail = [1500, 300, 65], 8, 24
    toks = [rng.integers(0, V, n + extra).tolist() for n in lens]

    def alone(model):
        eng = Engine(model, page_size=PAGE, max_tokens=round_up(max(lens) + extra, 64), num_slots=1)
        out = []
        for rid, (n, t) in enumerate(zip(lens, toks)):
            eng.admit(rid)
            rows = [eng.step([StepEntry(rid, t[:n], list(range(n - tail, n)))]).float().cpu()]
            for j in range(extra):      # a step's logits are only good until the next step
                rows.append(eng.step([StepEntry(rid, [t[n + j]], [0])]).float().cpu())
            eng.finish(rid)
            out.append(torch.cat(rows))
        eng.check_kernels()
        return out

    def together(model):
        eng = Engine(model, page_size=PAGE, num_slots=2,
                     max_tokens=round_up(lens[0] + extra, 64) + round_up(lens[1] + extra, 64))
        sizes = [129, 2, 1100, 64, 33, 300, 7]
        fed, turn, rows = [0, 0, 0], [0, 1, 2], [[], [], []]
        live, waiting = [0, 1], [2]
        for rid in live:
            eng.admit(rid)
        while live:
            entries, owners = [], []
            for rid in live:
                n, t, at = lens[rid], toks[rid], fed[rid]
                if at < n:
                    k = min(sizes[turn[rid] % len(sizes)], n - at)
                    turn[rid] += 1
                    want = [p - at for p in range(max(at, n - tail), at + k) if p < n]
                else:
                    k, want = 1, [0]
                entries.append(StepEntry(rid, t[at:at + k], want))
                owners += [rid] * len(want)
                fed[rid] = at + k
            logits = eng.step(entries).float().cpu()
            for row, rid in zip(logits, owners):
                rows[rid].append(row)
            for rid in list(live):
                if fed[rid] == lens[rid] + extra:
                    eng.finish(rid)
                    live.remove(rid)
                    if waiting:
                        nxt = waiting.pop(0)
                        eng.admit(nxt)
                        live.append(nxt)
        eng.check_kernels()
        return [torch.stack(r) for r in rows]

    got = {}
    for dtype in ("float32", "bfloat16"):
        model = tgo_b200.open_random(config, seed=seed, dtype=dtype, sigma=0.02, gain_sigma=0.05)
        got[dtype] = (alone(model.model), together(model.model))
        del model
        torch.cuda.empty_cache()
    ref = got["float32"][0]
    scale = max(float(r.abs().max()) for r in ref)
    rms = math.sqrt(sum(float((r.double() ** 2).sum()) for r in ref) / sum(r.numel() for r in ref))

    def worst(a, b):
        return max(float((x.double() - y.double()).abs().max()) for x, y in zip(a, b))

    def top1(a, b):
        same = sum(int((x.argmax(-1) == y.argmax(-1)).sum()) for x, y in zip(a, b))
        return same / sum(x.shape[0] for x in a)
    bound_bf16 = 4 * math.sqrt(6 * L + 2) * 2.0 ** -9 * scale
    bound_f32 = 8 * (2 * L + 1) * math.sqrt(config["hidden_size"]) * 2.0 ** -24 * 10 * max(scale, 1.0)
    line = {"only": "check", "shape": shape, "layers": L, "positions": sum(r.shape[0] for r in ref),
            "vocab": V, "largest_logit": round(scale, 4), "logit_rms": round(rms, 4),
            "float32_cut_vs_alone_max_abs": worst(got["float32"][1], ref), "float32_bound": bound_f32,
            "bfloat16_alone_vs_float32_max_abs": round(worst(got["bfloat16"][0], ref), 5),
            "bfloat16_cut_vs_float32_max_abs": round(worst(got["bfloat16"][1], ref), 5),
            "bfloat16_cut_vs_alone_max_abs": round(worst(got["bfloat16"][1], got["bfloat16"][0]), 5),
            "bfloat16_bound": round(bound_bf16, 5),
            "bfloat16_top1_agrees_with_float32": round(top1(got["bfloat16"][1], ref), 4)}
    line["ok"] = bool(line["float32_cut_vs_alone_max_abs"] <= bound_f32 and
                      line["bfloat16_alone_vs_float32_max_abs"] <= bound_bf16 and
                      line["bfloat16_cut_vs_float32_max_abs"] <= bound_bf16)
    print(json.dumps(line))
    return 0 if line["ok"] else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the 36 (0: all)")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64, and prefill")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES),
                    help="with --only: the 14B or 32B shape of the baseline record instead of the 8B one")
    ap.add_argument("--prompt", type=int, default=PROMPT, help="with --only decode: prompt length")
    ap.add_argument("--rows", default="256,512,1024,2048", help="with --only products: row counts")
    ap.add_argument("--only", default="", choices=["", "prefill", "decode", "serve", "check", "products"],
                    help="run just the 2,048-token prefill, just the decode steps, the "
                         "continuous-batching workload, or the exactness check at real layer "
                         "sizes (float32 against bfloat16, alone against cut and mixed; 4 layers "
                         "unless --layers says otherwise), or the four matrix products of a layer "
                         "at the --rows row counts against the library product, and print a "
                         "short line instead of the contract line")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print("bench: this engine runs on one GPU; --gpus must be 1")
        return 2
    warmup = max(args.warmup, 3)

    import torch

    import tgo_b200
    from tgo_b200.engine.measure import load_peaks, measure_decode, measure_prefill

    if args.shape != "8b" and not args.only:
        print("bench: the contract line is measured on the 8B shape; give --only with --shape")
        return 2
    config, seed = dict(SHAPES[args.shape][0]), SHAPES[args.shape][1]
    if args.layers:
        config["num_hidden_layers"] = args.layers
    if args.only == "check":
        if not args.layers:
            config["num_hidden_layers"] = 4
        return exactness_check(config, seed, args.shape)
    if args.only == "products":
        from tgo_b200.engine.measure import measure_products
        for rec in measure_products(config, [int(r) for r in args.rows.split(",") if r]):
            print(json.dumps({k: (round(v, 1) if isinstance(v, float) else v) for k, v in rec.items()}))
        return 0
    model = tgo_b200.open_random(config, seed=seed, dtype="bfloat16", sigma=0.02, gain_sigma=0.05)
    peaks = load_peaks()
    if args.only == "prefill":
        pre = measure_prefill(model, PREFILL_TOKENS, warmup=2, steps=max(1, min(args.steps, 3)),
                              seed=SEED, page_size=PAGE)
        print(json.dumps({"only": "prefill", "shape": args.shape, "layers": config["num_hidden_layers"],
                          "ms": round(pre["ms"], 3), "tokens_per_s": round(pre["tokens_per_s"], 1),
                          "tflops": round(pre["tflops"], 1),
                          "frac": round(pre["tflops"] / peaks["bf16_tflops"], 4)}))
        return 0
    if args.only == "serve":
        return serve_workload(model, config, args.shape)
    if args.only == "decode":
        r = measure_decode(model, args.batch, args.prompt, args.steps, warmup=warmup, seed=SEED,
                           page_size=PAGE)
        print(json.dumps({"only": "decode", "shape": args.shape, "layers": config["num_hidden_layers"],
                          "batch": args.batch, "prompt": args.prompt,
                          "ms_per_step": round(r["ms_per_step"], 4),
                          "tokens_per_s": round(r["tokens_per_s"], 1), "gbs": round(r["gbs"], 1),
                          "hbm_frac": round(r["gbs"] / peaks["hbm_gbs"], 3)}))
        return 0

    # the prefill first: it is the one measurement bound by the power cap, and it is compared
    # with a peak that was measured as a short burst
    prefill = None
    if not args.no_points:
        pre = measure_prefill(model, PREFILL_TOKENS, warmup=3, steps=3, seed=SEED, page_size=PAGE)
        prefill = {"value": round(pre["tokens_per_s"], 1), "tokens": PREFILL_TOKENS,
                   "ms": round(pre["ms"], 3),
                   "frac": round(pre["tflops"] / peaks["bf16_tflops"], 4)}
    clocks = ClockSampler()
    main_run = measure_decode(model, args.batch, PROMPT, args.steps, warmup=warmup, seed=SEED,
                              page_size=PAGE)
    clock_record = clocks.stop()
    e2e = e2e_decode(model, args.batch, args.steps, warmup)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            r = measure_decode(model, b, PROMPT, min(args.steps, 128), warmup=warmup, seed=SEED,
                               page_size=PAGE)
            points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(r["gbs"] / peaks["hbm_gbs"], 3)
    line = {
        "metric": "decode tokens/s, Qwen3-8B shape, batch 8, 1024-token prompts",
        "value": round(main_run["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random N(0,0.02) weights",
        "config": {"model": "Qwen3-8B shape", "layers": config["num_hidden_layers"],
                   "layers_of_full_model": 36, "hidden": 4096, "heads": 32, "kv_heads": 8,
                   "head_dim": 128, "intermediate": 12288, "vocab": 151936,
                   "global_batch": args.batch, "seq_len": PROMPT, "context_cap": CONTEXT_CAP,
                   "page_size": PAGE, "prefill_tokens": PREFILL_TOKENS, "seed": SEED,
                   "parallelism": "1 GPU",
                   "l2": "inputs larger than L2: every step streams all weights from HBM",
                   "order": "prefill, decode batch 8, end to end, batch 1, batch 64",
                   "peaks": peaks["source"]},
        "clocks": clock_record, "e2e": {k: (round(v, 2) if isinstance(v, float) else v)
                                        for k, v in e2e.items()},
        "gpu_launches": main_run["gpu_launches"],
        "roofline": {"bound": "hbm", "achieved": round(main_run["gbs"], 1),
                     "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["gbs"] / peaks["hbm_gbs"], 4)},
        "points": points,
    }
    if prefill is not None:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
