"""Command line in the manner of `tgo` (cmd/tgo/main.go:87-180, runcmd.go:42-113,
bench.go:36-106): flags before the model folder, the same names and meanings where the
reference has them.

    tgo run     [flags] <model-dir>     generate from a prompt of token ids
    tgo bench   [flags] <model-dir>     measure prefill and decode
    tgo info            <model-dir>     architecture, precision and what memory it costs
    tgo random  [flags] <model-dir>     write a folder with seeded random weights

Text is outside this engine (no tokenizer, no chat template), so --prompt holds token
ids ("5,17,3" or "5 17 3") and --raw is accepted for compatibility and changes nothing.
Beyond the reference's flags, `run` and `bench` take `--config cfg.json --random SEED` in
place of a model folder (random weights made on the device), `run` takes --prompt several
times (the prompts then run together through the scheduler), --prompt-len, --stop-ids,
--page-size and --kv-pages, and `bench` takes a list of batch sizes.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import time

USAGE = __doc__

PRECISIONS = {"auto": "bfloat16", "bf16": "bfloat16", "bfloat16": "bfloat16", "f32": "float32",
              "float32": "float32", "fp32": "float32"}


class UsageError(Exception):
    pass


def _parser(prog):
    return argparse.ArgumentParser(prog=f"tgo {prog}", add_help=True, allow_abbrev=False)


def _common(ap):
    ap.add_argument("--precision", default="auto",
                    help="bf16, f32 or auto (default auto: bf16)")
    ap.add_argument("--context", type=int, default=4096,
                    help="cache capacity in positions (default 4096)")
    ap.add_argument("--device", default="auto", help="auto or cuda:N (default auto)")
    ap.add_argument("--temp", type=float, default=0.0,
                    help="sampling temperature; 0 is greedy (default 0)")
    ap.add_argument("--seed", type=int, default=0, help="the sampler seed (default 0)")
    ap.add_argument("--config", default="",
                    help="with --random: a config.json to build a random-weights model from, "
                         "in place of <model-dir>")
    ap.add_argument("--random", type=int, default=None, metavar="SEED",
                    help="seed of the random weights of the --config model")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    ap.add_argument("model_dir", metavar="<model-dir>", nargs="?", default="")


def run_parser():
    ap = _parser("run")
    ap.add_argument("--prompt", action="append", default=None,
                    help="the prompt, as token ids separated by commas or spaces (default "
                         "\"1 2 3 4 5 6 7 8\"); given several times, the prompts run together "
                         "through the scheduler")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="in place of --prompt: a seeded random prompt of N token ids")
    ap.add_argument("--stop-ids", default="auto",
                    help="token ids that end a completion without being part of it; auto "
                         "(default): eos_token_id of the model folder; none: no stop ids")
    ap.add_argument("--kv-pages", type=int, default=0,
                    help="pages in the cache pool (default: enough for --context per prompt)")
    ap.add_argument("--raw", action="store_true",
                    help="accepted for compatibility; prompts are always token ids")
    ap.add_argument("--max-tokens", type=int, default=128,
                    help="stop after N generated tokens (default 128)")
    ap.add_argument("--top-k", type=int, default=0,
                    help="keep the K largest candidates; 0 disables the stage")
    ap.add_argument("--top-p", type=float, default=0.0,
                    help="nucleus mass in (0, 1]; 0 disables the stage")
    ap.add_argument("--repeat-penalty", type=float, default=1.0,
                    help="divisive repetition penalty; 1 is none (default 1)")
    _common(ap)
    return ap


def bench_parser():
    ap = _parser("bench")
    ap.add_argument("--tokens", type=int, default=128, help="decode steps to measure (default 128)")
    ap.add_argument("--prompt-tokens", type=int, default=128,
                    help="synthetic prompt length in tokens (default 128)")
    ap.add_argument("--batch", default="1",
                    help="sequences in flight; a list (1,8,64) measures each (default 1)")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help="length of the measured prefill (default: --prompt-tokens)")
    ap.add_argument("--warmup", type=int, default=8,
                    help="steps to run and discard before measuring (default 8)")
    ap.add_argument("--json", default="", help="write the machine-readable record here")
    _common(ap)
    return ap


def _precision(name):
    try:
        return PRECISIONS[name.lower()]
    except KeyError:
        raise UsageError(f"--precision {name}: bf16, f32 or auto") from None


def _device(name):
    if name == "auto":
        return "cuda:0"
    if not re.fullmatch(r"cuda(:\d+)?", name):
        raise UsageError(f"--device {name}: auto or cuda:N; this engine has no other device")
    return name


def _positive(name, n):
    if n <= 0:
        raise UsageError(f"--{name} {n}: it must be positive")


def _ids(text):
    parts = [p for p in re.split(r"[,\s]+", text.strip()) if p]
    if not parts:
        raise UsageError("--prompt is empty; there is nothing to condition on")
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise UsageError("--prompt holds token ids (integers separated by commas or spaces); "
                         "this engine has no tokenizer") from None


def _open(args, dtype, device, opener):
    """The model of a command: a folder, or (--config with --random) random weights."""
    import tgo_b200
    if args.random is not None or args.config:
        if args.random is None or not args.config:
            raise UsageError("--config and --random SEED go together: a config.json to take the "
                             "sizes from and the seed of the weights")
        if args.model_dir:
            raise UsageError("give a <model-dir> or --config with --random, not both")
        with open(args.config) as f:
            config = json.load(f)
        return tgo_b200.open_random(config, args.random, dtype=dtype, device=device)
    if not args.model_dir:
        raise UsageError("a <model-dir> is needed (or --config cfg.json --random SEED)")
    return (opener or tgo_b200.open)(args.model_dir, dtype=dtype, device=device)


def _stop_ids(text, model):
    if text == "auto":
        return list(getattr(model, "stop_ids", ()))
    if text in ("none", ""):
        return []
    try:
        return [int(p) for p in re.split(r"[,\s]+", text.strip()) if p]
    except ValueError:
        raise UsageError(f"--stop-ids {text}: token ids, auto or none") from None


def cmd_run(argv, out=sys.stdout, err=sys.stderr, opener=None):
    args = run_parser().parse_args(argv)
    dtype, device = _precision(args.precision), _device(args.device)
    _positive("max-tokens", args.max_tokens)
    _positive("context", args.context)
    _positive("page-size", args.page_size)
    if args.max_tokens > args.context:
        raise UsageError(f"--max-tokens {args.max_tokens} is more than the --context "
                         f"{args.context} the cache holds")
    if args.prompt_len < 0 or (args.prompt_len and args.prompt):
        raise UsageError("--prompt-len N stands in place of --prompt and is positive")
    if args.kv_pages < 0:
        raise UsageError(f"--kv-pages {args.kv_pages}: it cannot be negative")
    prompts = [_ids(p) for p in (args.prompt or ([] if args.prompt_len else ["1 2 3 4 5 6 7 8"]))]
    from .sampling.policy import Policy
    policy = Policy(temperature=args.temp, top_k=args.top_k, top_p=args.top_p,
                    repetition_penalty=args.repeat_penalty, seed=args.seed,
                    max_tokens=args.max_tokens)
    model = _open(args, dtype, device, opener)
    try:
        policy.check(model.spec.vocab_size)
    except ValueError as e:
        raise UsageError(str(e)) from None
    if args.prompt_len:
        from .engine.measure import random_prompts
        prompts = random_prompts(model.spec.vocab_size, 1, args.prompt_len, args.seed)
    stop_ids = _stop_ids(args.stop_ids, model)
    print(f"tgo: {model.info['architecture']} {dtype} context={args.context} "
          f"temp={args.temp} seed={args.seed} prompt={' + '.join(str(len(p)) for p in prompts)} "
          f"tokens stop_ids={stop_ids}", file=err)
    if len(prompts) > 1:
        return _run_together(args, model, prompts, policy, stop_ids, out, err)
    prompt = prompts[0]
    if args.kv_pages:
        if args.kv_pages * args.page_size < len(prompt) + 1:
            raise UsageError(f"--kv-pages {args.kv_pages} of {args.page_size} tokens do not hold "
                             f"the prompt")
        args.context = min(args.context, args.kv_pages * args.page_size)
        policy.max_tokens = min(policy.max_tokens, args.context - len(prompt))
    session = model.new_session(context=args.context, page_size=args.page_size, stop_ids=stop_ids)
    t0 = time.perf_counter()
    first = None
    n = 0
    for tok in session.complete(prompt, policy):
        if first is None:
            first = time.perf_counter() - t0
        n += 1
        print(tok, end=" ", file=out, flush=True)
    print(file=out)
    dt = time.perf_counter() - t0
    if n:
        print(f"tgo: {len(prompt)} prompt tokens, {n} generated, first token after "
              f"{first * 1e3:.1f} ms, {n / dt:.2f} tokens/s overall", file=err)
    return 0


def _run_together(args, model, prompts, policy, stop_ids, out, err):
    """Several prompts: continuous batching through the scheduler; one line of ids each."""
    import copy
    need = max(len(p) for p in prompts) + args.max_tokens
    if need > args.context:
        raise UsageError(f"a prompt of {need - args.max_tokens} tokens and --max-tokens "
                         f"{args.max_tokens} exceed the --context {args.context}")
    pool = args.kv_pages * args.page_size if args.kv_pages else None
    policies = []
    for i in range(len(prompts)):           # each request draws from a stream of its own
        pol = copy.copy(policy)
        pol.seed = policy.seed + i
        policies.append(pol)
    t0 = time.perf_counter()
    outs = model.generate(prompts, policies, slots=min(len(prompts), 64), pool_tokens=pool,
                          page_size=args.page_size, stop_ids=stop_ids)
    dt = time.perf_counter() - t0
    for o in outs:
        print(" ".join(str(t) for t in o), file=out)
    n = sum(len(o) for o in outs)
    runner = getattr(model, "last_runner", None)
    print(f"tgo: {len(prompts)} prompts, {sum(len(p) for p in prompts)} prompt tokens, {n} "
          f"generated in {getattr(runner, 'steps', 0)} steps "
          f"({getattr(runner, 'evictions', 0)} evictions), {n / dt:.2f} tokens/s overall", file=err)
    return 0


def cmd_bench(argv, out=sys.stdout, err=sys.stderr, opener=None):
    args = bench_parser().parse_args(argv)
    dtype, device = _precision(args.precision), _device(args.device)
    try:
        batches = [int(b) for b in re.split(r"[,\s]+", str(args.batch).strip()) if b]
    except ValueError:
        raise UsageError(f"--batch {args.batch}: a number or a list like 1,8,64") from None
    if not batches or min(batches) <= 0:
        raise UsageError(f"--batch {args.batch}: it must be positive")
    for name in ("tokens", "prompt_tokens", "context", "page_size"):
        _positive(name.replace("_", "-"), getattr(args, name))
    if args.warmup < 0:
        raise UsageError(f"--warmup {args.warmup}: it cannot be negative")
    if args.prompt_tokens + args.tokens > args.context:
        raise UsageError(f"--prompt-tokens {args.prompt_tokens} plus --tokens {args.tokens} is "
                         f"more than the --context {args.context} the cache holds")
    from .engine.measure import measure_decode, measure_prefill
    model = _open(args, dtype, device, opener)
    pre = measure_prefill(model, args.prefill_tokens or args.prompt_tokens,
                          warmup=min(args.warmup, 3), steps=3, seed=args.seed,
                          page_size=args.page_size)
    decs = [measure_decode(model, b, args.prompt_tokens, args.tokens, warmup=args.warmup,
                           seed=args.seed, page_size=args.page_size) for b in batches]
    dec = decs[0]
    record = {"model": model.info, "conditions": {
        "precision": dtype, "context": args.context, "batch": batches[0],
        "prompt_tokens": args.prompt_tokens, "tokens": args.tokens, "warmup": args.warmup,
        "temp": args.temp, "seed": args.seed, "prompt": "seeded uniform-random token ids",
        "page_size": args.page_size},
        "prefill": pre, "decode": dec}
    if len(decs) > 1:
        record["decode_by_batch"] = {str(b): d for b, d in zip(batches, decs)}
    print(f"model      {model.info['architecture']}  {dtype}  weights "
          f"{model.info['weight_bytes'] / 1e9:.2f} GB", file=out)
    print(f"conditions batch={args.batch} prompt={args.prompt_tokens} tokens={args.tokens} "
          f"warmup={args.warmup} context={args.context}", file=out)
    print(f"prefill    {pre['tokens_per_s']:.1f} tokens/s  ({pre['tokens']} tokens in "
          f"{pre['ms']:.2f} ms)", file=out)
    for b, d in zip(batches, decs):
        print(f"decode     {d['tokens_per_s']:.1f} tokens/s  batch {b}  (p50 {d['p50_ms']:.3f} ms, "
              f"p90 {d['p90_ms']:.3f} ms, p99 {d['p99_ms']:.3f} ms per step)", file=out)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(record, f, indent=1)
    return 0


def cmd_info(argv, out=sys.stdout, err=sys.stderr, opener=None):
    ap = _parser("info")
    ap.add_argument("--precision", default="auto")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--config", default="")
    ap.add_argument("--random", type=int, default=None, metavar="SEED")
    ap.add_argument("model_dir", metavar="<model-dir>", nargs="?", default="")
    args = ap.parse_args(argv)
    model = _open(args, _precision(args.precision), _device(args.device), opener)
    for k, v in model.info.items():
        print(f"{k:24s}{v}", file=out)
    return 0


def cmd_random(argv, out=sys.stdout, err=sys.stderr, opener=None):
    ap = _parser("random")
    ap.add_argument("--config", required=True, help="a config.json to take the sizes from")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--sigma", type=float, default=0.02, help="std of matrices and tables")
    ap.add_argument("--gain-sigma", type=float, default=0.1, help="std of norm gains around 1")
    ap.add_argument("model_dir", metavar="<model-dir>")
    args = ap.parse_args(argv)
    from .weights.random_init import write_random_model
    with open(args.config) as f:
        config = json.load(f)
    write_random_model(args.model_dir, config, args.seed, args.sigma, args.gain_sigma)
    print(f"wrote {os.path.join(args.model_dir, 'model.safetensors')}", file=out)
    return 0


COMMANDS = {"run": cmd_run, "bench": cmd_bench, "info": cmd_info, "random": cmd_random}


def main(argv=None, out=sys.stdout, err=sys.stderr, opener=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(USAGE, file=out)
        return 0 if argv else 2
    cmd = COMMANDS.get(argv[0])
    if cmd is None:
        print(f"tgo: unknown command {argv[0]!r}\n{USAGE}", file=err)
        return 2
    try:
        return cmd(argv[1:], out=out, err=err, opener=opener)
    except UsageError as e:
        print(f"tgo {argv[0]}: {e}", file=err)
        return 2
    except SystemExit as e:       # argparse
        return int(e.code or 0)


if __name__ == "__main__":
    sys.exit(main())
