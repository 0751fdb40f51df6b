"""The schedules that the benchmark measures, with their logits checked against the plain
implementation: steps of more than a thousand rows (the tcgen05 product inside a model),
many requests decoding together through the padded graph buckets, prompts of several
requests in one step, eviction and recomputation when pages run out mid-run, and a cache
whose unheld pages are poisoned."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, run) in tiny.TINIES.items():
        d = tiny.make_model_dir(tmp_path_factory.mktemp(f"sched{name}"), cfg, run["seed"], run["sigma"])
        out[name] = (d, cfg, run)
    return out


# ------------------------------------------------------------------ steps of many rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_more_than_a_thousand_rows(models, dtype):
    """One request of 1200 tokens through Tiny C (head size 128): whole in one step, and as
    one step of 1100 rows followed by portions and single tokens. In bfloat16 every product
    of those steps runs on the tcgen05 kernel (the gated one included) and hands its result
    to the next norm; the logits are the plain implementation's either way."""
    import tgo_b200
    from tgo_b200.kernels import ops
    d, cfg, run = models["C"]
    reqs = tiny.random_requests(cfg["vocab_size"], [1200], seed=31)
    toks = reqs["r0"]
    want, rounded = tiny.plain_logits(d, reqs), tiny.plain_logits_rounded(d, reqs)
    model = tgo_b200.open(d, dtype=dtype)
    cut = [{"step": 0, "entries": [{"id": "r0", "tokens": toks[:1100], "want": list(range(1100))}], "end": []},
           {"step": 1, "entries": [{"id": "r0", "tokens": toks[1100:1160], "want": list(range(60))}], "end": []}]
    for i in range(1160, 1200):
        cut.append({"step": len(cut), "entries": [{"id": "r0", "tokens": [toks[i]], "want": [0]}],
                    "end": ["r0"] if i == 1199 else []})
    for label, trace in (("whole", tiny.trace_whole(reqs)), ("cut", cut)):
        if dtype == "bfloat16":
            ops.gemm_tc_force_tile(0, 0)
        eng = model.new_engine(page_size=run["page_size"], max_tokens=1216, num_slots=1)
        got = tiny.run_trace_engine(eng, trace)
        eng.check_kernels()
        assert len(got) == 1200
        worst, where, tol = tiny.compare(got, want, cfg, dtype, f"many_rows/{label}/{dtype}", rounded)
        assert worst <= tol, f"{label}/{dtype}: error {worst:.3e} at {where}, allowed {tol:.3e}"
    if dtype == "bfloat16":
        assert ops.product_regime(1100) == 2 and ops.gemm_tc_last_plan()[0] in (128, 256)


@pytest.mark.parametrize("family", ["portions", "mixed"])
def test_replay_with_the_tcgen05_product_from_65_rows(models, family, monkeypatch):
    """The replay families of Tiny C in bfloat16 with the tcgen05 product taking every step of
    65 rows or more (it normally starts above 1024): portions of changing size and mixed
    batches then run through it with ragged row counts."""
    import tgo_b200
    from tgo_b200.kernels import ops
    monkeypatch.setattr(ops, "TC_MIN_ROWS", 65)
    d, cfg, run = models["C"]
    reqs = tiny.random_requests(cfg["vocab_size"], [3, 150, 66, 200, 31, 290], seed=12)
    want, rounded = tiny.plain_logits(d, reqs), tiny.plain_logits_rounded(d, reqs)
    model = tgo_b200.open(d, dtype="bfloat16")
    trace = tiny.trace_portions(reqs, sizes=(70, 2, 130, 65, 3, 200)) if family == "portions" \
        else tiny.trace_mixed(reqs, seed=3, tail=8)
    eng = model.new_engine(page_size=run["page_size"], max_tokens=tiny.max_tokens_of(trace), num_slots=4)
    got = tiny.run_trace_engine(eng, trace)
    eng.check_kernels()
    worst, where, tol = tiny.compare(got, want, cfg, "bfloat16", f"tc_from_65/{family}", rounded)
    assert worst <= tol, f"{family}: error {worst:.3e} at {where}, allowed {tol:.3e}"


# ------------------------------------------- the persistent decode products inside a model


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_through_the_persistent_products(tmp_path_factory, dtype):
    """Tiny D (hidden, q width and intermediate size 2048, head size 128): 1, 3 and 8 requests
    decoding together. In bfloat16 every product of those steps, the vocabulary product
    included, takes the persistent form of the weight-streaming kernel, the two norms of a
    layer are made inside the q/k/v and gate/up products, and the attention kernel norms,
    rotates and stores the step's own q, k and v. The logits are the plain implementation's."""
    import tgo_b200
    from tgo_b200.kernels import ops
    cfg, run = tiny.TINY_D, tiny.TINY_D_RUN
    d = tiny.make_model_dir(tmp_path_factory.mktemp("schedD"), cfg, run["seed"], run["sigma"])
    if dtype == "bfloat16":
        for M in (1, 3, 8):
            assert ops.folds_norm(M, 2048 + 2 * 512, 2048) and ops.folds_norm(M, 4096, 2048)
            assert ops.folds_norm(M, 512, 2048)
    reqs = tiny.random_requests(cfg["vocab_size"], [40, 23, 61, 17, 33, 50, 29, 45], seed=41)
    want, rounded = tiny.plain_logits(d, reqs), tiny.plain_logits_rounded(d, reqs)
    model = tgo_b200.open(d, dtype=dtype)
    for live in (1, 3, 8):
        some = {r: reqs[r] for r in list(reqs)[:live]}
        trace = crowd_trace(some, 12)
        eng = model.new_engine(page_size=run["page_size"], max_tokens=tiny.max_tokens_of(trace),
                               num_slots=live)
        launches = ops.LAUNCHES[0]
        got = tiny.run_trace_engine(eng, trace)
        eng.check_kernels()
        sub = {r: want[r] for r in some}
        assert {k[0] for k in got} == set(some) and len(got) == sum(len(t) for t in some.values())
        worst, where, tol = tiny.compare(got, sub, cfg, dtype, f"persistent_products/{live}/{dtype}",
                                         {r: rounded[r] for r in some})
        assert worst <= tol, f"{live} live/{dtype}: error {worst:.3e} at {where}, allowed {tol:.3e}"
        assert ops.LAUNCHES[0] > launches


# ---------------------------------------------------------- many requests live together


def crowd_trace(requests, decode_steps):
    """All prompts in one step (several requests, more than 1024 rows together), then the
    last `decode_steps` tokens of every request one per step, all requests in one batch; in
    two of those steps a few requests sit out and catch up later."""
    ids = list(requests)
    trace = [{"step": 0, "entries": [{"id": r, "tokens": requests[r][:-decode_steps],
                                      "want": list(range(len(requests[r]) - decode_steps))} for r in ids],
              "end": []}]
    at = {r: len(requests[r]) - decode_steps for r in ids}
    step = 1
    while any(at[r] < len(requests[r]) for r in ids):
        sit_out = set(ids[1::4]) if step in (3, 5) else set()
        entries, end = [], []
        for r in ids:
            if at[r] >= len(requests[r]) or r in sit_out:
                continue
            entries.append({"id": r, "tokens": [requests[r][at[r]]], "want": [0]})
            at[r] += 1
            if at[r] == len(requests[r]):
                end.append(r)
        trace.append({"step": step, "entries": entries, "end": end})
        step += 1
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live,prompt", [(9, 130), (20, 60), (64, 20)])
@pytest.mark.parametrize("name", ["B", "C"])
def test_many_requests_decode_together(models, name, live, prompt, dtype):
    """9, 20 and 64 live requests: their prompts run as one step of more than 1024 rows, then
    they decode together through the graph buckets of 16, 24 and 64 rows (padded rows
    beside live ones; the library's product range; the split plans of the decode attention
    at these batch sizes), some requests sitting steps out so that smaller buckets and
    other paddings come too."""
    import tgo_b200
    d, cfg, run = models[name]
    decode_steps = 8
    rng = np.random.default_rng(live)
    lengths = [prompt + decode_steps + int(rng.integers(0, 7)) for _ in range(live)]
    reqs = tiny.random_requests(cfg["vocab_size"], lengths, seed=live)
    assert sum(n - decode_steps for n in lengths) > 1024
    want, rounded = tiny.plain_logits(d, reqs), tiny.plain_logits_rounded(d, reqs)
    model = tgo_b200.open(d, dtype=dtype)
    trace = crowd_trace(reqs, decode_steps)
    eng = model.new_engine(page_size=run["page_size"], max_tokens=tiny.max_tokens_of(trace),
                           num_slots=live)
    got = tiny.run_trace_engine(eng, trace)
    eng.check_kernels()
    assert len(got) == sum(lengths)
    worst, where, tol = tiny.compare(got, want, cfg, dtype, f"crowd/{name}/{live}/{dtype}", rounded)
    assert worst <= tol, f"{name}/{live}/{dtype}: error {worst:.3e} at {where}, allowed {tol:.3e}"
    buckets = sorted({k[0] for k in eng._graphs})
    full = next(b for b in eng.BUCKETS if b >= live)
    assert full in buckets and len(buckets) >= 2, buckets          # padded, and more than one size
    assert all(p.free_count == p.num_pages for p in eng.cache.pools)


# ------------------------------------------------------ pages run out in the middle of a run


@pytest.mark.parametrize("name", ["A", "B"])
def test_pages_run_out_mid_run_evict_and_recompute(tmp_path, name):
    """Three requests are admitted with a small reserve into a pool that cannot hold all three
    once they have grown: in the middle of the run a step cannot get its pages, the latest
    arrival is evicted, waits, and is computed again from its prompt and what it had
    produced. Every request still gets exactly the plain implementation's greedy tokens."""
    import tgo_b200
    from tgo_b200.sampling.policy import Policy
    cfg, run = tiny.TINIES[name]
    d = tiny.make_model_dir(tmp_path / name, cfg, seed=21, sigma=0.25)
    pc, pw = plain.load_model_dir(d)
    ps = run["page_size"]
    prompts = list(tiny.random_requests(cfg["vocab_size"], [20, 24, 28], seed=4).values())
    new = 40
    want = [plain.greedy_generate(pc, pw, p, new) for p in prompts]
    model = tgo_b200.open(d, dtype="float32")
    admitted = sum(-(-(len(p) + ps) // ps) for p in prompts)      # prompt + reserve, in pages
    grown = sum(-(-(len(p) + new) // ps) for p in prompts)
    pool_pages = admitted + 1                     # all three get in; they cannot all grow
    assert pool_pages < grown
    got = model.generate(prompts, Policy(max_tokens=new), slots=3, chunk=16, reserve=ps,
                         pool_tokens=pool_pages * ps, page_size=ps)
    runner = model.last_runner
    assert runner.evictions >= 1, "the pool was large enough after all: nothing was evicted"
    assert got == want
    engine = runner.sched.engine
    assert all(p.free_count == p.num_pages for p in engine.cache.pools)
    engine.cache.check_invariants()


# --------------------------------------------------------------- unheld pages are poisoned


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unheld_pages_are_unreachable(models, name, dtype):
    """The mixed replay (up to four live requests, so few pages that they are used again)
    with NaN written into every page that no live request holds, before the first step and
    after every step: pages never handed out, pages of finished requests, pages a window has
    passed. Reads are bounded by a request's length, so the logits are finite and equal,
    bit for bit, those of the same replay with an untouched cache. The run also shows that
    pages were in fact handed to a second request."""
    import tgo_b200
    d, cfg, run = models[name]
    lengths = {"A": [5, 17, 33, 70, 100, 64], "B": [1, 9, 40, 70, 129, 48], "C": [3, 150, 66, 200, 31, 290]}[name]
    reqs = tiny.random_requests(cfg["vocab_size"], lengths, seed=10 + run["seed"])
    trace = tiny.trace_mixed(reqs)
    model = tgo_b200.open(d, dtype=dtype)
    results = []
    for poison in (False, True):
        eng = model.new_engine(page_size=run["page_size"], max_tokens=tiny.max_tokens_of(trace),
                               num_slots=4)
        owners = [dict() for _ in eng.cache.groups]
        results.append(tiny.run_trace_engine(eng, trace, poison=poison, owners=owners))
        shared = [p for g in owners for p, who in g.items() if len(who) > 1]
        assert shared, "no page was handed to a second request: the pool is too large to show reuse"
    clean, poisoned = results
    for k, row in poisoned.items():
        assert np.isfinite(row).all(), f"{name}/{dtype}: a poisoned page was read at {k}"
        assert np.array_equal(row, clean[k]), f"{name}/{dtype}: logits changed at {k}"
