"""Generation on the GPU through the entry points a user has: the library, the scheduler and
the command line; long decoding; the first tokens of a sequence; seeded sampling."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lively(tmp_path_factory):
    """Tiny models with weights large enough that the output is not one token repeated."""
    out = {}
    for name, (cfg, run) in tiny.TINIES.items():
        d = tiny.make_model_dir(tmp_path_factory.mktemp(f"lively{name}"), cfg, seed=21, sigma=0.25)
        out[name] = (d, cfg, run) + plain.load_model_dir(d)
    return out


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(lively, name):
    import tgo_b200
    from tgo_b200.sampling.policy import Policy
    d, cfg, run, pc, pw = lively[name]
    prompts = list(tiny.random_requests(cfg["vocab_size"], [5, 17, 33, 1], seed=8).values())
    want = [plain.greedy_generate(pc, pw, p, 8) for p in prompts]
    assert len({t for o in want for t in o}) > 4
    model = tgo_b200.open(d, dtype="float32")
    assert model.generate(prompts, Policy(max_tokens=8), slots=3, chunk=16,
                          page_size=run["page_size"]) == want
    # so few pages that a request waits for another's to come back
    assert model.generate(prompts, Policy(max_tokens=8), slots=4, chunk=7, pool_tokens=64,
                          page_size=run["page_size"]) == want
    # bfloat16: every token it picks is, in the plain logits, within rounding of the best
    got = tgo_b200.open(d, dtype="bfloat16").generate(prompts, Policy(max_tokens=8), slots=4,
                                                      page_size=run["page_size"])
    for p, o in zip(prompts, got):
        seq = list(p)
        for tok in o:
            logits = plain.forward(pc, pw, seq)[-1]
            slack = 2 * tiny.tolerance(cfg, "bfloat16", logits, plain.forward_rounded(pc, pw, seq)[-1])
            assert logits.max() - logits[tok] <= slack
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(lively, dtype):
    """Three prompt tokens, then 200 tokens one at a time (through the captured graph), every
    position's logits against the whole sequence run plainly; and sequences that start with
    single-token steps from an empty cache."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, run, pc, pw = lively["B"]
    toks = tiny.random_requests(cfg["vocab_size"], [203], seed=12)["r0"]
    want = plain.forward(pc, pw, toks)
    model = tgo_b200.open(d, dtype=dtype)
    eng = model.new_engine(page_size=run["page_size"], max_tokens=256, num_slots=2)
    eng.admit("long")
    rows = [eng.step([StepEntry("long", toks[:3], [0, 1, 2])]).float().cpu().numpy()]
    for t in toks[3:]:
        rows.append(eng.step([StepEntry("long", [t], [0])]).float().cpu().numpy())
    got = np.concatenate(rows)
    tol = tiny.tolerance(cfg, dtype, want, plain.forward_rounded(pc, pw, toks))
    tiny.note(f"long_decoding/{dtype}", float(np.abs(got - want).max()), tol)
    assert np.abs(got - want).max() <= tol
    eng.finish("long")
    eng.admit("first")
    rows = [eng.step([StepEntry("first", [t], [0])]).float().cpu().numpy() for t in toks[:5]]
    assert np.abs(np.concatenate(rows) - want[:5]).max() <= tol


def test_seeded_temperature_sampling_follows_the_plain_walk(lively):
    import tgo_b200
    from tgo_b200.sampling.policy import DrawStream, Policy
    d, cfg, run, pc, pw = lively["B"]
    model = tgo_b200.open(d, dtype="float32")
    prompts = list(tiny.random_requests(cfg["vocab_size"], [1, 9, 40, 70], seed=9).values())
    pol = Policy(temperature=0.8, seed=5, max_tokens=12)
    got = model.generate(prompts, pol, slots=4, chunk=16, page_size=8)
    assert got == model.generate(prompts, pol, slots=2, chunk=5, page_size=8)
    for p, o in zip(prompts, got):
        draws, seq = DrawStream(5), list(p)
        for tok in o:
            logits = plain.forward(pc, pw, seq)[-1].astype(np.float32)
            ids, w, total = plain.policy_distribution(logits, temperature=0.8)
            u = draws.next()
            want = plain.walk(ids, w, total, u)
            if tok != want:                 # only where rounding puts the draw on a boundary
                cdf = np.cumsum(np.asarray(w, np.float64))
                assert abs(cdf[min(ids.index(tok), ids.index(want))] - u * cdf[-1]) < 1e-4 * cdf[-1]
            seq.append(tok)
    top = model.generate(prompts[:2], Policy(temperature=1.5, top_k=3, top_p=0.9, seed=1, max_tokens=6),
                         slots=2, page_size=8)
    for p, o in zip(prompts[:2], top):
        seq = list(p)
        for tok in o:
            logits = plain.forward(pc, pw, seq)[-1].astype(np.float32)
            ids, _, _ = plain.policy_distribution(logits, temperature=1.5, top_k=3, top_p=0.9)
            assert tok in ids
            seq.append(tok)


def test_logprobs_of_generated_tokens(lively):
    """Policy.logprobs through generate and a session on the device: the same tokens with
    and without the report, each drawn token's share of its kept set against the plain
    distribution, the alternatives descending and summing to one over the kept set, and
    ln 1 at temperature 0 (specs/030-logprobs.md section 6 of the reference)."""
    import tgo_b200
    from tgo_b200.sampling.policy import Policy
    d, cfg, run, pc, pw = lively["B"]
    model = tgo_b200.open(d, dtype="float32")
    prompts = list(tiny.random_requests(cfg["vocab_size"], [9, 40], seed=9).values())
    quiet = Policy(temperature=0.8, top_k=8, seed=7, max_tokens=6)
    asked = Policy(temperature=0.8, top_k=8, seed=7, max_tokens=6, logprobs=True, top_logprobs=8)
    got = model.generate(prompts, [asked, quiet], slots=2, chunk=16, page_size=8)
    first, second = model.last_requests
    assert got[0] == model.generate(prompts[:1], quiet, slots=1, page_size=8)[0]
    assert second.logprobs == [] and [tp.id for tp in first.logprobs] == got[0]
    seq = list(prompts[0])
    for tok, tp in zip(got[0], first.logprobs):
        logits = plain.forward(pc, pw, seq)[-1].astype(np.float32)
        ids, w, total = plain.policy_distribution(logits, temperature=0.8, top_k=8)
        lp, _ = plain.token_logprobs(ids, w, total, tok, 0, cfg["vocab_size"])
        assert tok in ids and abs(tp.logprob - lp) < 1e-3           # the engine's float32 logits
        lps = [a.logprob for a in tp.top]
        assert len(lps) == 8 and lps == sorted(lps, reverse=True) and sorted(a.id for a in tp.top) == ids
        assert abs(sum(np.exp(v) for v in lps) - 1) < 1e-5
        seq.append(tok)
    s = model.new_session(context=64, page_size=8)
    for tok in s.complete(prompts[1], Policy(max_tokens=3, logprobs=True, top_logprobs=3)):
        (tp,) = s.logprobs()
        assert (tp.id, tp.logprob, tp.top[0].id) == (tok, 0.0, tok)
        assert [a.logprob for a in tp.top[1:]] == [-np.inf, -np.inf]


def test_scheduler_entry_points(lively):
    """admit / step / feed / finish by hand, as the reference's callers use them."""
    import tgo_b200
    from tgo_b200.kernels import ops
    import torch
    d, cfg, run, pc, pw = lively["A"]
    model = tgo_b200.open(d, dtype="float32")
    sched = model.new_scheduler(slots=2, chunk=8, reserve=16, pool_tokens=128, page_size=16)
    prompt = tiny.random_requests(256, [19], seed=3)["r0"]
    slot = sched.admit(prompt)
    produced = []
    for _ in range(40):
        res = sched.step()
        for p in res.produced:
            if p.sampleable():
                out = torch.empty(1, dtype=torch.int32, device="cuda:0")
                ops.argmax(res.logits[p.row:p.row + 1], out)
                produced.append(int(out))
                if len(produced) == 6:
                    break
                sched.feed(p.slot, produced[-1])
        if len(produced) == 6:
            break
    assert produced == plain.greedy_generate(pc, pw, prompt, 6)
    sched.finish(slot)
    assert sched.engine.cache.pools[0].free_count == sched.engine.cache.pools[0].num_pages


def test_command_line(lively, tmp_path):
    d, cfg, run, pc, pw = lively["A"]
    tgo = os.path.join(tiny.ROOT, "bin", "tgo")
    r = subprocess.run([sys.executable, tgo, "run", "--prompt", "5 17 3 200", "--max-tokens", "6",
                        "--precision", "f32", "--context", "64", d], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == plain.greedy_generate(pc, pw, [5, 17, 3, 200], 6)
    assert "tokens/s" in r.stderr
    out = tmp_path / "rec.json"
    r = subprocess.run([sys.executable, tgo, "bench", "--tokens", "8", "--prompt-tokens", "16",
                        "--warmup", "2", "--context", "64", "--json", str(out), d],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rec = json.loads(out.read_text())
    assert rec["decode"]["tokens_per_s"] > 0 and rec["prefill"]["tokens"] == 16
    assert "decode" in r.stdout and "prefill" in r.stdout
    r = subprocess.run([sys.executable, tgo, "info", d], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "Qwen3ForCausalLM" in r.stdout


def test_one_seed_gives_one_model_on_the_cpu_and_on_the_gpu():
    """The random-weights mode makes a model folder on the CPU and, for large models, makes
    the tensors on the device: one seed gives the same bits either way."""
    import torch
    from tgo_b200.weights.binder import WeightSpec
    from tgo_b200.weights.random_init import random_tensor
    for spec in (WeightSpec("w", (300, 129)), WeightSpec("g", (1000,), "gain")):
        for dtype in (torch.float32, torch.bfloat16):
            a = random_tensor(spec, 11, 0.02, 0.1, dtype, "cpu")
            b = random_tensor(spec, 11, 0.02, 0.1, dtype, "cuda:0")
            assert torch.equal(a, b.cpu())
