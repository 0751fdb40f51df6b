"""Replay on the GPU: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with page reuse, in float32 and in bfloat16, through
bin/trace_run (a subprocess, as a user runs it) and compared with the plain implementation."""
import numpy as np
import pytest

import tiny

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70, 100, 64], "B": [1, 9, 40, 70, 129, 48], "C": [3, 150, 66, 200, 31, 290]}
FAMILIES = {"whole": tiny.trace_whole, "tail": tiny.trace_tail, "portions": tiny.trace_portions,
            "mixed": tiny.trace_mixed}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, run) in tiny.TINIES.items():
        d = tiny.make_model_dir(tmp_path_factory.mktemp(f"tiny{name}"), cfg, run["seed"],
                                run["sigma"])
        reqs = tiny.random_requests(cfg["vocab_size"], LENGTHS[name], seed=10 + run["seed"])
        out[name] = (d, cfg, run, reqs, tiny.plain_logits(d, reqs), tiny.plain_logits_rounded(d, reqs))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_matches_plain(models, tmp_path, name, family, dtype):
    d, cfg, run, reqs, want, rounded = models[name]
    trace = FAMILIES[family](reqs)
    got = tiny.run_trace_program(d, dtype, trace, tmp_path / "out", cfg["vocab_size"],
                                 extra=["--page-size", str(run["page_size"])])
    assert len(got) == sum(len(t) for t in reqs.values())
    worst, where, tol = tiny.compare(got, want, cfg, dtype, f"replay/{name}/{family}/{dtype}", rounded)
    assert worst <= tol, f"{name}/{family}/{dtype}: error {worst:.3e} at {where}, allowed {tol:.3e}"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_float32_cuts_agree_bit_for_bit(models, name):
    """In float32 every sum's order depends on the position alone, so the four ways of
    cutting give the same bits, not just close values."""
    import tgo_b200
    d, cfg, run, reqs, _, _ = models[name]
    model = tgo_b200.open(d, dtype="float32")
    results = {}
    for fam, make in FAMILIES.items():
        trace = make(reqs)
        eng = model.new_engine(page_size=run["page_size"], max_tokens=tiny.max_tokens_of(trace),
                               num_slots=4)
        results[fam] = tiny.run_trace_engine(eng, trace)
    base = results["whole"]
    for fam, got in results.items():
        for k, row in got.items():
            assert np.array_equal(row, base[k]), f"{name}: {fam} differs from whole at {k}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_prompt_portions_through_graphs_give_the_same_bits(models, name, dtype):
    """Equal-sized portions of a long prompt: the second is captured as a CUDA graph and the
    later ones replay it. Same kernels, same order, so the logits equal those of an engine
    that never captures, bit for bit; and a portion of another request between the replays
    goes through the same graph with its own positions and pages."""
    import torch
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, run, reqs, _, _ = models[name]
    model = tgo_b200.open(d, dtype=dtype)
    rng = np.random.default_rng(5)
    long_a = rng.integers(0, cfg["vocab_size"], 200).tolist()
    long_b = rng.integers(0, cfg["vocab_size"], 120).tolist()
    size = 40
    steps = []
    for i in range(0, 200, size):
        steps.append(("a", long_a[i:i + size]))
        if i // size in (1, 2, 3):
            j = (i // size - 1) * size
            steps.append(("b", long_b[j:j + size]))
    got = {}
    for graphs in (False, True):
        eng = model.new_engine(page_size=run["page_size"], max_tokens=512, num_slots=2, graphs=graphs)
        eng.PORTION_GRAPH_MIN_TOKENS = 32
        eng.admit("a")
        eng.admit("b")
        outs = []
        for rid, toks in steps:
            outs.append(eng.step([StepEntry(rid, toks, [0, size - 1])]).clone())
        torch.cuda.synchronize()
        got[graphs] = outs
        if graphs:
            assert eng._portion_graphs, "no portion was captured"
    for a, b in zip(got[False], got[True]):
        assert torch.equal(a, b)


def test_more_portion_shapes_than_graphs_are_kept(models):
    """Five portion shapes in turn, again and again, with room for four captured graphs: the
    least recently used graph goes and its shape starts over, and whatever is replayed,
    captured or run directly, the logits are those of an engine that never captures."""
    import torch
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, run, _, _, _ = models["B"]
    model = tgo_b200.open(d, dtype="bfloat16")
    rng = np.random.default_rng(9)
    sizes = [33, 34, 35, 36, 37]
    rounds = 4
    toks = rng.integers(0, cfg["vocab_size"], sum(sizes) * rounds).tolist()
    got = {}
    for graphs in (False, True):
        eng = model.new_engine(page_size=run["page_size"], max_tokens=1024, num_slots=1, graphs=graphs)
        eng.PORTION_GRAPH_MIN_TOKENS = 32
        eng.admit("a")
        outs, at = [], 0
        for _ in range(rounds):
            for n in sizes:
                outs.append(eng.step([StepEntry("a", toks[at:at + n], [n - 1])]).clone())
                at += n
        torch.cuda.synchronize()
        got[graphs] = outs
        if graphs:
            assert 1 <= len(eng._portion_graphs) <= eng.PORTION_GRAPHS_KEPT
    for a, b in zip(got[False], got[True]):
        assert torch.equal(a, b)
