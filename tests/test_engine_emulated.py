"""The engine's host side without a GPU: batch building, block tables, page reuse, windows,
the scheduler's loop and sampling order, with torch stand-ins for the kernels
(tests/emulated_kernels.py). Compared with the plain implementation, which shares no code
with either."""
import numpy as np
import pytest
import torch

import emulated_kernels
import plain_qwen3 as plain
import tiny


@pytest.fixture()
def emulated(monkeypatch):
    emulated_kernels.install(monkeypatch)


def cpu_model(model_dir, cfg, dtype=torch.float32):
    from tgo_b200.api import LoadedModel
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    from tgo_b200.weights.binder import load_weights
    from tgo_b200.weights.safetensors import SafetensorsRepo
    model = Model(model_spec_from_config(cfg), dtype, "cpu")
    model.bind(load_weights(model.weight_specs(), SafetensorsRepo(model_dir), dtype, "cpu",
                            model.tied_alias()))
    return LoadedModel(model, cfg, model_dir)


@pytest.mark.parametrize("name", ["A", "B"])
def test_every_cutting_matches_plain(emulated, tmp_path, name):
    cfg, run = tiny.TINIES[name]
    d = tiny.make_model_dir(tmp_path / name, cfg, run["seed"], run["sigma"])
    reqs = tiny.random_requests(cfg["vocab_size"], [5, 33, 70, 41], seed=2)
    want = tiny.plain_logits(d, reqs)
    loaded = cpu_model(d, cfg)
    base = None
    for fam in (tiny.trace_whole, tiny.trace_tail, tiny.trace_portions, tiny.trace_mixed):
        trace = fam(reqs)
        eng = loaded.new_engine(page_size=run["page_size"], max_tokens=tiny.max_tokens_of(trace),
                                num_slots=4)
        got = tiny.run_trace_engine(eng, trace)
        worst, where, tol = tiny.compare(got, want, cfg, "float32")
        assert worst <= tol, (fam.__name__, worst, where)
        assert all(p.free_count == p.num_pages for p in eng.cache.pools)
        base = base or got
        assert set(got) == set(base)


def test_step_refuses_bad_batches(emulated, tmp_path):
    from tgo_b200.engine.step import StepEntry
    cfg, run = tiny.TINIES["A"]
    d = tiny.make_model_dir(tmp_path / "a", cfg, run["seed"], run["sigma"])
    eng = cpu_model(d, cfg).new_engine(page_size=16, max_tokens=64, num_slots=2)
    eng.admit("a")
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.step([StepEntry("a", [256], [0])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    with pytest.raises(KeyError, match="not admitted"):
        eng.step([StepEntry("b", [1], [0])])
    with pytest.raises(ValueError, match="no tokens"):
        eng.step([StepEntry("a", [], [])])
    with pytest.raises(ValueError, match="place 3"):
        eng.step([StepEntry("a", [1, 2], [3])])
    with pytest.raises(ValueError, match="empty batch"):
        eng.step([])
    assert eng.length("a") == 0                       # nothing of the refused steps stuck
    from tgo_b200.cache.pages import PagesExhausted
    with pytest.raises(PagesExhausted):
        eng.step([StepEntry("a", list(range(65)), [])])
    assert eng.length("a") == 0 and eng.cache.pools[0].free_count == 4
    logits = eng.step([StepEntry("a", [1, 2, 3], [])])
    assert logits.shape == (0, 256) and eng.length("a") == 3


def test_layer_run_twice_and_borrowed_cache(emulated, tmp_path):
    """The run order is data: a layer named twice shares weights and owns two caches; a call
    may read an earlier call's cache instead of writing its own."""
    from tgo_b200.config.spec import LayerCall
    from tgo_b200.engine.model import Model
    from tgo_b200.engine.step import Engine, StepEntry
    from tgo_b200.registry import model_spec_from_config
    from tgo_b200.weights.binder import load_weights
    from tgo_b200.weights.safetensors import SafetensorsRepo
    cfg, run = tiny.TINIES["A"]
    d = tiny.make_model_dir(tmp_path / "a", cfg, run["seed"], 0.2)
    spec = model_spec_from_config(cfg)
    spec.run_order = [LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache_from=1)]
    model = Model(spec, torch.float32, "cpu")
    model.bind(load_weights(model.weight_specs(), SafetensorsRepo(d), torch.float32, "cpu",
                            model.tied_alias()))
    assert [len(g.calls) for g in model.groups] == [3]          # calls 0, 1, 2 own a cache
    pc, pw = plain.load_model_dir(d)
    toks = tiny.random_requests(256, [23], seed=5)["r0"]

    want = tiny.repeated_layers_reference(pc, pw, toks)
    eng = Engine(model, page_size=8, max_tokens=64, num_slots=1)
    eng.admit("x")
    got = torch.cat([eng.step([StepEntry("x", toks[:9], list(range(9)))]),
                     eng.step([StepEntry("x", toks[9:], list(range(14)))])]).numpy()
    assert np.abs(got - want).max() < 1e-4 * max(1, np.abs(want).max())


def test_generate_greedy_and_seeded_sampling(emulated, tmp_path):
    from tgo_b200.sampling.policy import DrawStream, Policy
    cfg, run = tiny.TINIES["B"]
    d = tiny.make_model_dir(tmp_path / "b", cfg, seed=7, sigma=0.25)
    loaded = cpu_model(d, cfg)
    pc, pw = plain.load_model_dir(d)
    prompts = list(tiny.random_requests(384, [1, 9, 40], seed=4).values())
    out = loaded.generate(prompts, Policy(max_tokens=6), slots=2, chunk=16, page_size=8)
    for p, o in zip(prompts, out):
        assert o == plain.greedy_generate(pc, pw, p, 6)
    assert len({tuple(o) for o in out}) > 1 and len(set(out[2])) > 1     # not a degenerate model
    # temperature 0.8, seeded: the same draws walk the plain distribution to the same tokens
    pol = Policy(temperature=0.8, seed=11, max_tokens=5)
    got = loaded.generate(prompts[:2], pol, slots=2, chunk=16, page_size=8)
    again = loaded.generate(prompts[:2], pol, slots=1, chunk=5, page_size=8)
    assert got == again                                   # batching does not change the stream
    for p, o in zip(prompts[:2], got):
        draws, seq = DrawStream(11), list(p)
        for tok in o:
            logits = plain.forward(pc, pw, seq)[-1].astype(np.float32)
            ids, w, total = plain.policy_distribution(logits, temperature=0.8)
            assert tok == plain.walk(ids, w, total, draws.next())
            seq.append(tok)


def test_logprobs_through_generate_and_session(emulated, tmp_path):
    """Policy.logprobs: one TokenProb per generated token, of the distribution after the
    policy; the tokens are the same with and without the report (logprobs_test.go:62-183)."""
    from tgo_b200.sampling.policy import DrawStream, Policy
    cfg, run = tiny.TINIES["B"]
    d = tiny.make_model_dir(tmp_path / "b", cfg, seed=7, sigma=0.25)
    loaded = cpu_model(d, cfg)
    pc, pw = plain.load_model_dir(d)
    prompts = list(tiny.random_requests(384, [9, 40], seed=4).values())
    quiet = Policy(temperature=0.8, top_k=8, seed=7, max_tokens=4)
    asked = Policy(temperature=0.8, top_k=8, seed=7, max_tokens=4, logprobs=True, top_logprobs=8)
    out = loaded.generate(prompts, [asked, quiet], slots=2, chunk=16, page_size=8)
    first, second = loaded.last_requests
    assert out[0] == loaded.generate(prompts[:1], quiet, slots=1, page_size=8)[0]
    assert second.logprobs == [] and len(first.logprobs) == 4
    draws, seq = DrawStream(7), list(prompts[0])
    for tok, tp in zip(out[0], first.logprobs):
        logits = plain.forward(pc, pw, seq)[-1].astype(np.float32)
        ids, w, total = plain.policy_distribution(logits, temperature=0.8, top_k=8)
        assert tok == plain.walk(ids, w, total, draws.next()) == tp.id
        lp, top = plain.token_logprobs(ids, w, total, tok, 8, 384)
        assert abs(tp.logprob - lp) < 1e-5 and np.isfinite(tp.logprob)
        assert [a.id for a in tp.top] == [i for i, _ in top] and not tp.top[0].top
        assert abs(sum(np.exp(a.logprob) for a in tp.top) - 1) < 1e-5
        seq.append(tok)
    # greedy through a session: ln 1 at the argmax, -inf for every alternative after it
    s = loaded.new_session(context=64, page_size=8)
    assert s.logprobs() == []
    seen = 0
    for tok in s.complete(prompts[0], Policy(max_tokens=3, logprobs=True, top_logprobs=2)):
        (tp,) = s.logprobs()
        assert tp.id == tok and tp.logprob == 0 and tp.top[0].id == tok
        assert tp.top[1].logprob == -np.inf
        seen += 1
    assert seen == 3
    assert list(s.complete(prompts[0], Policy(max_tokens=2))) and s.logprobs() == []


def test_session_and_context_limits(emulated, tmp_path):
    from tgo_b200.engine.session import ContextExhausted
    from tgo_b200.sampling.policy import Policy
    cfg, run = tiny.TINIES["A"]
    d = tiny.make_model_dir(tmp_path / "a", cfg, run["seed"], 0.2)
    loaded = cpu_model(d, cfg)
    pc, pw = plain.load_model_dir(d)
    s = loaded.new_session(context=48, page_size=16, chunk=7)
    prompt = tiny.random_requests(256, [20], seed=1)["r0"]
    assert list(s.complete(prompt, Policy(max_tokens=5))) == plain.greedy_generate(pc, pw, prompt, 5)
    assert s.usage == {"prompt_tokens": 20, "completion_tokens": 5}
    assert list(s.complete(prompt[:3], Policy(max_tokens=2))) == plain.greedy_generate(pc, pw, prompt[:3], 2)
    with pytest.raises(ContextExhausted):
        list(s.complete(list(range(48))))
    with pytest.raises(ContextExhausted):
        list(s.complete(prompt, Policy(max_tokens=40)))
    with pytest.raises(ValueError, match="empty"):
        list(s.complete([]))
    assert s.engine.cache.pools[0].free_count == 3
    stop = plain.greedy_generate(pc, pw, prompt, 3)[2]
    s2 = loaded.new_session(context=48, stop_ids=[stop])
    assert len(list(s2.complete(prompt, Policy(max_tokens=5)))) <= 2


# ----------------------------------------------- a toy architecture defined here, on the CPU


class CountingMixer:
    """A mixer with fixed-size state and a one-plane paged cache of its own row shape, written
    with torch: state s <- s + sum of the step's inputs per request; it stores each token's
    input row in its cache plane and returns x + (mean of all cached rows so far) + s. It can
    be told to fail after it has advanced its state."""
    fail_next = False

    def __init__(self, spec, hidden, prefix, device=None):
        self.hidden = hidden

    def weight_specs(self):
        return []

    def bind(self, weights):
        pass

    def cache_need(self):
        from tgo_b200.parts.base import CacheNeed
        return CacheNeed("full", None, 1, (self.hidden,))

    def state_need(self):
        from tgo_b200.parts.base import StateNeed
        return StateNeed((self.hidden,))

    def forward(self, x, ctx, cache):
        plane = cache.planes[0]                        # [pages, page_size, hidden]
        rows = plane.view(-1, self.hidden)
        out = torch.empty_like(x)
        base = 0
        for b, n in enumerate(ctx.extents):
            slot = int(ctx.state_slots[b])
            first = int(ctx.context_lens[b]) - n
            for t in range(n):
                rows[int(cache.slots[base + t])] = x[base + t]
                cache.state[slot] += x[base + t].float()
                table = cache.block_tables[b]
                held = torch.stack([plane[int(table[p // cache.page_size]), p % cache.page_size]
                                    for p in range(first + t + 1)])
                out[base + t] = x[base + t] + held.float().mean(0) + cache.state[slot]
            base += n
        if CountingMixer.fail_next:
            CountingMixer.fail_next = False
            raise RuntimeError("the mixer gave up after it had advanced its state")
        return out


def counting_spec(raw):
    from tgo_b200.config.spec import (FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec,
                                      NormSpec)
    from tgo_b200.config.qwen3 import BLOCK_TENSORS, FEED_FORWARD_TENSORS
    norm = NormSpec("rmsnorm", 1e-5)
    layer = LayerSpec("prenorm_residual", "l0.", MixerSpec("test_counting"),
                      FeedForwardSpec("swiglu", raw["inner"], tensors=FEED_FORWARD_TENSORS), norm,
                      BLOCK_TENSORS)
    return ModelSpec("CountingToy", raw["width"], raw["vocab"], [layer], [LayerCall(0)], norm,
                     "embed.weight", "norm.weight", None, source=dict(raw))


@pytest.fixture()
def counting_registered():
    from tgo_b200.registry import ARCHITECTURES, MIXERS
    ARCHITECTURES.register("CountingToy", counting_spec, replace=True)
    MIXERS.register("test_counting", CountingMixer, replace=True)
    yield
    ARCHITECTURES.unregister("CountingToy")
    MIXERS.unregister("test_counting")


def test_a_step_that_fails_leaves_lengths_and_state_where_they_were(emulated, counting_registered,
                                                                   tmp_path):
    """A mixer from outside the package, with state of its own and a cache whose rows are not
    keys and values (one plane of [hidden]): built, stepped in two cuts with equal results,
    and a step that raises after the mixer advanced its state is undone."""
    from tgo_b200.engine.step import StepEntry
    raw = dict(architectures=["CountingToy"], width=24, vocab=40, inner=32)
    d = tiny.make_model_dir(tmp_path / "toy", raw, seed=5, sigma=0.2)
    loaded = cpu_model(d, raw)
    assert [(g.planes, g.row_shape) for g in loaded.model.groups] == [(1, (24,))]
    toks = [3, 9, 1, 30, 7, 7, 12, 5, 0, 39, 8]
    whole = loaded.new_engine(page_size=4, max_tokens=64, num_slots=2)
    assert whole.storage.kv[0].shape == (1, 1, 17, 4, 24)
    whole.admit("w")
    want = whole.step([StepEntry("w", toks, list(range(len(toks))))]).clone()
    eng = loaded.new_engine(page_size=4, max_tokens=64, num_slots=2)
    eng.admit("a")
    first = eng.step([StepEntry("a", toks[:6], list(range(6)))]).clone()
    state = {c: t.clone() for c, t in eng.storage.state.items()}
    CountingMixer.fail_next = True
    with pytest.raises(RuntimeError, match="gave up"):
        eng.step([StepEntry("a", toks[6:], list(range(5)))])
    assert eng.length("a") == 6
    for c, t in state.items():
        assert torch.equal(eng.storage.state[c], t)
    rest = eng.step([StepEntry("a", toks[6:], list(range(5)))])
    assert torch.allclose(torch.cat([first, rest]), want, atol=1e-5)
    # the toy counts no flops and reads no cache by its own account: measurement still adds up
    assert loaded.model.flops([5], [0]) == 2.0 * 5 * 24 * 3 * 32 + 2.0 * 24 * 40
    assert loaded.model.cache_bytes_read(100) == 0.0


def test_parts_count_their_own_flops_and_bytes(tmp_path):
    """Model.flops sums what the parts report: for the tiny configurations it is the count
    written out by hand here."""
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    for name in ("A", "B"):
        cfg, _ = tiny.TINIES[name]
        model = Model(model_spec_from_config(cfg), torch.float32, "cpu")
        d, H, Hkv, dh = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], \
            cfg["head_dim"]
        f, V, L = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
        n, first = 37, 11
        windows = [cfg.get("sliding_window") if (cfg.get("layer_types") or ["full_attention"] * L)[i]
                   == "sliding_attention" else None for i in range(L)]
        want = 2.0 * d * V
        for w in windows:
            want += 2.0 * n * d * (H * dh + 2 * Hkv * dh) + 2.0 * n * H * dh * d + 2.0 * n * d * 3 * f
            keys = sum(min(first + t + 1, w) if w else first + t + 1 for t in range(n))
            want += 4.0 * H * dh * keys
        assert model.flops([n], [first]) == want
        per_token = sum(2 * Hkv * dh * 4 * (min(100, w) if w else 100) for w in windows)
        assert model.cache_bytes_read(100) == per_token
        assert model.cache_bytes_per_token() == L * 2 * Hkv * dh * 4


def test_a_model_folder_written_by_plain_code(emulated, tmp_path):
    """The tiny configurations' folders are written by the product's own writer. This one is
    written by the plain code of the tests (names spelled out here, the container written
    from its description), so a fault that the product's writer and reader share cannot
    hide: the engine reads it and gives the plain implementation's logits."""
    import json
    import os
    cfg = dict(tiny.TINY_B)
    rng = np.random.default_rng(44)
    d, H, Hkv, dh, f, V = 96, 6, 2, 32, 224, 384
    arrays = {"model.embed_tokens.weight": rng.normal(0, 0.05, (V, d)),
              "lm_head.weight": rng.normal(0, 0.05, (V, d)),
              "model.norm.weight": 1 + rng.normal(0, 0.1, d)}
    for i in range(3):
        p = f"model.layers.{i}."
        arrays.update({
            p + "input_layernorm.weight": 1 + rng.normal(0, 0.1, d),
            p + "post_attention_layernorm.weight": 1 + rng.normal(0, 0.1, d),
            p + "self_attn.q_proj.weight": rng.normal(0, 0.05, (H * dh, d)),
            p + "self_attn.k_proj.weight": rng.normal(0, 0.05, (Hkv * dh, d)),
            p + "self_attn.v_proj.weight": rng.normal(0, 0.05, (Hkv * dh, d)),
            p + "self_attn.o_proj.weight": rng.normal(0, 0.05, (d, H * dh)),
            p + "self_attn.q_norm.weight": 1 + rng.normal(0, 0.1, dh),
            p + "self_attn.k_norm.weight": 1 + rng.normal(0, 0.1, dh),
            p + "mlp.gate_proj.weight": rng.normal(0, 0.05, (f, d)),
            p + "mlp.up_proj.weight": rng.normal(0, 0.05, (f, d)),
            p + "mlp.down_proj.weight": rng.normal(0, 0.05, (d, f))})
    folder = tmp_path / "by_hand"
    os.makedirs(folder)
    with open(folder / "config.json", "w") as fh:
        json.dump(cfg, fh)
    plain.write_safetensors(str(folder / "model.safetensors"), arrays, bfloat16=True)
    pc, pw = plain.load_model_dir(str(folder))
    assert np.abs(pw["model.layers.1.mlp.up_proj.weight"] -
                  arrays["model.layers.1.mlp.up_proj.weight"]).max() < 0.05 * 2 ** -7 * 6
    loaded = cpu_model(str(folder), cfg)
    toks = tiny.random_requests(V, [50], seed=1)["r0"]
    want = plain.forward(pc, pw, toks)
    eng = loaded.new_engine(page_size=8, max_tokens=64, num_slots=1)
    got = tiny.run_trace_engine(eng, tiny.trace_portions({"r0": toks}))
    worst, where, tol = tiny.compare(got, {"r0": want}, cfg, "float32")
    assert worst <= tol, (worst, where)
