"""Each part alone on the GPU against the plain implementation, and parts defined here, in
the test, registered, built and stepped without a change to the package: a mixer with state
of its own, and a position encoding the attention kernel does not know."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (3e-2 if dtype == torch.bfloat16 else 2e-5) * max(1.0, scale)


def rnd(*shape, scale=1.0, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def bf16_exact(t):
    return t.to(torch.bfloat16).float()


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from tgo_b200.config.spec import NormSpec
    from tgo_b200.parts.norm import RMSNorm
    d, eps = 200, 1e-5
    part = RMSNorm(NormSpec("rmsnorm", eps), d, "n.weight")
    assert [(w.name, w.shape, w.role) for w in part.weight_specs()] == [("n.weight", (d,), "gain")]
    gain = 1 + 0.1 * rnd(d, seed=1)
    part.bind({"n.weight": gain.to(DEV)})
    h, delta = rnd(7, d, seed=2), bf16_exact(rnd(7, d, seed=3))
    hd = h.to(DEV)
    out = part.forward(hd, delta.to(dtype).to(DEV), dtype)
    want = plain.rmsnorm((h + delta).double().numpy(), gain.double().numpy(), eps)
    assert np.abs(out.float().cpu().numpy() - want).max() < tol(dtype, np.abs(want).max())
    assert torch.allclose(hd.cpu(), h + delta, atol=1e-6)          # the add stays in the stream


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dh,rot", [(16, 16), (64, 32), (96, 96)])
def test_rope_part(dtype, dh, rot):
    from tgo_b200.config.spec import PositionSpec
    from tgo_b200.parts.base import StepContext
    from tgo_b200.parts.position import RopeHalfSplit
    H, Hkv, T, theta = 3, 1, 6, 12345.0
    part = RopeHalfSplit(PositionSpec("rope_half_split", rot, theta), dh, DEV)
    pos = torch.tensor([0, 1, 5, 77, 300, 4095], dtype=torch.int32, device=DEV)
    q, k = bf16_exact(rnd(T, H * dh, seed=1)), bf16_exact(rnd(T, Hkv * dh, seed=2))
    qd, kd = q.to(dtype).to(DEV), k.to(dtype).to(DEV)
    ctx = StepContext(T, 1, pos, pos, pos, pos, pos, pos, pos, dtype)
    part.apply(qd, kd, ctx, H, Hkv, dh)
    wq = plain.rope_half_split(q.double().numpy().reshape(T, H, dh), pos.cpu().numpy(), theta, rot)
    wk = plain.rope_half_split(k.double().numpy().reshape(T, Hkv, dh), pos.cpu().numpy(), theta, rot)
    assert np.abs(qd.float().cpu().numpy().reshape(T, H, dh) - wq).max() < tol(dtype, 3)
    assert np.abs(kd.float().cpu().numpy().reshape(T, Hkv, dh) - wk).max() < tol(dtype, 3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [3, 150])
@pytest.mark.parametrize("d,f", [(96, 224), (72, 100)])
def test_swiglu_part(dtype, T, d, f):
    from tgo_b200.config.spec import FeedForwardSpec
    from tgo_b200.parts.feed_forward import SwiGLU
    from tgo_b200.config.qwen3 import FEED_FORWARD_TENSORS
    part = SwiGLU(FeedForwardSpec("swiglu", f, tensors=FEED_FORWARD_TENSORS), d, "")
    assert {w.name: w.shape for w in part.weight_specs()} == {
        "mlp.gate_proj.weight": (f, d), "mlp.up_proj.weight": (f, d), "mlp.down_proj.weight": (d, f)}
    with pytest.raises(ValueError, match="names no tensor for the role 'down'"):
        SwiGLU(FeedForwardSpec("swiglu", f, tensors=FEED_FORWARD_TENSORS[:2]), d, "")
    w = {n: bf16_exact(rnd(*s.shape, scale=0.2, seed=i)) for i, (n, s) in
         enumerate((s.name, s) for s in part.weight_specs())}
    part.bind({n: t.to(dtype).to(DEV) for n, t in w.items()})
    assert part.interleaved == (f % 8 == 0)
    x = bf16_exact(rnd(T, d, seed=9))
    want = plain.swiglu_mlp(x.double().numpy(), *(w[f"mlp.{n}_proj.weight"].double().numpy()
                                                  for n in ("gate", "up", "down")))
    out = part.forward(x.to(dtype).to(DEV), None)
    assert np.abs(out.float().cpu().numpy() - want).max() < tol(dtype, np.abs(want).max())
    # with the stream offered, the part either adds into it (returning None) or hands the
    # result back for the caller to add; never both
    h = rnd(T, d, seed=4).to(DEV)
    h0 = h.clone()
    back = part.forward(x.to(dtype).to(DEV), None, residual=h)
    if back is None:
        assert np.abs((h - h0).cpu().numpy() - want).max() < tol(dtype, np.abs(want).max())
    else:
        assert torch.equal(h, h0)
        assert np.abs(back.float().cpu().numpy() - want).max() < tol(dtype, np.abs(want).max())


def attention_setup(dtype, window, H=6, Hkv=2, dh=32, d=96, theta=1e4, eps=1e-5):
    from tgo_b200.config.spec import MixerSpec, PositionSpec
    from tgo_b200.parts.attention import GQAAttention
    names = tuple((role, "a." + role + ("_norm.weight" if role.endswith("norm") else "_proj.weight"))
                  for role in ("q", "k", "v", "o")) + (("q_norm", "a.q_norm.weight"),
                                                      ("k_norm", "a.k_norm.weight"))
    spec = MixerSpec("gqa_attention", H, Hkv, dh, qk_norm=True, window=window,
                     position=PositionSpec("rope_half_split", dh, theta), norm_eps=eps,
                     tensors=names)
    part = GQAAttention(spec, d, "", DEV)
    w = {}
    for i, s in enumerate(part.weight_specs()):
        t = rnd(*s.shape, scale=0.15, seed=20 + i)
        w[s.name] = bf16_exact(1 + t if s.role == "gain" else t)
    part.bind({n: (t if n.endswith("norm.weight") else t.to(dtype)).to(DEV) for n, t in w.items()})
    cfg = dict(num_attention_heads=H, num_key_value_heads=Hkv, head_dim=dh, hidden_size=d,
               rms_norm_eps=eps, rope_theta=theta)
    return part, w, cfg


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_whole_and_in_portions(dtype, window):
    """The mixer alone over its own little cache: one request whole, then the same request in
    portions beside another request's single tokens."""
    from tgo_b200.parts.base import CacheNeed, LayerCache, StepContext
    part, w, cfg = attention_setup(dtype, window)
    assert part.cache_need() == CacheNeed("window" if window else "full", window, 2, (2, 32))
    assert part.state_need() is None
    T, ps, d = 45, 8, 96
    x = bf16_exact(rnd(T, d, seed=3))
    want = plain.attention_block(x.double().numpy(), np.arange(T),
                                 {k: v.double().numpy() for k, v in w.items()}, "a.", cfg, window)
    pages = 16
    planes = torch.zeros(2, pages, 2, ps, 32, dtype=dtype, device=DEV)      # keys, values
    table = torch.tensor([[9, 3, 12, 1, 7, 5], [2, 4, 6, 8, 10, 11]], dtype=torch.int32, device=DEV)

    def step(chunks):
        """chunks: list of (request, first position, rows of x)."""
        ids, pos, seq, slots, rows = [], [], [], [], []
        for b, (req, first, xs) in enumerate(chunks):
            n = xs.shape[0]
            pos += list(range(first, first + n))
            seq += [b] * n
            slots += [int(table[req, p // ps]) * ps + p % ps for p in range(first, first + n)]
            rows.append(xs)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)     # noqa: E731
        n_tok = len(pos)
        ctx = StepContext(n_tok, len(chunks), i32([0] * n_tok), i32(pos), i32(seq), i32([0]),
                          i32([0]), i32([0]), i32([0]), dtype, extents=[c[2].shape[0] for c in chunks],
                          max_context=max(c[1] + c[2].shape[0] for c in chunks),
                          decode_only=all(c[2].shape[0] == 1 for c in chunks))
        tb = torch.stack([table[c[0]] for c in chunks]).contiguous()
        cache = LayerCache(planes, ps, tb, i32(slots), True)
        out = part.forward(torch.cat(rows).to(dtype).to(DEV), ctx, cache)
        return out.float().cpu().numpy()
    got = step([(0, 0, x)])
    assert np.abs(got - want).max() < tol(dtype, np.abs(want).max())
    # again in portions of request 1's pages, with request 0 decoding beside it
    outs, o = [], 0
    for n in (7, 2, 16, 1, 1, 18):
        chunk = [(1, o, x[o:o + n])]
        if o:
            chunk.append((0, 44, x[44:45]))                   # rewrites its last position
        outs.append(step(chunk)[:n])
        o += n
    assert np.abs(np.concatenate(outs) - want).max() < tol(dtype, np.abs(want).max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype, tmp_path):
    """A whole layer (both norms, mixer, feed-forward, both adds) against the plain layer."""
    cfg, run = tiny.TINIES["B"]
    d = tiny.make_model_dir(tmp_path / "b", cfg, 3, 0.1)
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    model = tgo_b200.open(d, dtype=dtype)
    pc, pw = plain.load_model_dir(d)
    toks = tiny.random_requests(384, [30], 1)["r0"]
    eng = model.new_engine(page_size=8, max_tokens=64, num_slots=1, graphs=False)
    eng.admit("x")
    eng.cache.grow("x", 30)
    ctx, tables, slots = eng.build_context([StepEntry("x", toks, [])])
    h = torch.tensor(plain.embedding(pw["model.embed_tokens.weight"], toks), dtype=torch.float32,
                     device=DEV)
    block = model.model.blocks[1]                              # the layer with the window
    cache = model.model.layer_cache(1, ctx, eng.storage, tables, slots)
    h2, pending = block.forward(h.clone(), None, ctx, cache)
    got = (h2 if pending is None else h2 + pending.float()).cpu().numpy()
    x = h.double().cpu().numpy()
    p = "model.layers.1."
    n = plain.rmsnorm(x, pw[p + "input_layernorm.weight"], pc["rms_norm_eps"])
    x = x + plain.attention_block(n, np.arange(30), pw, p + "self_attn.", pc, 24)
    n = plain.rmsnorm(x, pw[p + "post_attention_layernorm.weight"], pc["rms_norm_eps"])
    x = x + plain.swiglu_mlp(n, pw[p + "mlp.gate_proj.weight"], pw[p + "mlp.up_proj.weight"],
                             pw[p + "mlp.down_proj.weight"])
    assert np.abs(got - x).max() < tol(dtype, np.abs(x).max())


# ------------------------------------------------------------- parts defined in the test


class DecayMixer:
    """A mixer with fixed-size state of its own and no keys or values: per request
    s <- decay * s + x_t, y_t = s . W^T, tokens in order. Written with torch on the device
    (a test part; the package's own mixers use its kernels)."""

    def __init__(self, spec, hidden, prefix, device=None):
        self.hidden = hidden
        self.name = prefix + dict(spec.tensors)["mix"]
        self.decay = dict(spec.extra)["decay"]
        self.w = None

    def weight_specs(self):
        from tgo_b200.weights.binder import WeightSpec
        return [WeightSpec(self.name, (self.hidden, self.hidden))]

    def bind(self, weights):
        self.w = weights.pop(self.name)

    def cache_need(self):
        return None

    def state_need(self):
        from tgo_b200.parts.base import StateNeed
        return StateNeed((self.hidden,))

    def read_state(self, state, slots, b):
        return state.index_select(0, slots[b:b + 1])[0]        # no trip to the host

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        slots = ctx.state_slots.long()
        base = 0
        for b, n in enumerate(ctx.extents):
            s = self.read_state(cache.state, slots, b)
            for t in range(base, base + n):
                s = self.decay * s + x[t].float()
                out[t] = (s @ self.w.float().t()).to(x.dtype)
            cache.state.index_copy_(0, slots[b:b + 1], s[None])
            base += n
        return out


class ChattyDecayMixer(DecayMixer):
    """The same, but it asks the host for the slot number: such a forward cannot be captured
    as a CUDA graph, and the engine then runs decode steps one launch at a time."""

    def read_state(self, state, slots, b):
        return state[int(slots[b].item())]


class ShiftPosition:
    """A position encoding the attention kernel does not know: channel 0 of every head of q
    and k gets + position / 64. Not fusable, so the mixer calls `apply` between its norm
    and its store."""
    fusable = False

    def __init__(self, spec, head_dim, device):
        self.head_dim = head_dim

    def apply(self, q, k, ctx, num_heads, num_kv_heads, head_dim):
        add = (ctx.positions.float() / 64)[:, None]
        for t, heads in ((q, num_heads), (k, num_kv_heads)):
            if t is not None:
                v = t.view(t.shape[0], heads, head_dim)
                v[:, :, 0] = (v[:, :, 0].float() + add).to(t.dtype)


class RoutedFeedForward:
    """A feed-forward with routing: float32 router logits x . R^T, each token goes to its one
    best expert (lowest id on ties), y = D_e . silu(U_e . x). Written with torch on the
    device, without a trip to the host, so decode steps with it are captured."""

    def __init__(self, spec, hidden, prefix, device=None):
        self.hidden, self.inter = hidden, spec.intermediate_size
        self.prefix = prefix + dict(spec.tensors)["root"]
        self.experts = dict(spec.extra)["experts"]

    def weight_specs(self):
        from tgo_b200.weights.binder import WeightSpec
        p, E = self.prefix, self.experts
        specs = [WeightSpec(p + "router.weight", (E, self.hidden))]
        for e in range(E):
            specs += [WeightSpec(p + f"experts.{e}.up.weight", (self.inter, self.hidden)),
                      WeightSpec(p + f"experts.{e}.down.weight", (self.hidden, self.inter))]
        return specs

    def bind(self, weights):
        p, E = self.prefix, self.experts
        self.router = weights.pop(p + "router.weight").float()
        self.up = torch.stack([weights.pop(p + f"experts.{e}.up.weight") for e in range(E)]).float()
        self.down = torch.stack([weights.pop(p + f"experts.{e}.down.weight") for e in range(E)]).float()

    def forward(self, x, ctx):
        xf = x.float()
        choice = torch.argmax(xf @ self.router.t(), dim=1)          # first of equal maxima
        u = torch.bmm(self.up.index_select(0, choice), xf[:, :, None])[:, :, 0]
        act = (u * torch.sigmoid(u)).to(x.dtype).float()
        return torch.bmm(self.down.index_select(0, choice), act[:, :, None])[:, :, 0].to(x.dtype)


def toy_spec(raw):
    """config.json -> ModelSpec of a two-layer toy: a decay mixer, then attention with the
    shift encoding. Nothing of it is a model of anyone's."""
    from tgo_b200.config.spec import (FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec,
                                      NormSpec, PositionSpec)
    d, V = raw["width"], raw["vocab"]
    norm = NormSpec("rmsnorm", raw["eps"])
    # the toy checkpoint has names of its own, and ships q, k and v as one matrix in layer 1
    # and gate and up as one matrix in both layers: the package's parts take the tables as given
    ffn = FeedForwardSpec("swiglu", raw["inner"],
                          tensors=(("gate_up", "ff.gu.weight"), ("down", "ff.out.weight")))
    ffn0 = FeedForwardSpec("test_routed", raw["inner"], tensors=(("root", "moe."),),
                           extra=(("experts", raw["experts"]),)) if raw.get("experts") else ffn
    block = (("mixer_norm", "n1.weight"), ("ffn_norm", "n2.weight"))
    layers = [LayerSpec("prenorm_residual", "layers.0.",
                        MixerSpec(raw.get("mixer", "test_decay"), tensors=(("mix", "decay.mix.weight"),),
                                  extra=(("decay", raw["decay"]),)),
                        ffn0, norm, block),
              LayerSpec("prenorm_residual", "layers.1.",
                        MixerSpec("gqa_attention", 4, 2, 16, qk_norm=True,
                                  position=PositionSpec("test_shift"), norm_eps=raw["eps"],
                                  tensors=(("qkv", "att.qkv.weight"), ("o", "att.out.weight"),
                                           ("q_norm", "att.qn.weight"), ("k_norm", "att.kn.weight"))),
                        ffn, norm, block)]
    return ModelSpec("ToyForTests", d, V, layers, [LayerCall(0), LayerCall(1)], norm, "embed.weight",
                     "norm.weight", None, source=dict(raw))


@pytest.fixture()
def toy_registered():
    from tgo_b200.registry import ARCHITECTURES, FEED_FORWARDS, MIXERS, POSITIONS
    ARCHITECTURES.register("ToyForTests", toy_spec, replace=True)
    FEED_FORWARDS.register("test_routed", RoutedFeedForward, replace=True)
    MIXERS.register("test_decay", DecayMixer, replace=True)
    MIXERS.register("test_chatty_decay", ChattyDecayMixer, replace=True)
    POSITIONS.register("test_shift", ShiftPosition, replace=True)
    yield
    ARCHITECTURES.unregister("ToyForTests")
    FEED_FORWARDS.unregister("test_routed")
    MIXERS.unregister("test_decay")
    MIXERS.unregister("test_chatty_decay")
    POSITIONS.unregister("test_shift")


def toy_plain(w, raw, toks):
    eps, T = raw["eps"], len(toks)
    h = w["embed.weight"][np.asarray(toks)]
    # layer 0: the decay mixer
    n = plain.rmsnorm(h, w["layers.0.n1.weight"], eps)
    s, ys = np.zeros(raw["width"]), []
    for t in range(T):
        s = raw["decay"] * s + n[t]
        ys.append(s @ w["layers.0.decay.mix.weight"].T)
    h = h + np.stack(ys)
    f = raw["inner"]

    def joined_ffn(layer, x):
        gu = w[f"layers.{layer}.ff.gu.weight"]
        return plain.swiglu_mlp(x, gu[:f], gu[f:], w[f"layers.{layer}.ff.out.weight"])
    n = plain.rmsnorm(h, w["layers.0.n2.weight"], eps)
    if raw.get("experts"):
        choice = np.argmax(n @ w["layers.0.moe.router.weight"].T, axis=1)
        ys = []
        for t in range(T):
            u = w[f"layers.0.moe.experts.{choice[t]}.up.weight"] @ n[t]
            ys.append(w[f"layers.0.moe.experts.{choice[t]}.down.weight"] @ (u / (1 + np.exp(-u))))
        h = h + np.stack(ys)
    else:
        h = h + joined_ffn(0, n)
    # layer 1: attention with the shift encoding, q, k, v from one joined matrix
    p = "layers.1.att."
    n = plain.rmsnorm(h, w["layers.1.n1.weight"], eps)
    qkv = plain.linear(n, w[p + "qkv.weight"])
    q = plain.rmsnorm(qkv[:, :64].reshape(T, 4, 16), w[p + "qn.weight"], eps)
    k = plain.rmsnorm(qkv[:, 64:96].reshape(T, 2, 16), w[p + "kn.weight"], eps)
    v = qkv[:, 96:].reshape(T, 2, 16)
    q[:, :, 0] += np.arange(T)[:, None] / 64
    k[:, :, 0] += np.arange(T)[:, None] / 64
    a = plain.causal_gqa_attention(q, k, v, 0.25).reshape(T, 64)
    h = h + plain.linear(a, w[p + "out.weight"])
    n = plain.rmsnorm(h, w["layers.1.n2.weight"], eps)
    h = h + joined_ffn(1, n)
    return plain.linear(plain.rmsnorm(h, w["norm.weight"], eps), w["embed.weight"])


@pytest.mark.parametrize("dtype,mixer,experts", [
    ("float32", "test_decay", 0), ("bfloat16", "test_decay", 0), ("float32", "test_chatty_decay", 0),
    ("float32", "test_decay", 3)])
def test_toy_parts_are_registered_built_and_stepped(toy_registered, tmp_path, dtype, mixer, experts):
    """Parts from outside the package: a mixer with state of its own, a position encoding the
    kernels do not know, and (last case) a feed-forward that routes each token to one of
    three experts."""
    import tgo_b200
    raw = dict(architectures=["ToyForTests"], width=48, vocab=90, inner=80, eps=1e-5, decay=0.75,
               mixer=mixer, experts=experts)
    d = tiny.make_model_dir(tmp_path / "toy", raw, seed=2, sigma=0.15)
    model = tgo_b200.open(d, dtype=dtype)
    assert model.model.state_shapes == {0: (48,)} and [g.calls for g in model.model.groups] == [[1]]
    w = plain.read_safetensors(str(tmp_path / "toy" / "model.safetensors"))
    reqs = tiny.random_requests(90, [40, 3, 21], seed=6)
    want = {rid: toy_plain(w, raw, toks) for rid, toks in reqs.items()}
    for fam in (tiny.trace_whole, tiny.trace_tail, tiny.trace_portions, tiny.trace_mixed):
        trace = fam(reqs)
        eng = model.new_engine(page_size=8, max_tokens=tiny.max_tokens_of(trace), num_slots=4)
        got = tiny.run_trace_engine(eng, trace)
        scale = max(np.abs(v).max() for v in want.values())
        worst = max(np.abs(row - want[rid][pos]).max() for (rid, pos), row in got.items())
        assert worst < tol(torch.bfloat16 if dtype == "bfloat16" else torch.float32, scale) * 2, \
            (fam.__name__, worst)
        if fam is tiny.trace_tail:             # single-token steps: captured, unless chatty
            assert eng.use_graphs == (mixer == "test_decay")


# --------------------------------------------------------------- the run order is data


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_run_twice_and_borrowed_cache_on_the_gpu(tmp_path, dtype):
    """Calls [0, 1, 0, 1] over two layers' weights, the last call reading call 1's cache: a
    prompt in two portions, then tokens one by one (captured decode steps), against the plain
    implementation of the same order."""
    import plain_qwen3 as plain
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
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    model = Model(spec, dt, DEV)
    model.bind(load_weights(model.weight_specs(), SafetensorsRepo(d), dt, DEV, model.tied_alias()))
    assert [len(g.calls) for g in model.groups] == [3]          # calls 0, 1, 2 own a cache
    pc, pw = plain.load_model_dir(d)
    toks = tiny.random_requests(256, [40], seed=5)["r0"]
    want = tiny.repeated_layers_reference(pc, pw, toks)
    eng = Engine(model, page_size=8, max_tokens=64, num_slots=2)
    eng.admit("x")
    rows = [eng.step([StepEntry("x", toks[:9], list(range(9)))]).float().cpu(),
            eng.step([StepEntry("x", toks[9:30], list(range(21)))]).float().cpu()]
    for t in toks[30:]:
        rows.append(eng.step([StepEntry("x", [t], [0])]).float().cpu())
    got = torch.cat(rows).numpy()
    # the bound is a function of the number of layers a token passes: four calls here
    tol = tiny.tolerance(dict(cfg, num_hidden_layers=len(spec.run_order)), dtype, want,
                         tiny.repeated_layers_reference(pc, pw, toks, plain.round_bfloat16))
    tiny.note(f"run_twice/{dtype}", float(np.abs(got - want).max()), tol)
    assert np.abs(got - want).max() <= tol


def test_toy_model_through_the_bench_command(toy_registered, tmp_path):
    """`tgo bench` on the toy architecture: its foreign parts count no flops and read no cache
    by their own account, and the measurement still runs and adds up what the package's parts
    report (nothing in the measuring code knows a mixer's or a feed-forward's fields)."""
    import io
    import json

    from tgo_b200 import cli
    raw = dict(architectures=["ToyForTests"], width=48, vocab=90, inner=80, eps=1e-5, decay=0.75,
               mixer="test_decay", experts=3)
    d = tiny.make_model_dir(tmp_path / "toy", raw, seed=2, sigma=0.15)
    out, err, rec = io.StringIO(), io.StringIO(), tmp_path / "rec.json"
    rc = cli.main(["bench", "--tokens", "6", "--prompt-tokens", "12", "--warmup", "2", "--context", "64",
                   "--batch", "1,3", "--page-size", "8", "--json", str(rec), d], out=out, err=err)
    assert rc == 0, err.getvalue()
    got = json.loads(rec.read_text())
    assert got["decode"]["tokens_per_s"] > 0 and set(got["decode_by_batch"]) == {"1", "3"}
    # layer 1 of the toy is the package's attention and feed-forward: their flops are counted
    attention = 2 * 12 * 48 * (64 + 64) + 2 * 12 * 64 * 48 + 4 * 64 * (12 * 13 // 2)
    feed_forward = 2 * 12 * 48 * 3 * 80
    assert got["prefill"]["flops"] == attention + feed_forward + 2 * 48 * 90
