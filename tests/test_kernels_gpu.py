"""Each CUDA kernel alone against a plain float32 (or float64) torch restatement of the
same operation, at sizes other than the tiny models': widths that are no power of two,
head sizes in steps of 16, odd head counts and groups, scattered pages, windows."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from tgo_b200.kernels import ops as o
    return o


def attention_part():
    """The module that picks the attention kernel for a step."""
    from tgo_b200.parts import attention
    return attention


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


# --------------------------------------------------------------------- elementwise


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    table = rnd(1000, 200, dtype=dtype)
    ids = torch.tensor([0, 999, 17, 17, 501], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 200, dtype=torch.float32, device=DEV)
    ops().embed(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("d", [72, 200, 4096, 5120, 20000])
@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(d, act):
    T, eps = 5, 1e-5
    h = rnd(T, d, seed=1)
    delta = rnd(T, d, dtype=act, seed=2)
    gain = 1 + 0.1 * rnd(d, seed=3)
    want_h = h + delta.float()
    want = (want_h * torch.rsqrt((want_h * want_h).mean(-1, keepdim=True) + eps)) * gain
    out = torch.empty(T, d, dtype=act, device=DEV)
    h2 = h.clone()
    ops().add_rmsnorm(h2, delta, gain, eps, out)
    assert torch.allclose(h2, want_h, rtol=0, atol=1e-6)
    assert torch.allclose(out.float(), want, **tol(act))
    # no delta
    out2 = torch.empty(T, d, dtype=act, device=DEV)
    h3 = h.clone()
    ops().add_rmsnorm(h3, None, gain, eps, out2)
    want2 = (h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps)) * gain
    assert torch.equal(h3, h) and torch.allclose(out2.float(), want2, **tol(act))
    # selected rows: h stays, the add happens on the fly
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, d, dtype=act, device=DEV)
    h4 = h.clone()
    ops().add_rmsnorm(h4, delta, gain, eps, out3, rows)
    assert torch.equal(h4, h) and torch.allclose(out3.float(), want[rows.long()], **tol(act))


@pytest.mark.parametrize("f,T", [(88, 7), (200, 1), (12288, 3), (1001, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(f, T, dtype):
    gu = rnd(T, 2 * f, dtype=dtype, scale=2.0)
    out = torch.empty(T, f, dtype=dtype, device=DEV)
    ops().swiglu(gu, out)
    g, u = gu[:, :f].float(), gu[:, f:].float()
    want = g / (1 + torch.exp(-g)) * u
    assert torch.allclose(out.float(), want, **tol(dtype))
    if f % 8 == 0:
        v = gu.reshape(T, f // 8, 2, 8)
        g, u = v[:, :, 0].reshape(T, f).float(), v[:, :, 1].reshape(T, f).float()
        ops().swiglu(gu, out, interleaved=True)
        assert torch.allclose(out.float(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


def rope_ref(x, pos, theta, rot):
    half = rot // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float64, device=x.device) / rot)
    ang = pos.double()[:, None] * inv[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    y = x.clone()
    lo, hi = x[..., :half], x[..., half:rot]
    y[..., :half] = lo * cos - hi * sin
    y[..., half:rot] = lo * sin + hi * cos
    return y


@pytest.mark.parametrize("H,Hkv", [(8, 2), (5, 1), (32, 8), (3, 3)])
def test_qk_norm_rope_cache_many_tokens(H, Hkv):
    """Head size 128, bfloat16, a prompt portion's worth of tokens: the kernel with half a
    warp per head vector (head counts that leave half-warps idle or mix q, k and v in a warp)."""
    T, ps, pages, eps, theta, dh = 70, 16, 9, 1e-6, 1e6, 128
    dtype = torch.bfloat16
    qkv = rnd(T, (H + 2 * Hkv) * dh, dtype=dtype, seed=H)
    q, k, v = qkv[:, :H * dh], qkv[:, H * dh:(H + Hkv) * dh], qkv[:, (H + Hkv) * dh:]
    qg, kg = 1 + 0.1 * rnd(dh, seed=5), 1 + 0.1 * rnd(dh, seed=6)
    pos = torch.arange(300, 300 + T, dtype=torch.int32, device=DEV)
    slot_list = [(5 * t + 3) % (pages * ps) if t != 11 else -1 for t in range(T)]     # scattered, one padded
    assert len({s for s in slot_list if s >= 0}) == T - 1
    slots = torch.tensor(slot_list, dtype=torch.int32, device=DEV)
    inv = (theta ** (-2.0 * torch.arange(dh // 2, dtype=torch.float64) / dh)).to(DEV)
    kc = torch.zeros(pages, Hkv, ps, dh, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)

    def norm(x, g):
        x = x.float()
        return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)) * g
    want_q = rope_ref(norm(q.reshape(T, H, dh), qg), pos, theta, dh)
    want_k = rope_ref(norm(k.reshape(T, Hkv, dh), kg), pos, theta, dh)
    want_v = v.reshape(T, Hkv, dh).clone()
    table = ops().rope_table(pos, inv)
    ops().qk_norm_rope_cache(q, k, v, H, Hkv, dh, qg, kg, eps, table, dh, slots, kc, vc, ps)
    assert torch.allclose(q.reshape(T, H, dh).float(), want_q, **tol(dtype))
    for t in range(T):
        s = slot_list[t]
        if s < 0:
            continue
        assert torch.allclose(kc[s // ps, :, s % ps].float(), want_k[t], **tol(dtype))
        assert torch.equal(vc[s // ps, :, s % ps], want_v[t])
    written = {s for s in slot_list if s >= 0}
    for s in range(pages * ps):
        if s not in written:
            assert not kc[s // ps, :, s % ps].any() and not vc[s // ps, :, s % ps].any()


@pytest.mark.parametrize("H,Hkv,dh,rot", [(5, 5, 16, 16), (6, 2, 48, 32), (8, 1, 128, 128),
                                          (3, 3, 80, 80)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qk_norm_rope_cache(H, Hkv, dh, rot, dtype):
    T, ps, pages, eps, theta = 9, 4, 12, 1e-5, 5e5
    width = (H + 2 * Hkv) * dh
    qkv = rnd(T, width, dtype=dtype)
    q, k, v = qkv[:, :H * dh], qkv[:, H * dh:(H + Hkv) * dh], qkv[:, (H + Hkv) * dh:]
    qg, kg = 1 + 0.1 * rnd(dh, seed=5), 1 + 0.1 * rnd(dh, seed=6)
    pos = torch.tensor([0, 1, 2, 3, 100, 101, 7, 4000, 9], dtype=torch.int32, device=DEV)
    slots = torch.tensor([4, 5, 6, 7, 40, 41, -1, 13, 47], dtype=torch.int32, device=DEV)
    inv = (theta ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV)
    kc = torch.zeros(pages, Hkv, ps, dh, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)

    def norm(x, g):
        x = x.float()
        return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)) * g
    want_q = rope_ref(norm(q.reshape(T, H, dh), qg), pos, theta, rot)
    want_k = rope_ref(norm(k.reshape(T, Hkv, dh), kg), pos, theta, rot)
    want_v = v.reshape(T, Hkv, dh).clone()
    table = ops().rope_table(pos, inv)
    ops().qk_norm_rope_cache(q, k, v, H, Hkv, dh, qg, kg, eps, table, rot, slots, kc, vc, ps)
    assert torch.allclose(q.reshape(T, H, dh).float(), want_q, **tol(dtype))
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        assert torch.allclose(kc[s // ps, :, s % ps].float(), want_k[t], **tol(dtype))
        assert torch.equal(vc[s // ps, :, s % ps], want_v[t])
    written = {int(s) for s in slots if s >= 0}
    for s in range(pages * ps):
        if s not in written:
            assert not kc[s // ps, :, s % ps].any() and not vc[s // ps, :, s % ps].any()


@pytest.mark.parametrize("M,N,K", [(1, 5, 7), (3, 130, 96), (70, 65, 33), (129, 257, 1000)])
def test_sgemm(M, N, K):
    x, w = rnd(M, K, seed=1), rnd(N, K, seed=2)
    out = torch.empty(M, N, device=DEV)
    ops().sgemm_tn(x, w, out)
    want = (x.double() @ w.double().t()).float()
    assert torch.allclose(out, want, rtol=1e-5, atol=1e-4)
    # a row's result does not depend on the rows beside it
    out1 = torch.empty(1, N, device=DEV)
    ops().sgemm_tn(x[M - 1:M].contiguous(), w, out1)
    assert torch.equal(out1[0], out[M - 1])


# ----------------------------------------------------------------------- attention


def paged_case(extents, firsts, H, Hkv, dh, ps, dtype, seed=0, crafted=None):
    """A ragged batch over a scattered paged cache. Returns the kernel inputs and the
    per-request dense keys and values."""
    g = torch.Generator().manual_seed(seed)
    B = len(extents)
    ctx_lens = [f + e for f, e in zip(firsts, extents)]
    n_pages = sum((c + ps - 1) // ps for c in ctx_lens) + 3
    perm = (torch.randperm(n_pages - 1, generator=g) + 1).tolist()      # page 0 stays unused
    width = max((c + ps - 1) // ps for c in ctx_lens)
    bt = torch.zeros(B, width, dtype=torch.int32)
    kc = torch.full((n_pages, Hkv, ps, dh), float("nan"))
    vc = torch.full((n_pages, Hkv, ps, dh), float("nan"))
    dense = []
    for b in range(B):
        K = torch.randn(ctx_lens[b], Hkv, dh, generator=g)
        V = torch.randn(ctx_lens[b], Hkv, dh, generator=g)
        if crafted is not None:
            crafted(b, K, V)
        K, V = K.to(dtype).float(), V.to(dtype).float()
        dense.append((K, V))
        for i in range((ctx_lens[b] + ps - 1) // ps):
            page = perm.pop()
            bt[b, i] = page
            n = min(ps, ctx_lens[b] - i * ps)
            kc[page, :, :n] = K[i * ps:i * ps + n].transpose(0, 1)
            vc[page, :, :n] = V[i * ps:i * ps + n].transpose(0, 1)
    T = sum(extents)
    q = torch.randn(T, H * dh, generator=g)
    pos, seq = [], []
    for b in range(B):
        pos += list(range(firsts[b], ctx_lens[b]))
        seq += [b] * extents[b]
    return dict(q=q.to(dtype).to(DEV), kc=kc.to(dtype).to(DEV), vc=vc.to(dtype).to(DEV),
                bt=bt.to(DEV), pos=torch.tensor(pos, dtype=torch.int32, device=DEV),
                seq=torch.tensor(seq, dtype=torch.int32, device=DEV), dense=dense,
                extents=extents, firsts=firsts)


def attention_ref(case, H, Hkv, dh, scale, window):
    q = case["q"].float().cpu()
    out = torch.zeros_like(q)
    t = 0
    G = H // Hkv
    for b, (e, f) in enumerate(zip(case["extents"], case["firsts"])):
        K, V = case["dense"][b]
        for i in range(e):
            p = f + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(H):
                s = (K[lo:p + 1, h // G] @ q[t, h * dh:(h + 1) * dh]) * scale
                w = torch.softmax(s.double(), 0).float()
                out[t, h * dh:(h + 1) * dh] = w @ V[lo:p + 1, h // G]
            t += 1
    return out


class Ctx:
    """The fields of a StepContext that the attention dispatch reads."""

    def __init__(self, case, decode):
        self.extents = case["extents"]
        self.positions, self.seq_ids = case["pos"], case["seq"]
        self.token_ids = case["pos"]
        self.num_seqs = len(self.extents)
        self.max_context = max(f + e for f, e in zip(case["firsts"], case["extents"]))
        self.decode_only = decode
        self.aux = {}


class Cache:
    def __init__(self, case, ps):
        self.k, self.v, self.block_tables, self.page_size = case["kc"], case["vc"], case["bt"], ps


SHAPES = [(4, 2, 16, 16), (6, 2, 32, 8), (8, 8, 64, 16), (32, 8, 128, 16), (5, 1, 48, 4),
          (3, 3, 128, 32), (16, 2, 128, 16), (16, 1, 128, 8), (12, 2, 128, 64)]


@pytest.mark.parametrize("H,Hkv,dh,ps", SHAPES)
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixed_batch(H, Hkv, dh, ps, window, dtype):
    """Prompt portions beside single tokens, through whichever kernel the dispatch picks."""
    extents, firsts = [70, 1, 5, 1, 130], [0, 199, 61, 0, 100]
    case = paged_case(extents, firsts, H, Hkv, dh, ps, dtype, seed=H + dh)
    scale = 1 / math.sqrt(dh)
    want = attention_ref(case, H, Hkv, dh, scale, window)
    out = torch.zeros_like(case["q"])
    attention_part().paged_attention(case["q"], out, H, Hkv, dh, Cache(case, ps), Ctx(case, False), scale,
                          window)
    assert torch.allclose(out.float().cpu(), want, **tol(dtype))
    out2 = torch.zeros_like(case["q"])
    ops().attention_generic(case["q"], out2, H, Hkv, dh, case["kc"], case["vc"], ps, case["bt"],
                            case["seq"], case["pos"], scale, window)
    assert torch.allclose(out2.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("H,Hkv,dh,ps", SHAPES)
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_split(H, Hkv, dh, ps, window):
    """Decode-only batch in bfloat16: keys cut over several CTAs and joined."""
    extents, firsts = [1, 1, 1, 1], [0, 63, 64, 700]
    case = paged_case(extents, firsts, H, Hkv, dh, ps, torch.bfloat16, seed=3)
    scale = 1 / math.sqrt(dh)
    want = attention_ref(case, H, Hkv, dh, scale, window)
    for n_splits in (1, 2, 5, 8, 16):
        out = torch.zeros_like(case["q"])
        if not ops().flash_supports(dh, H // Hkv):
            pytest.skip("no tensor-core instance for this head size")
        ops().attention_flash(case["q"], out, H, Hkv, dh, case["kc"], case["vc"], ps, case["bt"],
                              case["pos"], case["seq"], None, None, scale, window,
                              n_splits=n_splits)
        assert torch.allclose(out.float().cpu(), want, **tol(torch.bfloat16)), n_splits


@pytest.mark.parametrize("H,Hkv,ps", [(32, 8, 16), (3, 3, 32), (16, 2, 8), (16, 1, 64), (12, 2, 16)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("norm,rotate", [(True, True), (False, True), (True, False)])
def test_attention_decode_fused_equals_the_two_kernels(H, Hkv, ps, window, norm, rotate):
    """The decode kernel that norms, rotates and stores the step's own q, k and v itself gives
    the bits of qk_norm_rope_cache followed by the decode kernel: in the attention's result
    and in the cache. The requests' own positions lie at the start, the end and the middle of
    a tile of 64 keys and of a page, and in every split."""
    dh = 128
    o = ops()
    extents, firsts = [1, 1, 1, 1, 1, 1], [0, 63, 64, 700, 255, 130]
    case = paged_case(extents, firsts, H, Hkv, dh, ps, torch.bfloat16, seed=H + ps)
    T = len(extents)
    g = torch.Generator().manual_seed(5)
    qkv = (torch.randn(T, (H + 2 * Hkv) * dh, generator=g) * 2).to(torch.bfloat16).to(DEV)
    qw, kw = H * dh, Hkv * dh
    q_gain = (1 + 0.3 * torch.randn(dh, generator=g)).to(DEV) if norm else None
    k_gain = (1 + 0.3 * torch.randn(dh, generator=g)).to(DEV) if norm else None
    rope = None
    if rotate:
        inv = torch.tensor([10000.0 ** (-2 * i / dh) for i in range(dh // 2)], dtype=torch.float64, device=DEV)
        rope = o.rope_table(case["pos"], inv)
    slots = torch.empty(T, dtype=torch.int32)
    for t in range(T):
        pos = firsts[t]
        slots[t] = int(case["bt"][t, pos // ps]) * ps + pos % ps
    slots = slots.to(DEV)
    scale = 1 / math.sqrt(dh)
    # the two kernels
    a = qkv.clone()
    kc1, vc1 = case["kc"].clone(), case["vc"].clone()
    o.qk_norm_rope_cache(a[:, :qw], a[:, qw:qw + kw], a[:, qw + kw:], H, Hkv, dh, q_gain, k_gain, 1e-6,
                         rope, dh if rotate else 0, slots, kc1, vc1, ps)
    for n_splits in (1, 3, 8):
        want = torch.zeros(T, qw, dtype=torch.bfloat16, device=DEV)
        o.attention_flash(a[:, :qw], want, H, Hkv, dh, kc1, vc1, ps, case["bt"], case["pos"], case["seq"],
                          None, None, scale, window, n_splits=n_splits)
        b = qkv.clone()
        kc2, vc2 = case["kc"].clone(), case["vc"].clone()
        assert o.decode_attention_fuses(b[:, :qw], dh, H // Hkv, ps, kc2, vc2, dh if rotate else 0)
        got = torch.zeros(T, qw, dtype=torch.bfloat16, device=DEV)
        o.attention_decode_fused(b[:, :qw], b[:, qw:qw + kw], b[:, qw + kw:], got, H, Hkv, dh, q_gain,
                                 k_gain, 1e-6, rope, slots, kc2, vc2, ps, case["bt"], case["pos"],
                                 case["seq"], scale, window, n_splits=n_splits)
        bits = lambda t: t.view(torch.int16)               # unwritten rows of the cache hold NaN
        assert torch.equal(bits(kc2), bits(kc1)) and torch.equal(bits(vc2), bits(vc1)), n_splits
        assert torch.equal(bits(got), bits(want)), n_splits
        assert torch.equal(b, qkv)                         # the raw rows are left as they came
    assert o.attention_decode_tma_error() == 0


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 127, 128, 499])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dh", [64, 128])
def test_attention_far_key_stands_out(far, dtype, dh):
    """One key among 500 is made to carry nearly all the weight; a kernel that skips it (a
    tile's or a page's edge) returns something else entirely. Head size 64 goes through the
    mma.sync kernels, 128 (in bfloat16) through the tcgen05 kernel for the portion and the
    TMA-fed kernel for the single token."""
    H, Hkv, ps = 8, 2, 16

    def crafted(b, K, V):
        K *= 0.05
        K[far] = 0
        K[far, :, 0] = 30.0
        V[far] = 7.0
    case = paged_case([1, 12], [499, 488], H, Hkv, dh, ps, dtype, seed=far, crafted=crafted)
    q = torch.zeros_like(case["q"])
    q[:, 0::dh] = 8.0                       # channel 0 of every head
    case["q"] = q
    scale = 1 / math.sqrt(dh)
    out = torch.zeros_like(q)
    attention_part().paged_attention(q, out, H, Hkv, dh, Cache(case, ps), Ctx(case, False), scale, 0)
    sees = case["pos"] >= far                # rows before the far key cannot read it
    assert sees.any()
    assert torch.allclose(out[sees].float(), torch.full_like(out[sees], 7.0).float(), atol=0.05)
    out = torch.zeros_like(q[:1])
    case1 = dict(case, q=q[:1], pos=case["pos"][:1], seq=case["seq"][:1], extents=[1], firsts=[499])
    attention_part().paged_attention(q[:1], out, H, Hkv, dh, Cache(case, ps), Ctx(case1, True), scale, 0)
    assert torch.allclose(out.float(), torch.full_like(out, 7.0).float(), atol=0.05)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,dh,ps", [(4, 2, 32, 8), (8, 2, 128, 16), (32, 8, 128, 16)])
def test_attention_window_edge(dtype, H, Hkv, dh, ps):
    """The key just outside the window carries a huge score and must not be read; the key
    just inside must be. (Head size 128 in bfloat16: the TMA-fed decode kernel, and the
    tcgen05 kernel when the token comes as a portion.)"""
    W = 40
    p = 200
    for edge, expect in ((p - W, 1.0), (p - W + 1, 7.0)):
        def crafted(b, K, V, edge=edge):
            K *= 0.01
            V[:] = 1.0
            K[edge, :, 0] = 50.0
            V[edge] = 7.0
        case = paged_case([1], [p], H, Hkv, dh, ps, dtype, seed=1, crafted=crafted)
        q = torch.zeros_like(case["q"])
        q[:, 0::dh] = 8.0
        for decode in (True, False):
            out = torch.zeros_like(q)
            attention_part().paged_attention(q, out, H, Hkv, dh, Cache(case, ps), Ctx(case, decode),
                                  1 / math.sqrt(dh), W)
            assert torch.allclose(out.float(), torch.full_like(out, expect).float(), atol=0.05)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,dh,ps", [(4, 2, 32, 8), (8, 2, 128, 16), (32, 8, 128, 16), (6, 2, 64, 32)])
def test_attention_window_edge_inside_a_portion(dtype, H, Hkv, dh, ps):
    """A prompt portion of 121 tokens at positions 140..260 with a window of 40, so the
    window's start moves through the kernel's key tiles row by row. Key 170 carries a huge
    score and the value 7, every other value is 1: exactly the rows at positions 170..209
    may read it (earlier rows are before it, later rows' windows have passed it)."""
    W, first, n, edge = 40, 140, 121, 170

    def crafted(b, K, V):
        K *= 0.01
        V[:] = 1.0
        K[edge, :, 0] = 50.0
        V[edge] = 7.0
    case = paged_case([n], [first], H, Hkv, dh, ps, dtype, seed=4, crafted=crafted)
    q = torch.zeros_like(case["q"])
    q[:, 0::dh] = 8.0
    out = torch.zeros_like(q)
    attention_part().paged_attention(q, out, H, Hkv, dh, Cache(case, ps), Ctx(case, False),
                                     1 / math.sqrt(dh), W)
    pos = torch.arange(first, first + n, device=DEV)
    sees = (pos >= edge) & (pos - W + 1 <= edge)
    want = torch.where(sees, 7.0, 1.0)[:, None].expand_as(out)
    bad = (out.float() - want).abs().amax(dim=1) > 0.05
    assert not bad.any(), f"wrong at positions {pos[bad].tolist()}"


def test_attention_unusual_head_size_falls_back():
    """Head sizes without a tensor-core instance run through the generic kernel."""
    H, Hkv, dh, ps = 4, 2, 80, 16
    case = paged_case([33, 1], [0, 50], H, Hkv, dh, ps, torch.bfloat16)
    want = attention_ref(case, H, Hkv, dh, 0.1, 0)
    out = torch.zeros_like(case["q"])
    attention_part().paged_attention(case["q"], out, H, Hkv, dh, Cache(case, ps), Ctx(case, False), 0.1, 0)
    assert torch.allclose(out.float().cpu(), want, **tol(torch.bfloat16))


def test_kernels_refuse_what_they_cannot_take():
    o = ops()
    q = torch.zeros(1, 4 * 528, dtype=torch.float32, device=DEV)
    with pytest.raises(o.KernelError):
        o.qk_norm_rope_cache(q, None, None, 4, 4, 528, None, None, 1e-6, None, 0, None, None,
                             None, 0)
    with pytest.raises(o.KernelError):
        o.embed(torch.zeros(4, 4), torch.zeros(1, dtype=torch.int32), torch.zeros(1, 4))


# ------------------------------------------------------------------------ sampling


def test_argmax_lowest_id_on_ties():
    logits = torch.zeros(3, 151936, device=DEV)
    logits[0, 77] = 5.0
    logits[0, 150000] = 5.0
    logits[1, 151935] = 1.0
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    ops().argmax(logits, out)
    assert out.tolist() == [77, 151935, 0]


@pytest.mark.parametrize("V", [1000, 151936])
@pytest.mark.parametrize("policy", [dict(temperature=0.8), dict(temperature=1.3, top_k=40),
                                    dict(temperature=0.7, top_p=0.9),
                                    dict(temperature=1.0, top_k=128, top_p=0.5),
                                    dict(temperature=0.0)])
def test_sample_matches_plain(V, policy):
    import plain_qwen3 as plain
    n = 6
    logits = rnd(n, V, scale=3.0, seed=V)
    draws = [0.0, 0.13, 0.5, 0.77, 0.999, 0.31]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops().sample(logits, torch.full((n,), policy.get("temperature", 0.0), device=DEV),
                 torch.full((n,), policy.get("top_k", 0), dtype=torch.int32, device=DEV),
                 torch.full((n,), policy.get("top_p", 0.0), device=DEV),
                 torch.tensor(draws, device=DEV), out)
    host = logits.cpu().numpy()
    for r in range(n):
        ids, w, total = plain.policy_distribution(host[r], **policy)
        want = plain.walk(ids, w, total, draws[r])
        got = int(out[r])
        if got == want:
            continue
        # The device sums the weights in another order than the plain single ascending
        # float32 sum; over 150k terms the two running sums differ by about 1e-4 of the
        # total, which moves a boundary by a few ids. The chosen id must be a kept one whose
        # interval of the exact (float64) distribution lies within that distance of the draw.
        assert got in ids, f"row {r}: {got} is not a kept id"
        cdf = np.cumsum(np.asarray(w, np.float64))
        target = draws[r] * cdf[-1]
        i = ids.index(got)
        lo = cdf[i - 1] if i > 0 else 0.0
        slack = 5e-4 * cdf[-1]
        assert lo - slack <= target <= cdf[i] + slack, (r, got, want)


@pytest.mark.parametrize("V", [300, 151936])
@pytest.mark.parametrize("policy", [dict(temperature=0.8), dict(temperature=1.3, top_k=40),
                                    dict(temperature=0.7, top_p=0.9),
                                    dict(temperature=1.0, top_k=3, top_p=0.99),
                                    dict(temperature=0.0)])
def test_sample_reports_the_distribution_it_drew_from(V, policy):
    """The report of sample: the drawn token's share of the kept weights and the most likely
    alternatives, against the plain distribution in float64; rows that ask for nothing stay
    untouched, and asking changes no draw."""
    import plain_qwen3 as plain
    n = 6
    logits = rnd(n, V, scale=3.0, seed=V + 1)
    logits[2, 17] = logits[2, 5] = logits[2].max() + 1          # a tie at the top: lower id first
    draws = [0.0, 0.13, 0.5, 0.77, 0.999, 0.31]
    wants = [0, 5, 128, -1, 1, 20]
    args = (logits, torch.full((n,), policy.get("temperature", 0.0), device=DEV),
            torch.full((n,), policy.get("top_k", 0), dtype=torch.int32, device=DEV),
            torch.full((n,), policy.get("top_p", 0.0), device=DEV), torch.tensor(draws, device=DEV))
    quiet = torch.empty(n, dtype=torch.int32, device=DEV)
    ops().sample(*args, quiet)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    lp = torch.full((n,), 7.0, device=DEV)
    top_ids = torch.full((n, 128), -1, dtype=torch.int32, device=DEV)
    top_lp = torch.full((n, 128), 7.0, device=DEV)
    ops().sample(*args, out, torch.tensor(wants, dtype=torch.int32, device=DEV), lp, top_ids, top_lp)
    assert out.tolist() == quiet.tolist()
    host = logits.cpu().numpy()
    for r, w_ in enumerate(wants):
        if w_ < 0:
            assert float(lp[r]) == 7.0 and int(top_ids[r, 0]) == -1
            continue
        # the oracle's totals are float64 sums: the plain single ascending float32 sum is
        # itself 1e-4 off over 150k terms, the device's (per thread, then over the threads in
        # order) about 1e-6
        ids, w, total = plain.policy_distribution(host[r], exact_totals=True, **policy)
        got = int(out[r])
        want_lp, want_top = plain.token_logprobs(ids, w, total, got, w_, V)
        assert got in ids and np.isfinite(float(lp[r]))          # a drawn token is a kept one
        assert abs(float(lp[r]) - want_lp) < 2e-5, (r, float(lp[r]), want_lp)
        k = min(w_, V)
        got_ids, got_lp = top_ids[r, :k].tolist(), top_lp[r, :k].tolist()
        assert int(top_ids[r, k]) == -1 if k < 128 else True
        assert all(a >= b for a, b in zip(got_lp, got_lp[1:])), r
        for j, ((i, v), gi, gv) in enumerate(zip(want_top, got_ids, got_lp)):
            if v == -np.inf:
                assert gv == -np.inf and gi == i, (r, j)
            else:
                assert abs(gv - v) < 2e-5, (r, j, gv, v)
                # equal ids, but for neighbours whose float32 weights are within rounding
                assert gi == i or abs(host[r][gi] - host[r][i]) < 1e-5 * abs(host[r][i]), (r, j)
        if r == 2 and w_ >= 2 and policy.get("temperature", 0.0) > 0:
            assert got_ids[:2] == [5, 17]
        if policy.get("top_k", 0) and k >= policy["top_k"]:
            kept = min(policy["top_k"], len(ids))
            assert abs(sum(math.exp(v) for v in got_lp[:kept]) - 1) < 1e-4
            assert all(v == -np.inf for v in got_lp[kept:])


def test_logits_adjust_matches_plain():
    import plain_qwen3 as plain
    V = 500
    row = rnd(V, scale=2.0, seed=9)
    history = [3, 3, 7, 499, 3, 0]
    want = plain.penalize(row.cpu().numpy() + 0, history, rep=1.3, presence=0.5, frequency=0.25)
    want[11] += 0  # no bias on 11
    from tgo_b200.sampling.policy import Policy
    from tgo_b200.sampling.sampler import adjust_row
    pol = Policy(repetition_penalty=1.3, presence_penalty=0.5, frequency_penalty=0.25,
                 logit_bias={5: -2.0})
    base = row.cpu().numpy().copy()
    base[5] += -2.0
    want = plain.penalize(base, history, rep=1.3, presence=0.5, frequency=0.25)
    adjust_row(row, pol, history)
    assert np.allclose(row.cpu().numpy(), want, rtol=1e-6, atol=1e-6)


# ------------------------------------------------------------- weight-streaming GEMM


# at most 8 rows, 256 or more rows of W and a K that is a multiple of 2048 go to the persistent
# form (one CTA an SM, x staged in shared memory) unless x is too large for that (8 x 12288);
# the rest to the form of one CTA a 16-row tile
@pytest.mark.parametrize("M,N,K", [(1, 16, 64), (3, 50, 96), (8, 257, 224), (9, 64, 4096),
                                   (16, 100, 1000), (17, 33, 72), (40, 48, 512), (64, 130, 264),
                                   (1, 256, 2048), (5, 4099, 2048), (8, 6144, 520), (7, 300, 72),
                                   (8, 2500, 4096), (2, 1000, 12288), (8, 304, 12288),
                                   (3, 777, 6144)])
def test_gemm_skinny(M, N, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
    want = x.float() @ w.float().t()
    for dt in (torch.bfloat16, torch.float32):
        out = torch.empty(M, N, dtype=dt, device=DEV)
        ops().gemm_skinny(x, w, out)
        assert torch.allclose(out.float(), want, rtol=1e-2 if dt == torch.bfloat16 else 1e-4,
                              atol=2e-2 if dt == torch.bfloat16 else 1e-3), (M, N, K, dt)
    h = rnd(M, N, seed=3)
    h2 = h.clone()
    ops().gemm_skinny(x, w, h2, accumulate=True)
    assert torch.allclose(h2, h + want, rtol=1e-4, atol=1e-3)
    # a row's result does not depend on the rows beside it (bit for bit while the same form of
    # the kernel takes both: the two forms cut K differently)
    out_all = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops().gemm_skinny(x, w, out_all)
    out_one = torch.empty(1, N, dtype=torch.float32, device=DEV)
    ops().gemm_skinny(x[M - 1:M].contiguous(), w, out_one)
    if ops().folds_norm(M, N, K) == ops().folds_norm(1, N, K):
        assert torch.equal(out_one[0], out_all[M - 1])
    else:
        assert torch.allclose(out_one[0], out_all[M - 1], rtol=1e-4, atol=1e-3)


def interleave8(gate, up):
    f, d = gate.shape
    return torch.stack([gate.view(f // 8, 8, d), up.view(f // 8, 8, d)], dim=1).reshape(2 * f, d)


@pytest.mark.parametrize("M,f,K", [(2, 224, 64), (8, 128, 96), (16, 1000, 264), (8, 1000, 2048),
                                   (3, 688, 4096)])
def test_gemm_skinny_gated_output(M, f, K):
    """A gate/up matrix with rows interleaved in eights: the kernel applies the gate itself."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=4)
    wg = rnd(f, K, dtype=torch.bfloat16, scale=0.2, seed=5)
    wu = rnd(f, K, dtype=torch.bfloat16, scale=0.2, seed=6)
    g = (x.float() @ wg.float().t()).to(torch.bfloat16).float()
    u = (x.float() @ wu.float().t()).to(torch.bfloat16).float()
    want = g / (1 + torch.exp(-g)) * u
    w = interleave8(wg, wu).contiguous()
    out = torch.empty(M, f, dtype=torch.bfloat16, device=DEV)
    ops().gemm_skinny(x, w, out, gated=True)
    assert torch.allclose(out.float(), want, rtol=2e-2, atol=2e-2)
    # the separate kernel on the interleaved product gives the same
    gu = (x.float() @ w.float().t()).to(torch.bfloat16)
    out2 = torch.empty(M, f, dtype=torch.bfloat16, device=DEV)
    ops().swiglu(gu, out2, interleaved=True)
    assert torch.allclose(out2.float(), want, rtol=2e-2, atol=2e-2)
    # and gated_linear picks either
    got = ops().gated_linear(x, w, True)
    assert torch.allclose(got.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,N,K", [(1, 256, 2048), (5, 4099, 2048), (8, 6144, 4096), (8, 1008, 4096),
                                   (3, 304, 8192), (2, 320, 6144)])
def test_gemm_skinny_with_the_norm_folded_in(M, N, K):
    """RMSNorm of the float32 stream made while the product stages its rows: against the
    norm kernel followed by the product, and against float64."""
    o = ops()
    assert o.folds_norm(M, N, K) and not o.folds_norm(8, 4096, 12288) and not o.folds_norm(2, 64, 2048)
    assert not o.folds_norm(8, 5120, 5120) and o.folds_norm(4, 4096, 12288)
    h = rnd(M, K, scale=3.0, seed=11)
    h[M - 1, 5] = 400.0                                        # a row with its own scale
    gain = 1 + rnd(K, scale=0.2, seed=12)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=13)
    lazy = o.NormedRows(h, gain, 1e-5, torch.bfloat16)
    x = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    o.add_rmsnorm(h, None, gain, 1e-5, x)
    hd = h.double()
    exact = (hd * torch.rsqrt((hd * hd).mean(1, keepdim=True) + 1e-5) * gain.double())
    want = exact.to(torch.bfloat16).double() @ w.double().t()
    for dt in (torch.bfloat16, torch.float32):
        sep = torch.empty(M, N, dtype=dt, device=DEV)
        o.gemm_skinny(x, w, sep)
        got = torch.empty(M, N, dtype=dt, device=DEV)
        o.gemm_skinny_normed(lazy, w, got)
        # the two norms add their squares in another order: a row of x may differ by one
        # bfloat16 step in a few places
        tol = 2e-2 if dt == torch.bfloat16 else 2e-3
        assert torch.allclose(got.double(), want, rtol=tol, atol=tol * want.abs().max().item())
        assert torch.allclose(got.float(), sep.float(), rtol=tol, atol=tol * want.abs().max().item())
        assert torch.equal(o.linear(lazy, w, dt), got)          # linear folds it the same way
    assert torch.equal(lazy.rows(), x)                          # and what does not fold asks for the rows
    # a row's result does not depend on the rows beside it
    one = torch.empty(1, N, dtype=torch.float32, device=DEV)
    o.gemm_skinny_normed(o.NormedRows(h[M - 1:].contiguous(), gain, 1e-5, torch.bfloat16), w, one)
    assert torch.equal(one[0], got[M - 1])
    if N % 16 == 0:
        gated = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        o.gemm_skinny_normed(lazy, w, gated, gated=True)
        sep = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        o.gemm_skinny(x, w, sep, gated=True)
        assert torch.allclose(gated.float(), sep.float(), rtol=3e-2, atol=3e-2 * sep.float().abs().max().item())
        assert torch.equal(o.gated_linear(lazy, w, True), gated)


# ------------------------------------------------------------------ tcgen05 product


def tc_flag():
    return int(ops().gemm_tc_error_flag(DEV).item())


@pytest.mark.parametrize("M,N,K", [
    (128, 128, 64), (200, 300, 264), (700, 520, 1000), (1024, 2048, 4096), (300, 512, 2048),
    (2048, 4096, 192), (2048, 6144, 128), (130, 1001, 72), (33, 200, 264), (8, 128, 64)])
def test_gemm_tc(M, N, K):
    """The tcgen05 kernel with tails in every dimension."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=M + K)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=N + K)
    want = x.float() @ w.float().t()
    atol = 3 * 2.0 ** -8.5 * math.sqrt(K) * 0.1 + 1e-3         # float32 accumulation of exact bf16 products
    for dt in (torch.float32, torch.bfloat16):
        out = torch.zeros(M, N, dtype=dt, device=DEV)
        ops().gemm_tc(x, w, out)
        torch.cuda.synchronize()
        assert tc_flag() == 0
        if dt == torch.float32:
            assert torch.allclose(out, want, rtol=1e-4, atol=1e-3), (M, N, K)
        else:
            assert torch.allclose(out.float(), want, rtol=1e-2, atol=atol + 2e-2)
    h = rnd(M, N, seed=3)
    h2 = h.clone()
    ops().gemm_tc(x, w, h2, accumulate=True)
    assert torch.allclose(h2, h + want, rtol=1e-4, atol=1e-3) and tc_flag() == 0


@pytest.mark.parametrize("M,f,K", [(300, 512, 264), (1000, 1000, 512), (24, 256, 512), (64, 1008, 264)])
def test_gemm_tc_gated_output(M, f, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=4)
    wg = rnd(f, K, dtype=torch.bfloat16, scale=0.2, seed=5)
    wu = rnd(f, K, dtype=torch.bfloat16, scale=0.2, seed=6)
    g = (x.float() @ wg.float().t()).to(torch.bfloat16).float()
    u = (x.float() @ wu.float().t()).to(torch.bfloat16).float()
    want = g / (1 + torch.exp(-g)) * u
    out = torch.zeros(M, f, dtype=torch.bfloat16, device=DEV)
    ops().gemm_tc(x, interleave8(wg, wu).contiguous(), out, gated=True)
    torch.cuda.synchronize()
    assert tc_flag() == 0
    assert torch.allclose(out.float(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))


@pytest.mark.parametrize("rows,width", [(128, 64), (128, 144), (128, 224), (128, 256), (256, 64),
                                        (256, 96), (256, 176), (256, 240), (256, 256)])
@pytest.mark.parametrize("M", [600, 700])
def test_gemm_tc_tile_shapes(rows, width, M):
    """Every kind of tile the kernel takes, forced instead of chosen: one accumulator or two
    (128 or 256 rows), narrow, odd and full widths, with tails in rows and columns (600 rows
    leave the lower accumulator of the last tile wholly outside, 700 partly); plain, added
    and gated outputs."""
    N, K = 1008, 328
    x = rnd(M, K, dtype=torch.bfloat16, seed=M)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=width)
    want = x.float() @ w.float().t()
    ops().gemm_tc_force_tile(rows, width)
    try:
        out = torch.zeros(M, N, dtype=torch.float32, device=DEV)
        ops().gemm_tc(x, w, out)
        h = rnd(M, N, seed=3)
        h2 = h.clone()
        ops().gemm_tc(x, w, h2, accumulate=True)
        gated = torch.zeros(M, N // 2, dtype=torch.bfloat16, device=DEV)
        ops().gemm_tc(x, interleave8(w[:N // 2], w[N // 2:]).contiguous(), gated, gated=True)
        torch.cuda.synchronize()
    finally:
        ops().gemm_tc_force_tile(0, 0)
    assert tc_flag() == 0
    assert torch.allclose(out, want, rtol=1e-4, atol=1e-3)
    assert torch.allclose(h2, h + want, rtol=1e-4, atol=1e-3)
    g = want[:, :N // 2].to(torch.bfloat16).float()
    u = want[:, N // 2:].to(torch.bfloat16).float()
    act = g / (1 + torch.exp(-g)) * u
    assert torch.allclose(gated.float(), act, rtol=2e-2, atol=2e-2 * float(act.abs().max()))


@pytest.mark.parametrize("M,N,K,rows,width,parts", [
    (300, 512, 2048, 128, 256, 4),      # 6 tiles, each cut four ways
    (300, 512, 2048, 256, 128, 4),      # 8 tiles of two accumulators, cut four ways
    (2100, 2600, 1024, 128, 256, 2),    # 187 tiles: a full round, then 39 tiles cut in two
    (2100, 2600, 1024, 256, 256, 1),    # 99 tiles, fewer than SMs: no cut (148 / 99 < 2)
    (2100, 2600, 1536, 256, 176, 1),    # 135 tiles: no cut
    (1100, 2608, 1024, 256, 176, 1),    # 75 tiles: no cut
    (700, 1008, 4096, 256, 240, 8),     # 15 tiles cut eight ways (a part has 8 k-blocks at least)
    (520, 4000, 1280, 128, 112, 2)])    # 180 tiles: one round, the 32 left cut in two
def test_gemm_tc_cut_last_round(M, N, K, rows, width, parts):
    """The tiles of the last round, cut along K over the idle CTAs and joined through the
    workspace: the same results as without the cut (up to the order of float32 sums), in
    every output form, and again on a second launch (the flags went back to zero)."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=M)
    w = rnd(N - N % 16, K, dtype=torch.bfloat16, scale=0.1, seed=width)
    N = w.shape[0]
    want = x.float() @ w.float().t()
    h = rnd(M, N, seed=3)
    wgu = interleave8(w[:N // 2], w[N // 2:]).contiguous()
    got = {}
    for cut in (False, True, True):
        ops().gemm_tc_force_tile(rows, width, cut_last_round=cut)
        try:
            out = torch.zeros(M, N, dtype=torch.float32, device=DEV)
            ops().gemm_tc(x, w, out)
            h2 = h.clone()
            ops().gemm_tc(x, w, h2, accumulate=True)
            ob = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
            ops().gemm_tc(x, w, ob)
            gated = torch.zeros(M, N // 2, dtype=torch.bfloat16, device=DEV)
            ops().gemm_tc(x, wgu, gated, gated=True)
            torch.cuda.synchronize()
        finally:
            ops().gemm_tc_force_tile(0, 0)
        assert tc_flag() == 0
        if torch.cuda.get_device_properties(0).multi_processor_count == 148:
            assert ops().gemm_tc_last_plan() == (rows, width, parts if cut else 1)
        assert torch.allclose(out, want, rtol=1e-4, atol=1e-3)
        assert torch.allclose(h2, h + want, rtol=1e-4, atol=1e-3)
        if cut in got:      # the second launch with the cut: bit for bit the first
            for a, b in zip(got[cut], (out, h2, ob, gated)):
                assert torch.equal(a, b)
        got[cut] = (out, h2, ob, gated)
    assert torch.allclose(got[True][0], got[False][0], rtol=1e-5, atol=1e-4)
    assert torch.allclose(got[True][2].float(), got[False][2].float(), rtol=1e-2, atol=2e-2)
    assert torch.allclose(got[True][3].float(), got[False][3].float(), rtol=2e-2,
                          atol=2e-2 * float(got[False][3].float().abs().max()))
    flags = ops()._tc_tail_buffers(DEV)[1]
    assert int(flags.abs().sum().item()) == 0


def test_linear_picks_by_rows_and_agrees():
    """1..8 rows: the weight-streaming kernel; from TC_MIN_ROWS rows: tcgen05; between them
    the library. The same product through each differs by bfloat16 rounding only."""
    w = rnd(384, 512, dtype=torch.bfloat16, scale=0.1, seed=6)
    x = rnd(ops().TC_MIN_ROWS + 70, 512, dtype=torch.bfloat16, seed=7)
    many = ops().linear(x, w)
    mid = ops().linear(x[:40].contiguous(), w)
    few = ops().linear(x[:5].contiguous(), w)
    assert torch.allclose(many[:40].float(), mid.float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(many[:5].float(), few.float(), rtol=2e-2, atol=2e-2)
    assert tc_flag() == 0


# --------------------------------------------------------------------- attention on tcgen05


TC_CASES = [
    # extents, firsts, H, Hkv, page size, window
    ([32], [0], 4, 1, 16, 0),                               # one query tile, one key tile
    ([200], [0], 8, 2, 16, 0),                              # ragged last tile, two key tiles
    ([70, 1, 5, 1, 130], [0, 199, 61, 0, 100], 32, 8, 16, 0),      # portions beside single tokens
    ([70, 1, 5, 1, 130], [0, 199, 61, 0, 100], 32, 8, 16, 37),     # with a window
    ([300, 17], [50, 400], 3, 3, 32, 0),                    # no grouping, odd head count
    ([300], [0], 16, 1, 64, 100),                           # 16 heads a group, window over tiles
    ([513], [0], 8, 4, 128, 0),                             # a page as large as a key tile
    ([40], [1000], 8, 2, 8, 0),                             # small pages, a long context behind
    ([300, 9], [20, 0], 5, 1, 16, 0),                       # five heads a group: 25 tokens a tile, 3 rows idle
    ([200], [0], 6, 2, 32, 50),                             # three heads a group
    ([130], [70], 40, 8, 16, 0),                            # the 14B shape's heads
    ([40], [17000], 4, 1, 16, 0),                           # more pages than the on-chip table slice holds
    ([40], [17000], 4, 1, 16, 300),                         # the same behind a window
]


@pytest.mark.parametrize("extents,firsts,H,Hkv,ps,window", TC_CASES)
def test_attention_tc_prefill(extents, firsts, H, Hkv, ps, window):
    """The tcgen05 attention kernel alone (head size 128; one CTA per SM drawing items) over a
    scattered paged cache whose unwritten rows hold NaN, against the plain float32
    attention."""
    o, dh = ops(), 128
    assert o.attention_tc_supports(dh, H // Hkv, ps)
    case = paged_case(extents, firsts, H, Hkv, dh, ps, torch.bfloat16, seed=len(extents) + ps)
    scale = 1 / math.sqrt(dh)
    want = attention_ref(case, H, Hkv, dh, scale, window)
    out = torch.full_like(case["q"], float("nan"))
    tok0, ntok = attention_part().step_tiles(Ctx(case, False), 128 // (H // Hkv))
    o.attention_tc_prefill(case["q"], out, H, Hkv, dh, case["kc"], case["vc"], ps, case["bt"],
                           case["pos"], case["seq"], tok0, ntok, scale, window)
    torch.cuda.synchronize()
    assert o.attention_tc_error() == 0
    assert torch.allclose(out.float().cpu(), want, **tol(torch.bfloat16))


def test_attention_tc_far_key_and_growing_scores():
    """Head size 128 through the dispatch: one key among 700 carries nearly all the weight
    (a tile's or a page's edge would lose it), and scores that grow along the keys force the
    kernel to move its running maximum and rescale what it has summed."""
    H, Hkv, dh, ps = 8, 2, 128, 16
    for far in (0, 127, 128, 255, 256, 640, 699):
        def crafted(b, K, V, far=far):
            K *= 0.05
            K[far] = 0
            K[far, :, 0] = 30.0
            V[far] = 7.0
        case = paged_case([40], [660], H, Hkv, dh, ps, torch.bfloat16, seed=far, crafted=crafted)
        q = torch.zeros_like(case["q"])
        q[:, 0::dh] = 8.0
        case["q"] = q
        out = torch.zeros_like(q)
        attention_part().paged_attention(q, out, H, Hkv, dh, Cache(case, ps), Ctx(case, False), 1 / math.sqrt(dh), 0)
        sees = case["pos"] >= far
        assert torch.allclose(out[sees].float(), torch.full_like(out[sees], 7.0).float(), atol=0.05), far

    def ramp(b, K, V):
        n = K.shape[0]
        K[:] = 0
        K[:, :, 0] = torch.arange(n, dtype=torch.float32)[:, None] * 0.25     # later keys score higher
    case = paged_case([64], [600], H, Hkv, dh, ps, torch.bfloat16, seed=5, crafted=ramp)
    q = torch.zeros_like(case["q"])
    q[:, 0::dh] = 4.0
    case["q"] = q
    want = attention_ref(case, H, Hkv, dh, 1.0, 0)
    out = torch.zeros_like(q)
    attention_part().paged_attention(q, out, H, Hkv, dh, Cache(case, ps), Ctx(case, False), 1.0, 0)
    assert ops().attention_tc_error() == 0
    assert torch.allclose(out.float().cpu(), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("window", [0, 300])
def test_attention_decode_beyond_the_on_chip_table(window):
    """One decode token 17000 keys into its request (head size 128, pages of 16): more pages
    than the kernel keeps of the block table in shared memory, so the rest comes from global
    memory; with and without key splits."""
    H, Hkv, dh, ps = 4, 1, 128, 16
    case = paged_case([1, 1], [17000, 5], H, Hkv, dh, ps, torch.bfloat16, seed=9)
    scale = 1 / math.sqrt(dh)
    want = attention_ref(case, H, Hkv, dh, scale, window)
    for n_splits in (1, 7):
        out = torch.zeros_like(case["q"])
        ops().attention_flash(case["q"], out, H, Hkv, dh, case["kc"], case["vc"], ps, case["bt"],
                              case["pos"], case["seq"], None, None, scale, window,
                              n_splits=n_splits)
        assert torch.allclose(out.float().cpu(), want, **tol(torch.bfloat16)), n_splits
    assert ops().attention_decode_tma_error() == 0
