"""The plain implementation checked against hand-computed values and the structural facts the
reference's oracle tests assert (internal/oracle/*_test.go; model/graph_rig_test.go:455)."""
import math

import numpy as np

import plain_qwen3 as plain


def test_rmsnorm_by_hand():
    x = np.array([[3.0, 4.0]])
    y = plain.rmsnorm(x, np.array([2.0, 0.5]), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert np.allclose(y, [[3 / rms * 2, 4 / rms * 0.5]])
    # eps sits inside the root
    assert np.allclose(plain.rmsnorm(np.zeros((1, 2)), np.ones(2), 1e-6), 0)


def test_silu_and_linear():
    assert np.allclose(plain.silu(np.array([0.0, 1.0])), [0, 1 / (1 + math.e ** -1)])
    x, w = np.array([[1.0, 2.0]]), np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])
    assert np.allclose(plain.linear(x, w), [[1, 2, 3]])


def test_rope_half_split_equals_interleaved_after_permutation():
    """The model pairs (i, i + d/2); the reference's kernel pairs (2i, 2i+1) on channels
    permuted y[2i] = x[i], y[2i+1] = x[i + d/2] (weights/convert.go:88-125)."""
    rng = np.random.default_rng(0)
    T, H, d, theta = 5, 3, 8, 10000.0
    x = rng.normal(size=(T, H, d))
    pos = np.array([0, 1, 2, 7, 100])
    got = plain.rope_half_split(x, pos, theta)
    perm = np.empty(d, dtype=int)
    perm[0::2], perm[1::2] = np.arange(d // 2), np.arange(d // 2) + d // 2
    y = x[..., perm]
    out = np.empty_like(y)
    for i in range(d // 2):
        ang = pos * theta ** (-2.0 * i / d)
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        out[..., 2 * i] = y[..., 2 * i] * c - y[..., 2 * i + 1] * s
        out[..., 2 * i + 1] = y[..., 2 * i] * s + y[..., 2 * i + 1] * c
    assert np.allclose(got[..., perm], out)
    assert np.allclose(plain.rope_half_split(x, np.zeros(T), theta), x)       # position 0: identity
    part = plain.rope_half_split(x, pos, theta, rotary_dim=4)
    assert np.array_equal(part[..., 4:], x[..., 4:])                          # the tail is left alone


def test_attention_groups_masks_and_windows():
    rng = np.random.default_rng(1)
    T, H, Hkv, d = 6, 4, 2, 8
    q, k, v = rng.normal(size=(T, H, d)), rng.normal(size=(T, Hkv, d)), rng.normal(size=(T, Hkv, d))
    out = plain.causal_gqa_attention(q, k, v, 0.3)
    assert np.allclose(out[0, 0], v[0, 0]) and np.allclose(out[0, 3], v[0, 1])   # floor(h / 2)
    # decode equals the last row of prefill: the last row depends on nothing after it
    again = plain.causal_gqa_attention(q[:4], k[:4], v[:4], 0.3)
    assert np.allclose(out[:4], again)
    # a key in the future changes nothing before it
    k2 = k.copy()
    k2[5] += 10
    assert np.allclose(plain.causal_gqa_attention(q, k2, v, 0.3)[:5], out[:5])
    # window 2: row 5 reads keys 4 and 5 only
    w = plain.causal_gqa_attention(q, k, v, 0.3, window=2)
    s = np.array([q[5, 0] @ k[4, 0], q[5, 0] @ k[5, 0]]) * 0.3
    p = np.exp(s - s.max())
    p /= p.sum()
    assert np.allclose(w[5, 0], p[0] * v[4, 0] + p[1] * v[5, 0])
    assert np.allclose(w[:2], out[:2])


def test_norm_before_rotation_matters():
    rng = np.random.default_rng(2)
    cfg = dict(num_attention_heads=2, num_key_value_heads=1, head_dim=4, hidden_size=8,
               rms_norm_eps=1e-6, rope_theta=100.0)
    w = {"q_proj.weight": rng.normal(size=(8, 8)), "k_proj.weight": rng.normal(size=(4, 8)),
         "v_proj.weight": rng.normal(size=(4, 8)), "o_proj.weight": rng.normal(size=(8, 8)),
         "q_norm.weight": 1 + rng.normal(size=4), "k_norm.weight": 1 + rng.normal(size=4)}
    x = rng.normal(size=(5, 8))
    pos = np.arange(5)
    right = plain.attention_block(x, pos, w, "", cfg)
    q = plain.linear(x, w["q_proj.weight"]).reshape(5, 2, 4)
    k = plain.linear(x, w["k_proj.weight"]).reshape(5, 1, 4)
    v = plain.linear(x, w["v_proj.weight"]).reshape(5, 1, 4)
    q2 = plain.rmsnorm(plain.rope_half_split(q, pos, 100.0), w["q_norm.weight"], 1e-6)
    k2 = plain.rmsnorm(plain.rope_half_split(k, pos, 100.0), w["k_norm.weight"], 1e-6)
    wrong = plain.linear(plain.causal_gqa_attention(q2, k2, v, 0.5).reshape(5, 8), w["o_proj.weight"])
    assert not np.allclose(right, wrong, atol=1e-3)


def test_sampling_order_and_ties():
    assert plain.argmax_lowest(np.array([1.0, 3.0, 3.0, 2.0])) == 1
    logits = np.array([2.0, 1.0, 0.5, -1.0], dtype=np.float32)
    ids, w, total = plain.policy_distribution(logits, temperature=1.0, top_k=2)
    assert ids == [0, 1] and np.isclose(total, 1 + math.exp(-1), rtol=1e-6)
    ids, w, total = plain.policy_distribution(logits, temperature=1.0, top_p=0.6)
    assert ids == [0]                      # exp(0) / sum = 0.61 reaches 0.6 alone
    ids, w, total = plain.policy_distribution(logits, temperature=1.0, top_p=0.7)
    assert ids == [0, 1]                   # the entry that crosses the threshold is kept
    assert plain.walk([3, 7, 9], np.array([1, 1, 2], np.float32), np.float32(4), 0.49) == 7
    assert plain.walk([3, 7, 9], np.array([1, 1, 2], np.float32), np.float32(4), 0.5) == 9
    pen = plain.penalize([2.0, -2.0, 1.0], [0, 1, 1], rep=2.0, presence=0.5, frequency=0.25)
    assert np.allclose(pen, [2 / 2 - 0.75, -2 * 2 - 1.0, 1.0])
    ids, w, total = plain.policy_distribution(logits, history=[0], temperature=0.0, rep=4.0)
    assert ids == [1]                      # penalties come before the greedy branch


def test_token_logprobs_describe_the_distribution_drawn_from():
    """The rows of the reference's table of logprob tests that need no device
    (specs/030-logprobs.md section 6, logprobs_test.go:22-143)."""
    logits = np.array([2.0, 1.0, 0.5, -1.0, 1.0], dtype=np.float32)
    ids, w, total = plain.policy_distribution(logits, temperature=0.8, top_k=3)
    lp, top = plain.token_logprobs(ids, w, total, 1, 5, 5)
    e = np.exp((logits[[0, 1, 4]].astype(np.float64) - 2.0) / 0.8)
    assert abs(lp - math.log(e[1] / e.sum())) < 1e-6             # its share of the kept set
    assert [i for i, _ in top] == [0, 1, 4, 2, 3]                # ties and unkept: lower id first
    assert abs(sum(math.exp(v) for _, v in top[:3]) - 1) < 1e-6 and top[3][1] == -np.inf
    assert plain.token_logprobs(ids, w, total, 3, 0, 5) == (-np.inf, [])
    ids, w, total = plain.policy_distribution(logits, temperature=0.0)
    lp, top = plain.token_logprobs(ids, w, total, 0, 3, 5)
    assert lp == 0 and top == [(0, 0.0), (1, -np.inf), (2, -np.inf)]     # greedy: one at the argmax
    ids, w, total = plain.policy_distribution(logits, temperature=1.0)
    lp, top = plain.token_logprobs(ids, w, total, 3, 9, 5)
    z = np.exp(logits.astype(np.float64) - 2.0)
    assert abs(lp - math.log(z[3] / z.sum())) < 1e-6 and len(top) == 5


def test_tiny_forward_is_causal_and_tied(tmp_path):
    import tiny
    cfg, run = tiny.TINIES["A"]
    d = tiny.make_model_dir(tmp_path / "a", cfg, run["seed"], run["sigma"])
    c, w = plain.load_model_dir(d)
    toks = [5, 200, 17, 3, 99, 42]
    full = plain.forward(c, w, toks)
    assert full.shape == (6, 256)
    assert np.allclose(plain.forward(c, w, toks[:4]), full[:4])      # no cache, still causal
    assert "lm_head.weight" not in w


# ------------------------------------------------- the reference's own inputs and expected values
# Each test below takes its inputs and its expected numbers from the reference's oracle tests
# (internal/oracle/*_test.go), which its authors computed outside their package. Where the
# reference draws inputs from its own generator (randf) and asserts a relation rather than
# numbers, the relation is asserted here on inputs drawn here.

TOL_ULP = 4 * 2.0 ** -52          # oracle_test.go: a few units in the last place of a float64


def close(got, want, tol=TOL_ULP):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return np.all(np.abs(got - want) <= tol * np.maximum(1.0, np.abs(want)))


def test_reference_rmsnorm_vectors():
    """internal/oracle/oracle_test.go:69-77 (hand computed), :79-88 (eps inside the root),
    :90-106 (each row of width len(gain) on its own: the per-head q/k norm)."""
    x = np.array([[1.0, 2.0, 3.0, 4.0]])
    want = [0.3651483716701107, 1.4605934866804429, 0.5477225575051661, -1.4605934866804429]
    assert close(plain.rmsnorm(x, np.array([1.0, 2.0, 0.5, -1.0]), 0.0)[0], want)
    want = [0.3651483473268884, 0.7302966946537768, 1.0954450419806652, 1.4605933893075536]
    assert close(plain.rmsnorm(x, np.ones(4), 1e-6)[0], want)
    heads = np.array([[1.0, 1.0], [100.0, 100.0]])              # two heads of width 2
    assert close(plain.rmsnorm(heads, np.ones(2), 0.0), [[1, 1], [1, 1]])
    wide = plain.rmsnorm(heads.reshape(1, 4), np.ones(4), 0.0)
    assert abs(wide[0, 0] - 1) > 1e-3                           # one row of 4 would mix the heads


def test_reference_matmul_vectors():
    """internal/oracle/oracle_test.go:112-118, :120-128, :130-137. The reference multiplies
    x [m,k] by w [k,n]; `linear` takes the weight as the checkpoint stores it, [n,k]."""
    x = np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    w = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    assert close(plain.linear(x, w.T), [[22, 28], [49, 64]])
    row = np.array([[1.0, -2.0, 3.5, 0.0, 7.0]])
    assert close(plain.linear(row, np.eye(5)), row)
    w = np.array([[1.0, 10.0, 100.0], [1.0, 10.0, 100.0]])
    assert close(plain.linear(np.array([[2.0, 3.0]]), w.T), [[5, 50, 500]])


def test_reference_silu_and_swiglu_vectors():
    """internal/oracle/oracle_test.go:155-160 (values), :162-174 (saturation), :176-186
    (the gate multiplies the up branch)."""
    assert close(plain.silu(np.array([0.0, 1.0, -2.0])), [0, 0.7310585786300049, -0.2384058440442351])
    with np.errstate(over="ignore"):
        big = plain.silu(np.array([800.0, -800.0]))
    assert big[0] == 800 and big[1] == 0
    gate, up = np.array([0.0, 1.0, -2.0, 3.0]), np.array([5.0, -1.0, 2.0, 0.5])
    want = [0 * 5, 0.7310585786300049 * -1, -0.2384058440442351 * 2, 3 / (1 + math.exp(-3)) * 0.5]
    assert close(plain.silu(gate) * up, want)
    # through the feed-forward: a one-channel input of 1 makes x Wg^T = gate and x Wu^T = up
    got = plain.swiglu_mlp(np.array([[1.0]]), gate[:, None], up[:, None], np.eye(4))
    assert close(got[0], want)


def one_head(q, k, v, scale, base=None):
    """The reference's Attention(q, k, v, qSeq, 1, 1, headDim, kvLen, scale, causalBase) for
    the cases below: the queries are the last rows of a sequence whose keys are k."""
    q, k, v = (np.asarray(a, dtype=np.float64) for a in (q, k, v))
    n_q, n_k = q.shape[0], k.shape[0]
    first = n_k - n_q if base is None else base
    pad = np.zeros((first, q.shape[1]))
    out = plain.causal_gqa_attention(np.concatenate([pad, q])[:, None, :][:first + n_q],
                                     k[:first + n_q, None, :], v[:first + n_q, None, :], scale)
    return out[first:, 0, :]


def test_reference_attention_vectors():
    """internal/oracle/attention_test.go:21-35 (one key returns the value, exactly), :37-61
    (floor grouping: four query heads over two kv heads read 0,0,1,1), :194-207 (scale 0 is
    the mean of the values), :209-224 (a softmax computed by hand)."""
    got = one_head([[0.5, -2, 100]], [[1, 1, 1]], [[7, 8, 9]], 0.125)
    assert np.array_equal(got[0], [7, 8, 9])
    rng = np.random.default_rng(21)
    q, k = rng.normal(size=(2, 4, 2)), rng.normal(size=(2, 2, 2))
    v = np.empty((2, 2, 2))
    v[:, 0, :], v[:, 1, :] = 10.0, 20.0                      # the value names the kv head read
    got = plain.causal_gqa_attention(q, k, v, 0.7)[1]
    assert close(got, [[10, 10], [10, 10], [20, 20], [20, 20]], 4 * TOL_ULP)
    rng = np.random.default_rng(71)
    v = [[1, 10], [2, 20], [3, 30], [4, 40]]
    got = one_head(rng.normal(size=(1, 2)), rng.normal(size=(4, 2)), v, 0.0)
    assert close(got[0], [2.5, 25], 8 * TOL_ULP)
    got = one_head([[1, 0]], [[1, 0], [0, 1]], [[1, 2], [3, 4]], 2.0)
    e0, e1 = math.exp(2.0), math.exp(0.0)
    w0, w1 = e0 / (e0 + e1), e1 / (e0 + e1)
    assert close(got[0], [w0 * 1 + w1 * 3, w0 * 2 + w1 * 4], 4 * TOL_ULP)


def test_reference_attention_relations():
    """internal/oracle/attention_test.go:63-101 (heads of a group read the same keys),
    :103-134 (the future is masked, bit for bit), :136-149 (the first query reads only its
    own key), :151-168 (decode equals the last row of prefill)."""
    rng = np.random.default_rng(91)
    k, v = rng.normal(size=(3, 2, 3)), rng.normal(size=(3, 2, 3))
    q = np.tile(rng.normal(size=(1, 1, 3)), (3, 4, 1))
    got = plain.causal_gqa_attention(q, k, v, 0.6)[2]
    assert np.array_equal(got[0], got[1]) and np.array_equal(got[2], got[3])
    assert not np.array_equal(got[0], got[2])
    q, k, v = rng.normal(size=(3, 1, 2)), rng.normal(size=(3, 1, 2)), rng.normal(size=(3, 1, 2))
    before = plain.causal_gqa_attention(q, k, v, 0.5)
    k2, v2 = k.copy(), v.copy()
    k2[2] += 5
    v2[2] += 5
    after = plain.causal_gqa_attention(q, k2, v2, 0.5)
    assert np.array_equal(before[:2], after[:2]) and not np.array_equal(before[2], after[2])
    q, k, v = rng.normal(size=(4, 1, 3)), rng.normal(size=(4, 1, 3)), rng.normal(size=(4, 1, 3))
    assert np.array_equal(plain.causal_gqa_attention(q, k, v, 0.3)[0, 0], v[0, 0])
    q, k, v = rng.normal(size=(3, 4, 5)), rng.normal(size=(3, 2, 5)), rng.normal(size=(3, 2, 5))
    whole = plain.causal_gqa_attention(q, k, v, 0.44)
    assert np.array_equal(plain.causal_gqa_attention(q, k, v, 0.44)[2], whole[2])


def test_reference_rope_vectors():
    """internal/oracle/rope_test.go:198-215 (the angle: pair i at position m turns by
    m * base^(-2i/rotary_dim); pair 0 by m radians), :217-250 (theta divides by rotary_dim,
    not by the head's width), :170-181 (channels past rotary_dim are left alone). The
    reference's vectors are laid out for its interleaved kernel, pairs (2i, 2i+1); the same
    pairs in half-split layout are (i, i + rotary_dim/2)."""
    m, base = 2.0, 1e6
    # interleaved x = [1, 0, 1, 0]: pair 0 = (1, 0), pair 1 = (1, 0); half-split: [1, 1, 0, 0]
    got = plain.rope_half_split(np.array([[[1.0, 1.0, 0.0, 0.0]]]), np.array([2]), base)[0, 0]
    assert close([got[0], got[2]], [math.cos(m), math.sin(m)])
    theta1 = base ** -0.5
    assert close([got[1], got[3]], [math.cos(m * theta1), math.sin(m * theta1)])
    # width 8, rotary_dim 4: pair 1 turns by base^(-2/4), not base^(-2/8)
    x = np.array([[[1.0, 1.0, 0.0, 0.0, 9.0, 9.0, 9.0, 9.0]]])
    got = plain.rope_half_split(x, np.array([2]), base, rotary_dim=4)[0, 0]
    want_theta, wrong_theta = base ** (-2.0 / 4.0), base ** (-2.0 / 8.0)
    assert close([got[1], got[3]], [math.cos(m * want_theta), math.sin(m * want_theta)])
    assert abs(got[1] - math.cos(m * wrong_theta)) > 1e-6
    assert np.array_equal(got[4:], [9, 9, 9, 9])
    x = np.array([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]])
    got = plain.rope_half_split(x, np.array([9]), base, rotary_dim=4)[0, 0]
    assert got[4] == 5 and got[5] == 6 and not (got[0] == 1 and got[1] == 2)


def test_reference_rope_relations():
    """internal/oracle/rope_test.go:139-168 (a rotation keeps each pair's norm, at positions
    0, 1, 17, 512, 4095 with base 1e6), :183-196 (each row turns by its own position)."""
    rng = np.random.default_rng(5)
    rows, width, rot = 5, 8, 6
    x = rng.normal(size=(rows, 1, width))
    pos = np.array([0, 1, 17, 512, 4095])
    got = plain.rope_half_split(x, pos, 1e6, rotary_dim=rot)
    for i in range(rot // 2):
        before = x[:, 0, i] ** 2 + x[:, 0, i + rot // 2] ** 2
        after = got[:, 0, i] ** 2 + got[:, 0, i + rot // 2] ** 2
        assert close(after, before, 4 * TOL_ULP)
    same = np.tile(np.array([[[1.0, 2.0]]]), (3, 1, 1))
    got = plain.rope_half_split(same, np.array([0, 1, 1]), 1e6)
    assert np.array_equal(got[1], got[2]) and not np.array_equal(got[0], got[1])


def test_reference_sampling_vectors():
    """sample/stages_test.go:67-89 (the penalty's arithmetic, exact in float32), :93-105 (a
    negative logit is multiplied, not divided), :110-116 (zero is in the multiply branch),
    :120-130 (once per token, however often it came), :247-255 and :260-266 (ties at the edge
    of the nucleus and of top-k go to the lower id), :365-374 (greedy is one-hot), :376-380
    (argmax ties go to the lowest id)."""
    r, alpha, beta = 2.0, 0.5, 0.25
    logits = [3.0, -3.0, 0.0, 5.0]
    got = plain.penalize(logits, [0, 0, 1], rep=r, presence=alpha, frequency=beta)
    want = np.array([3 / r - alpha - beta * 2, -3 * r - alpha - beta * 1, 0.0, 5.0], dtype=np.float32)
    assert np.array_equal(np.asarray(got, dtype=np.float32), want)
    assert plain.penalize([-4.0], [0], rep=2.0)[0] == -8.0
    assert plain.penalize([0.0], [0], rep=4.0)[0] == 0.0
    assert plain.penalize([8.0], [0], rep=2.0)[0] == plain.penalize([8.0], [0, 0, 0, 0], rep=2.0)[0]
    ids, _, _ = plain.policy_distribution(np.array([1, 0, 0], np.float32), temperature=1.0, top_p=0.7)
    assert ids == [0, 1]
    ids, _, _ = plain.policy_distribution(np.array([0, 0, 0], np.float32), temperature=1.0, top_k=2)
    assert ids == [0, 1]
    ids, w, total = plain.policy_distribution(np.array([1, 9, 3], np.float32))
    assert ids == [1] and float(w[0]) == float(total)
    assert plain.argmax_lowest(np.array([2.0, 7.0, 7.0, 1.0])) == 1
    ids, _, _ = plain.policy_distribution(np.array([3, 2, 1, 0, -1], np.float32), temperature=1.0, top_k=10)
    assert ids == [0, 1, 2, 3, 4]                   # sample/stages_test.go:294-303
