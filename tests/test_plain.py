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
