"""The plain implementation itself (no GPU): its vectorised parts against a scalar, loop-by-loop
restatement of the same formulas, and the properties the engine is later held to."""
import math

import numpy as np
import pytest

from tests.plain import qwen3_plain as P


def scalar_forward(ids, cfg, w):
    """Token by token, head by head, element by element; written as the reference's float64
    oracle is (internal/qwen3lm/lmtest/lmtest.go:165-283) but with eps and theta from the
    configuration."""
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]

    def norm(x, wt):
        ss = sum(v * v for v in x) / len(x)
        inv = 1 / math.sqrt(ss + eps)
        return [v * inv * float(wt[i]) for i, v in enumerate(x)]

    def matvec(m, x):
        return [sum(float(m[i, j]) * x[j] for j in range(len(x))) for i in range(m.shape[0])]

    def rope(v, pos):
        half = d // 2
        v = list(v)
        for i in range(half):
            ang = pos / math.pow(theta, 2 * i / d)
            c, s = math.cos(ang), math.sin(ang)
            a, b = v[i], v[i + half]
            v[i], v[i + half] = a * c - b * s, b * c + a * s
        return v

    n = len(ids)
    h = [[float(x) for x in w["model.embed_tokens.weight"][t]] for t in ids]
    for l in range(L):
        p = f"model.layers.{l}."
        q, k, v = [], [], []
        for i in range(n):
            x = norm(h[i], w[p + "input_layernorm.weight"])
            qi, ki, vi = (matvec(w[p + f"self_attn.{nm}_proj.weight"], x) for nm in "qkv")
            qi = sum((rope(norm(qi[a * d:(a + 1) * d], w[p + "self_attn.q_norm.weight"]), i) for a in range(nh)), [])
            ki = sum((rope(norm(ki[a * d:(a + 1) * d], w[p + "self_attn.k_norm.weight"]), i) for a in range(nkv)), [])
            q.append(qi), k.append(ki), v.append(vi)
        for i in range(n):
            ctx = [0.0] * (nh * d)
            for a in range(nh):
                g = a // (nh // nkv)
                sc = [sum(q[i][a * d + e] * k[j][g * d + e] for e in range(d)) / math.sqrt(d) for j in range(i + 1)]
                m = max(sc)
                ex = [math.exp(s - m) for s in sc]
                z = sum(ex)
                for j in range(i + 1):
                    for e in range(d):
                        ctx[a * d + e] += ex[j] / z * v[j][g * d + e]
            o = matvec(w[p + "self_attn.o_proj.weight"], ctx)
            h[i] = [a + b for a, b in zip(h[i], o)]
            x = norm(h[i], w[p + "post_attention_layernorm.weight"])
            gate, up = matvec(w[p + "mlp.gate_proj.weight"], x), matvec(w[p + "mlp.up_proj.weight"], x)
            act = [gt / (1 + math.exp(-gt)) * u for gt, u in zip(gate, up)]
            dn = matvec(w[p + "mlp.down_proj.weight"], act)
            h[i] = [a + b for a, b in zip(h[i], dn)]
    out = []
    head = P.head_weight(w)
    for i in range(n):
        y = norm(h[i], w["model.norm.weight"])
        out.append(matvec(head, y))
    return np.array(out)


@pytest.mark.parametrize("name", ["A", "C"])
def test_vectorised_parts_match_the_scalar_restatement(plain_models, name):
    cfg, w = plain_models[name]
    rng = np.random.default_rng(1)
    ids = rng.integers(0, cfg["vocab_size"], size=6).tolist()
    a = P.forward_logits(ids, cfg, w)
    b = scalar_forward(ids, cfg, w)
    assert np.max(np.abs(a - b)) < 1e-10 * max(1.0, np.max(np.abs(b)))


def test_logits_do_not_depend_on_later_tokens(plain_models):
    cfg, w = plain_models["B"]
    rng = np.random.default_rng(2)
    ids = rng.integers(0, cfg["vocab_size"], size=12).tolist()
    full = P.forward_logits(ids, cfg, w)
    part = P.forward_logits(ids[:7], cfg, w)
    assert np.max(np.abs(full[:7] - part)) < 1e-9


def test_rope_rotates_pairs_and_keeps_norms():
    x = np.random.default_rng(0).standard_normal((3, 2, 8))
    cos, sin = P.rope_tables(np.array([0, 5, 9]), 8, 10000.0)
    y = P.apply_rope(x, cos, sin)
    assert np.allclose(y[0], x[0])  # position 0 rotates nothing
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1))
    # pair (i, i + 4) at position 5, i = 1: angle 5 * 10000^(-2/8)
    ang = 5 * 10000.0 ** (-2 / 8)
    assert np.isclose(y[1, 0, 1], x[1, 0, 1] * math.cos(ang) - x[1, 0, 5] * math.sin(ang))
    assert np.isclose(y[1, 0, 5], x[1, 0, 5] * math.cos(ang) + x[1, 0, 1] * math.sin(ang))
    # partial rotary leaves the tail alone
    cos4, sin4 = P.rope_tables(np.array([0, 5, 9]), 4, 10000.0)
    z = P.apply_rope(x, cos4, sin4)
    assert np.array_equal(z[..., 4:], x[..., 4:]) and not np.allclose(z[1:, :, :4], x[1:, :, :4])


def test_attention_window_and_groups():
    rng = np.random.default_rng(3)
    q, k, v = rng.standard_normal((10, 4, 8)), rng.standard_normal((10, 2, 8)), rng.standard_normal((10, 2, 8))
    full = P.causal_attention(q, k, v, 0.3)
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    k2 = k.copy()
    k2[:, 1] *= 2.0
    alt = P.causal_attention(q, k2, v, 0.3)
    assert np.allclose(alt[:, :2], full[:, :2]) and not np.allclose(alt[:, 2:], full[:, 2:])
    win = P.causal_attention(q, k, v, 0.3, window=3)
    assert np.allclose(win[:3], full[:3]) and not np.allclose(win[5], full[5])
    one = P.causal_attention(q, k, v, 0.3, window=1)
    assert np.allclose(one[:, 0], v[:, 0])  # a window of one sees only itself


def test_argmax_takes_the_first_maximum_and_never_a_nan():
    assert P.argmax_first(np.array([1.0, 3.0, 3.0, 2.0])) == 1
    assert P.argmax_first(np.array([float("nan"), 1.0, float("nan"), 1.0])) == 1
    assert P.argmax_first(np.array([float("nan")] * 3)) == 0


def test_draw_is_a_pure_function_in_the_unit_interval():
    us = [P.draw01(7, i) for i in range(2000)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 1990
    assert P.draw01(7, 3) == P.draw01(7, 3) != P.draw01(8, 3)
    assert abs(np.mean(us) - 0.5) < 0.03


def test_sampler_follows_softmax_over_top_k():
    logits = np.array([math.log(3.0), 0.0, -50.0, math.log(3.0) - 1e-3], dtype=np.float32)
    counts = np.zeros(4)
    n = 4000
    for i in range(n):
        t, cand, _ = P.sample_token(logits, 1.0, 2, 0.0, seed=11, draw=i)
        counts[t] += 1
        assert cand == [0, 3]  # never outside the two likeliest
    assert abs(counts[0] / n - 0.5) < 0.03
    counts = np.zeros(4)
    for i in range(n):
        t, _, _ = P.sample_token(logits[:2], 1.0, 0, 0.0, seed=5, draw=i)
        counts[t] += 1
    assert abs(counts[0] / counts[1] - 3.0) < 0.35  # logits ln 3 apart draw 3 : 1 (qwen3/chat_test.go:32-60)
    # temperature sharpens, top_p cuts the tail
    t, cand, _ = P.sample_token(np.array([2.0, 1.0, 0.0, -1.0]), 1.0, 0, 0.6, seed=1, draw=0)
    assert cand == [0]
    t, cand, _ = P.sample_token(np.array([2.0, 1.0, 0.0, -1.0]), 1.0, 0, 0.7, seed=1, draw=0)
    assert cand == [0, 1]
    assert P.sample_token(np.array([0.0, 5.0, 1.0]), 0.0, 0, 0.0, 1, 0)[0] == 1


def test_greedy_generation_stops_without_emitting_the_stop_token(plain_models):
    cfg, w = plain_models["A"]
    ids = [3, 9, 27]
    out = P.greedy_generate(ids, 4, cfg, w)
    assert len(out) == 4
    again = P.greedy_generate(ids, 4, cfg, w, stop_ids=[out[2]])
    assert again == out[:out.index(out[2])]
