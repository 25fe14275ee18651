"""The plain implementation itself: closed-form anchors from the reference's unit tests
(tests/ops.rs:4-33) and structural properties (no GPU)."""
import math

import numpy as np
import pytest

import plain_qwen3 as P
from helpers import TINY, make_model_dir, random_tokens


def test_rms_norm_closed_form():
    # rms of [3, 4] is sqrt(12.5); weights [1, 2]  (tests/ops.rs:4-10)
    out = P.rms_norm(np.array([3.0, 4.0]), np.array([1.0, 2.0]), 0.0)
    s = 1.0 / math.sqrt(12.5)
    np.testing.assert_allclose(out, [3 * s, 8 * s], rtol=1e-12)
    # eps sits inside the square root
    np.testing.assert_allclose(P.rms_norm(np.array([0.0, 0.0]), np.ones(2), 1e-6), [0.0, 0.0])
    assert P.rms_norm(np.array([1e-3, 0.0]), np.ones(2), 1e-6)[0] == pytest.approx(1e-3 / math.sqrt(5e-7 + 1e-6))


def test_rope_position_zero_is_identity_and_pairs_rotate():
    x = np.arange(8, dtype=np.float64).reshape(1, 1, 8)
    np.testing.assert_array_equal(P.rope_neox(x, [0], 8, 10000.0), x)          # tests/ops.rs:13-18
    y = P.rope_neox(np.array([[[1.0, 0.0, 0.0, 0.0]]]), [1], 4, 10000.0)[0, 0]  # tests/ops.rs:21-33
    c, s = float(np.float32(math.cos(1.0))), float(np.float32(math.sin(1.0)))
    np.testing.assert_allclose(y, [c, 0.0, s, 0.0], atol=1e-12)
    # pair (1, 3) turns by theta = pos * base^(-2/4)
    z = P.rope_neox(np.array([[[0.0, 1.0, 0.0, 0.0]]]), [3], 4, 10000.0)[0, 0]
    th = 3 * 10000.0 ** -0.5
    np.testing.assert_allclose(z, [0.0, math.cos(th), 0.0, math.sin(th)], atol=1e-7)
    # dims beyond n_rot are untouched
    w = P.rope_neox(np.ones((1, 1, 6)), [5], 4, 100.0)[0, 0]
    assert w[4] == 1.0 and w[5] == 1.0


def test_rope_scores_depend_on_distance_only():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 1, 16)), rng.standard_normal((1, 1, 16))
    a = (P.rope_neox(q, [10], 16, 1e4) * P.rope_neox(k, [7], 16, 1e4)).sum()
    b = (P.rope_neox(q, [103], 16, 1e4) * P.rope_neox(k, [100], 16, 1e4)).sum()
    assert a == pytest.approx(b, abs=1e-5)


def test_softmax_and_silu():
    s = P.softmax(np.array([[1000.0, 1000.0, -np.inf]]))
    np.testing.assert_allclose(s, [[0.5, 0.5, 0.0]])
    assert P.silu(np.array([0.0]))[0] == 0.0 and P.silu(np.array([20.0]))[0] == pytest.approx(20.0, rel=1e-8)


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(1)
    T, nq, nkv, hd = 9, 4, 2, 8
    q, k, v = rng.standard_normal((T, nq, hd)), rng.standard_normal((T, nkv, hd)), rng.standard_normal((T, nkv, hd))
    o = P.attention_scores(q, k, v, nkv)
    np.testing.assert_allclose(o[0, :2], np.broadcast_to(v[0, 0], (2, hd)))     # one visible key; heads 0,1 → kv 0
    np.testing.assert_allclose(o[0, 2:], np.broadcast_to(v[0, 1], (2, hd)))
    k2, v2 = k.copy(), v.copy()
    k2[5:], v2[5:] = 99.0, -99.0                                                # the future does not matter
    np.testing.assert_allclose(P.attention_scores(q, k2, v2, nkv)[:5], o[:5])
    ow = P.attention_scores(q, k, v, nkv, window=3)
    np.testing.assert_allclose(ow[:3], o[:3])                                   # window not yet full
    # position 6 with window 3 sees keys 4, 5, 6 only
    s = (q[6, 0] @ k[4:7, 0].T) / math.sqrt(hd)
    np.testing.assert_allclose(ow[6, 0], P.softmax(s[None])[0] @ v[4:7, 0])
    assert not np.allclose(ow[6], o[6])


def test_whole_sequence_logits_are_causal(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "B")
    cfg, w = P.read_model(d)
    toks = random_tokens(cfg["vocab_size"], 40, 3)
    full = P.forward_logits(cfg, w, toks)
    np.testing.assert_allclose(P.forward_logits(cfg, w, toks[:17]), full[:17], rtol=1e-9, atol=1e-12)
    other = list(toks)
    other[30] = (other[30] + 1) % cfg["vocab_size"]
    np.testing.assert_allclose(P.forward_logits(cfg, w, other)[:30], full[:30], rtol=1e-9, atol=1e-12)
    assert P.layer_window(cfg, 1) == 24 and P.layer_window(cfg, 0) is None


def test_window_layer_forgets_far_tokens(tmp_path):
    """With every layer sliding (window w, L layers) the logits at position t depend on tokens t-L(w-1)..t only."""
    d = make_model_dir(str(tmp_path / "m"), "A")
    cfg, w = P.read_model(d)
    cfg = dict(cfg, use_sliding_window=True, sliding_window=4, layer_types=["sliding_attention"] * 2)
    toks = random_tokens(cfg["vocab_size"], 30, 4)
    a = P.forward_logits(cfg, w, toks)
    other = list(toks)
    other[5] = (other[5] + 7) % cfg["vocab_size"]
    b = P.forward_logits(cfg, w, other)
    assert not np.allclose(a[5 + 6], b[5 + 6])       # reach of two layers: 2 * (4 - 1) = 6
    np.testing.assert_allclose(a[5 + 7:], b[5 + 7:], rtol=1e-9, atol=1e-12)


def test_tied_head_uses_the_token_table(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "A")
    cfg, w = P.read_model(d)
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w
    x = np.random.default_rng(0).standard_normal((2, cfg["hidden_size"]))
    h = P.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    np.testing.assert_allclose(P.head(x, w, cfg), h @ w["model.embed_tokens.weight"].T)


def test_greedy_takes_the_first_index_on_ties():
    assert int(np.argmax(np.array([1.0, 3.0, 3.0, 2.0]))) == 1      # what greedy_generate relies on (src/ops.rs:110-112)
