"""The two plain implementations against each other: whole-sequence float64 algebra (plain_qwen3) and the
token-at-a-time restatement of the reference's ``Model::step`` (plain_step_qwen3), written apart from the same source
lines.  In wide arithmetic they must agree to 1e-6; run in the reference's own float32, the second one shows how far
"equal to the reference" can be asked for at all."""
import numpy as np
import pytest

import plain_qwen3 as P
import plain_step_qwen3 as S
from helpers import TINY, random_tokens

N_TOKENS = 40


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_two_plain_implementations_agree(tiny_models, name):
    cfg, w = P.read_model(tiny_models[name])
    cfg2, t2 = S.load(tiny_models[name])
    assert cfg2 == cfg and sorted(t2) == sorted(w)
    for k in w:                                               # two readers, one file
        assert np.array_equal(t2[k].astype(np.float64), w[k]), k
    toks = random_tokens(cfg["vocab_size"], N_TOKENS, 31)
    whole = P.forward_logits(cfg, w, toks)
    scale = np.max(np.abs(whole))
    wide = S.logits_of(cfg2, t2, toks, np.float64)
    err64 = float(np.max(np.abs(wide - whole)) / scale)
    assert err64 <= 1e-6, f"{name}: the two float64 statements differ by {err64:.3e}"
    narrow = S.logits_of(cfg2, t2, toks, np.float32)
    assert narrow.dtype == np.float32
    err32 = float(np.max(np.abs(narrow.astype(np.float64) - whole)) / scale)
    # the reference's own arithmetic (float32, sums in order) against exact arithmetic: the floor of any comparison
    assert err32 <= 1e-5, f"{name}: float32 token-at-a-time differs by {err32:.3e}"
    assert np.array_equal(np.argmax(narrow, axis=1), np.argmax(whole, axis=1))
    print(f"{name}: float64 step vs whole {err64:.2e}; float32 step (the reference's precision) vs whole {err32:.2e}")


def test_step_model_pieces_on_closed_forms():
    """The anchors of the reference's unit tests (tests/ops.rs:4-33) on this implementation's own functions."""
    cfg = {"rms_norm_eps": 0.0, "rope_theta": 10000.0, "head_dim": 4, "hidden_size": 4, "num_attention_heads": 1}
    m = S.StepModel(cfg, {}, np.float32)
    out = m.rms_norm(np.array([3.0, 4.0], np.float32), np.array([1.0, 2.0], np.float32))
    assert np.allclose(out, [3 / np.sqrt(12.5), 8 / np.sqrt(12.5)], rtol=1e-6)
    x = np.array([1.0, 0.0, 0.0, 0.0], np.float32)
    assert np.array_equal(m.rope_neox(x, 0), x)
    r = m.rope_neox(x, 1)
    assert np.allclose(r, [np.cos(1.0), 0.0, np.sin(1.0), 0.0], atol=1e-7)
    assert np.allclose(m.softmax(np.array([1.0, 2.0, 3.0], np.float32)), np.exp([1, 2, 3]) / np.exp([1, 2, 3]).sum(), rtol=1e-6)
    assert abs(float(m.silu(np.float32(1.5))) - 1.5 / (1 + np.exp(-1.5))) < 1e-6
    # a sum in order is not a pairwise sum: 1 + 1e-8 * n stays 1 in float32 however many terms follow
    assert m.fold(np.array([1.0] + [1e-8] * 1000, np.float32)) == np.float32(1.0)
