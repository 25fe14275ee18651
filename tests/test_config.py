"""Configuration and architecture registry (no GPU)."""
import copy

import pytest

from helpers import TINY
from rustingstrata_b200.config import (ConfigError, Qwen3Config, register_architecture, registered_architectures,
                                       resolve_architecture, unregister_architecture)
from rustingstrata_b200.config.model_config import FULL_ATTENTION, SLIDING_ATTENTION
import rustingstrata_b200.models  # noqa: F401  registers qwen3


def cfg(name="A", **over):
    d = copy.deepcopy(TINY[name]["config"])
    d.update(over)
    return d


def test_reads_every_size_from_config():
    c = Qwen3Config.from_dict(cfg("B"))
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 96, 6, 2, 32)
    assert (c.intermediate_size, c.vocab_size, c.rms_norm_eps, c.rope_theta) == (250, 515, 1e-5, 1e6)
    assert c.tie_word_embeddings is False and c.max_position_embeddings == 512
    assert c.layer_types == (FULL_ATTENTION, SLIDING_ATTENTION, FULL_ATTENTION) and c.sliding_window == 24


def test_head_dim_defaults_to_hidden_over_heads():
    d = cfg("A")
    del d["head_dim"]
    assert Qwen3Config.from_dict(d).head_dim == 16


def test_window_ignored_unless_enabled():
    c = Qwen3Config.from_dict(cfg("A", sliding_window=8, use_sliding_window=False))
    assert c.sliding_window is None and set(c.layer_types) == {FULL_ATTENTION}


def test_max_window_layers_selects_sliding_layers():
    c = Qwen3Config.from_dict(cfg("C"))
    assert c.layer_types == (FULL_ATTENTION, SLIDING_ATTENTION) and c.sliding_window == 40


def test_rope_parameters_block_is_read():
    d = cfg("A")
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert Qwen3Config.from_dict(d).rope_theta == 12345.0


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "vocab_size", "rms_norm_eps", "max_position_embeddings",
                                 "rope_theta"])
def test_missing_required_key_is_named(key):
    d = cfg("A")
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("over, word", [
    ({"num_attention_heads": 3}, "multiple"), ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"head_dim": 15}, "even"), ({"hidden_size": "64"}, "integer"), ({"num_hidden_layers": 0}, "positive"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"use_sliding_window": True, "sliding_window": 8, "layer_types": ["full_attention"]}, "layer_types"),
])
def test_rejects_what_the_architecture_does_not_have(over, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(cfg("A", **over))


def test_round_trip_through_to_dict():
    for name in TINY:
        c = Qwen3Config.from_dict(cfg(name))
        assert Qwen3Config.from_dict(c.to_dict()) == c


def test_registry_resolves_by_architecture_and_model_type():
    a = resolve_architecture({"architectures": ["Qwen3ForCausalLM"]})
    b = resolve_architecture({"model_type": "qwen3"})
    assert a is b and a.config_class is Qwen3Config
    assert "Qwen3ForCausalLM" in registered_architectures() and "qwen3" in registered_architectures()


def test_unknown_architecture_lists_registered_names():
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    with pytest.raises(ConfigError, match="neither"):
        resolve_architecture({})


def test_register_and_unregister_another_architecture():
    class C:
        @classmethod
        def from_dict(cls, d, where=""):
            return cls()
    register_architecture("ToyForCausalLM", C, lambda c: None, aliases=("toy",))
    try:
        assert resolve_architecture({"model_type": "toy"}).config_class is C
        with pytest.raises(ValueError):
            register_architecture("toy", C, lambda c: None)
    finally:
        unregister_architecture("ToyForCausalLM")
    assert "toy" not in registered_architectures()


def test_spec_has_no_sizes_of_its_own():
    """The spec a configuration builds carries exactly the configuration's numbers."""
    for name in TINY:
        d = cfg(name)
        arch = resolve_architecture(d)
        c = arch.config_class.from_dict(d)
        spec = arch.build_spec(c)
        assert len(spec.layers) == c.num_hidden_layers and [o.layer for o in spec.order] == list(range(c.num_hidden_layers))
        for i, ls in enumerate(spec.layers):
            assert sorted(ls.parts) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm", "position"]
            p = ls.parts["mixer"].params
            assert (p["n_heads"], p["n_kv_heads"], p["head_dim"], p["eps"]) == (
                c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rms_norm_eps)
            assert p["window"] == (c.sliding_window if c.layer_types[i] == SLIDING_ATTENTION else None)
            assert ls.parts["position"].params == {"n_rot": c.head_dim, "base": c.rope_theta}
            assert ls.parts["feed_forward"].params["intermediate"] == c.intermediate_size
            assert ls.parts["mixer_norm"].params["eps"] == c.rms_norm_eps
        tied = spec.head.tensors["weight"] == spec.embedding.tensors["weight"]
        assert tied == c.tie_word_embeddings
