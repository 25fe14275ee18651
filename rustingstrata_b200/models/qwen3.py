"""Qwen3 dense: the one architecture of this engine, as a description in parts.

Every layer is a pre-norm block of paged attention (GQA, per-head QK RMSNorm, NEOX
rotation over the whole head) and a SiLU-gated feed-forward; no biases; the output
head is the token table when ``tie_word_embeddings``; a layer listed as
``sliding_attention`` sees the last ``sliding_window`` keys.  Formulas and tensor
names: reference src/model.rs:587-607,747-820 and the HF-name map at
src/gguf.rs:553-564 (q_proj, k_proj, v_proj, o_proj, q_norm, k_norm, gate_proj,
up_proj, down_proj, input_layernorm, post_attention_layernorm; ``norm.weight`` and
``lm_head.weight`` at src/gguf.rs:381-395).  The ``model.`` prefix follows Hugging
Face checkpoints of this architecture; the loader accepts names with or without it.
"""
from __future__ import annotations

from ..config.model_config import SLIDING_ATTENTION, Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def build_qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    H = cfg.hidden_size
    position = PartSpec("rope_neox", {"n_rot": cfg.head_dim, "base": cfg.rope_theta})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        window = cfg.sliding_window if cfg.layer_types[i] == SLIDING_ATTENTION else None
        mixer = PartSpec("paged_attention", {
            "hidden": H, "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "qk_norm": True, "eps": cfg.rms_norm_eps, "window": window, "scale": None,
        }, {
            "q_proj": p + "self_attn.q_proj.weight", "k_proj": p + "self_attn.k_proj.weight",
            "v_proj": p + "self_attn.v_proj.weight", "o_proj": p + "self_attn.o_proj.weight",
            "q_norm": p + "self_attn.q_norm.weight", "k_norm": p + "self_attn.k_norm.weight",
        })
        ff = PartSpec("gated_mlp", {"hidden": H, "intermediate": cfg.intermediate_size, "activation": cfg.hidden_act}, {
            "gate_proj": p + "mlp.gate_proj.weight", "up_proj": p + "mlp.up_proj.weight",
            "down_proj": p + "mlp.down_proj.weight",
        })
        norm = lambda name: PartSpec("rmsnorm", {"width": H, "eps": cfg.rms_norm_eps}, {"weight": p + name})  # noqa: E731
        layers.append(LayerSpec(PartSpec("pre_norm", {"hidden": H}), {
            "mixer_norm": norm("input_layernorm.weight"), "mixer": mixer, "position": position,
            "feed_forward_norm": norm("post_attention_layernorm.weight"), "feed_forward": ff}))
    embed_name = "model.embed_tokens.weight"
    return ModelSpec(
        name="qwen3", vocab_size=cfg.vocab_size, hidden_size=H, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "width": H}, {"weight": embed_name}),
        layers=tuple(layers), order=tuple(LayerCall(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"width": H, "eps": cfg.rms_norm_eps}, {"weight": "model.norm.weight"}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "width": H},
                      {"weight": embed_name if cfg.tie_word_embeddings else "lm_head.weight"}),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_spec, aliases=("qwen3",), replace=True)
