"""Plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache.

This file is the oracle of the test suite.  It shares no code with the package: it has
its own safetensors reader and one small function per part, each written from the
reference's formulas (cited as file:line of RustingStudio/RustingStrata).  The reference's
own model code (Rust, src/model.rs + src/ops.rs) cannot be compiled here (no Rust
toolchain, no crates offline), so this implementation rests on the formulas, not on a
run of the reference; the closed-form anchors of the reference's unit tests
(tests/ops.rs:4-33) are repeated in tests/test_plain.py.

Arithmetic is float64 throughout (the reference's oracle is float32 with the rotation
angle in float64, src/ops.rs:36-45); sin/cos are rounded to float32 as the reference
does.  Weights are used exactly as stored.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ----------------------------------------------------------------------------- file reading
def read_safetensors(path):
    """name → float64 ndarray.  Container layout as parsed at src/gguf.rs:207-229."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        tag = info["dtype"]
        if tag == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif tag == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif tag == "F16":
            a = np.frombuffer(raw, dtype="<f2")
        else:
            raise ValueError(f"{name}: dtype {tag} not handled by the plain reader")
        out[name] = a.astype(np.float64).reshape(info["shape"])
    return out


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ----------------------------------------------------------------------------- parts
def rms_norm(x, w, eps):
    """out_i = x_i * (1/sqrt(mean(x^2) + eps)) * w_i   (src/ops.rs:3-7); x: [..., n]."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x * (1.0 / np.sqrt(ms + eps)) * w


def silu(x):
    """x / (1 + exp(-x))   (src/ops.rs:14)."""
    return x / (1.0 + np.exp(-x))


def softmax(s):
    """Max-subtracted softmax over the last axis (src/ops.rs:18-23)."""
    m = np.max(s, axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def rope_neox(x, positions, n_rot, base):
    """Rotation of pairs (i, i + n_rot/2) by theta = pos * base^(-2i/n_rot)  (src/ops.rs:36-45).

    x: [T, heads, hd]; positions: [T].  The angle is float64; sin and cos are rounded to
    float32 before use, as in the reference.
    """
    half = n_rot // 2
    out = x.copy()
    i = np.arange(half, dtype=np.float64)
    inv = np.power(np.float64(np.float32(base)), -2.0 * i / n_rot)          # base is an f32 in the reference
    theta = np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]  # [T, half]
    s = np.sin(theta).astype(np.float32).astype(np.float64)[:, None, :]
    c = np.cos(theta).astype(np.float32).astype(np.float64)[:, None, :]
    a, b = x[..., :half], x[..., half:n_rot]
    out[..., :half] = a * c - b * s
    out[..., half:n_rot] = a * s + b * c
    return out


def attention_scores(q, k, v, n_kv_heads, window=None):
    """Causal attention of a whole sequence (src/model.rs:747-801).

    q: [T, nq, hd]; k, v: [T, nkv, hd].  Query head i reads kv head i // (nq/nkv)
    (src/model.rs:780); score = (q . k) / sqrt(hd) (src/model.rs:778,785); position t
    sees keys 0..t, or the last `window` keys t-window+1..t in a sliding layer
    (src/model.rs:751-755); softmax, then the weighted sum of values
    (src/model.rs:787-791).
    """
    T, nq, hd = q.shape
    group = nq // n_kv_heads
    scale = 1.0 / math.sqrt(hd)
    out = np.zeros_like(q)
    tq = np.arange(T)[:, None]
    tk = np.arange(T)[None, :]
    visible = tk <= tq
    if window is not None:
        visible &= tk > tq - window
    for i in range(nq):
        g = i // group
        s = (q[:, i, :] @ k[:, g, :].T) * scale
        s = np.where(visible, s, -np.inf)
        out[:, i, :] = softmax(s) @ v[:, g, :]
    return out


def attention_mixer(h, w, prefix, cfg, positions, window):
    """q/k/v projections, per-head RMSNorm on q and k with a weight shared by all heads,
    rotation, attention, output projection (src/model.rs:757-800)."""
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, base = cfg["rms_norm_eps"], cfg["rope_theta"]
    T = h.shape[0]
    q = (h @ w[prefix + "self_attn.q_proj.weight"].T).reshape(T, nq, hd)
    k = (h @ w[prefix + "self_attn.k_proj.weight"].T).reshape(T, nkv, hd)
    v = (h @ w[prefix + "self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
    q = rope_neox(rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps), positions, hd, base)
    k = rope_neox(rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps), positions, hd, base)
    o = attention_scores(q, k, v, nkv, window).reshape(T, nq * hd)
    return o @ w[prefix + "self_attn.o_proj.weight"].T


def swiglu_ffn(h, w, prefix):
    """down(silu(gate h) * (up h))   (src/model.rs:803-811,818-820)."""
    a = silu(h @ w[prefix + "mlp.gate_proj.weight"].T) * (h @ w[prefix + "mlp.up_proj.weight"].T)
    return a @ w[prefix + "mlp.down_proj.weight"].T


def block(x, w, il, cfg, positions, window):
    """x += mixer(norm(x)); x += ffn(norm(x))   (src/model.rs:587-599)."""
    p = f"model.layers.{il}."
    eps = cfg["rms_norm_eps"]
    x = x + attention_mixer(rms_norm(x, w[p + "input_layernorm.weight"], eps), w, p, cfg, positions, window)
    x = x + swiglu_ffn(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), w, p)
    return x


def embed(tokens, w):
    """Row lookup, no scale (src/model.rs:334-339)."""
    return w["model.embed_tokens.weight"][np.asarray(tokens, dtype=np.int64)]


def head(x, w, cfg):
    """Final norm, then the output matrix; the token table when tied (src/model.rs:602-607)."""
    h = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    m = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return h @ m.T


def layer_window(cfg, il):
    """The window of layer il, or None: only when use_sliding_window is set and the layer
    is listed as sliding (src/config.rs:350-353; src/gguf.rs:511,529)."""
    if not cfg.get("use_sliding_window"):
        return None
    lt = cfg.get("layer_types")
    if lt is not None:
        return cfg["sliding_window"] if lt[il] == "sliding_attention" else None
    return cfg["sliding_window"] if il >= cfg.get("max_window_layers", 0) else None


def forward_logits(cfg, w, tokens, order=None):
    """Logits [T, V] of every position of one whole sequence."""
    if "head_dim" not in cfg:
        cfg = dict(cfg, head_dim=cfg["hidden_size"] // cfg["num_attention_heads"])
    positions = np.arange(len(tokens))
    x = embed(tokens, w)
    for il in (order if order is not None else range(cfg["num_hidden_layers"])):
        x = block(x, w, il, cfg, positions, layer_window(cfg, il))
    return head(x, w, cfg)


def greedy_generate(cfg, w, prompt, n_new):
    """Argmax continuation, the first index on ties (src/ops.rs:110-112); recomputes the
    whole sequence for every token."""
    toks = list(prompt)
    for _ in range(n_new):
        logits = forward_logits(cfg, w, toks)[-1]
        toks.append(int(np.argmax(logits)))
    return toks[len(prompt):]
