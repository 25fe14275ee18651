"""A second plain implementation of the Qwen3 dense decoder: one token at a time, as the reference's host model runs.

``plain_qwen3.py`` states the model as whole-sequence matrix algebra in float64.  This file states it the way
RustingStudio/RustingStrata's own oracle computes it (``Model::step``, src/model.rs:342-364): a state that holds, per
layer, the keys and values of all earlier tokens as growing flat lists; one token in, one row of logits out; every dot
product a sum of rounded products added one after the other from zero (``iter().zip().map(a * b).sum()``,
src/weights.rs:29-36).  It was written from those source lines, not from the other file, so that a misreading of the
reference would have to be made twice to go unnoticed; tests/test_plain_step.py requires the two to agree.

``dtype=np.float32`` follows the reference's own precision: float32 values, products rounded to float32, sums
accumulated left to right in float32 (a cumulative sum is exactly that fold), the rotation angle in float64 with sine
and cosine rounded to float32.  ``dtype=np.float64`` is the same program with wide arithmetic.  No code is shared with
the package or with plain_qwen3.py; the reference's Rust cannot be compiled here, so this rests on its formulas.
"""
from __future__ import annotations

import json
import os

import numpy as np


def load(model_dir):
    """config.json and the tensors of model.safetensors as float32 arrays (BF16 and F32 storage)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    blob = open(os.path.join(model_dir, "model.safetensors"), "rb").read()
    n = int.from_bytes(blob[:8], "little")
    index = json.loads(blob[8:8 + n])
    body = memoryview(blob)[8 + n:]
    tensors = {}
    for name, meta in index.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        if meta["dtype"] == "BF16":
            halves = np.frombuffer(body[lo:hi], dtype=np.uint16)
            vals = np.zeros(halves.size, dtype=np.uint32)
            vals[:] = halves
            vals <<= 16
            arr = vals.view(np.float32)
        elif meta["dtype"] == "F32":
            arr = np.frombuffer(body[lo:hi], dtype=np.float32).copy()
        else:
            raise ValueError(f"{name}: storage type {meta['dtype']} is not read here")
        tensors[name] = arr.reshape(meta["shape"])
    return cfg, tensors


class StepModel:
    """``Model`` of src/model.rs for the qwen3 dense case: ``new_state()`` then ``step(state, token)``."""

    def __init__(self, cfg, tensors, dtype=np.float32):
        self.c = cfg
        self.dt = np.dtype(dtype)
        self.w = {k: v.astype(self.dt) for k, v in tensors.items()}
        self.hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]     # src/config.rs:299
        self.eps = self.dt.type(cfg["rms_norm_eps"])
        self.base = np.float32(cfg["rope_theta"])                                             # the reference holds an f32

    # ---- scalar helpers ------------------------------------------------------------------------------
    def fold(self, terms, axis=-1):
        """Sum of ``terms`` added one after the other from zero in this model's precision (``.sum::<f32>()``)."""
        return np.cumsum(terms, axis=axis, dtype=self.dt).take(-1, axis=axis)

    def mv(self, name, x):
        """y[r] = row_r . x for all rows (``Tensor::matvec``, src/weights.rs:29-36)."""
        return self.fold(self.w[name] * x[None, :], axis=1)

    def rms_norm(self, x, w):
        """ms = sum(v*v) / n;  s = 1 / sqrt(ms + eps);  out = v * s * w   (src/ops.rs:3-7)."""
        ms = self.fold(x * x) / self.dt.type(x.size)
        s = self.dt.type(1.0) / np.sqrt(ms + self.eps)
        return x * s * w

    def rope_neox(self, x, pos):
        """Pairs (i, i + n_rot/2) turned by theta = pos * base^(-2i/n_rot), theta in float64, sine and cosine rounded
        to float32 (src/ops.rs:36-45); n_rot is the head size for qwen3 (src/config.rs:362)."""
        n_rot = self.hd
        half = n_rot // 2
        out = x.copy()
        for i in range(half):
            theta = float(pos) * float(np.float64(self.base) ** (-2.0 * i / n_rot))
            s, c = self.dt.type(np.float32(np.sin(theta))), self.dt.type(np.float32(np.cos(theta)))
            a, b = x[i], x[i + half]
            out[i] = a * c - b * s
            out[i + half] = a * s + b * c
        return out

    def softmax(self, v):
        """m = max;  v = exp(v - m), s += v in order;  v /= s   (src/ops.rs:18-23)."""
        e = np.exp(v - np.max(v)).astype(self.dt)
        return e / self.fold(e)

    def silu(self, x):
        """x / (1 + exp(-x))   (src/ops.rs:14)."""
        return x / (self.dt.type(1.0) + np.exp(-x).astype(self.dt))

    # ---- the model -----------------------------------------------------------------------------------
    def new_state(self):
        """Per layer the keys and the values of all tokens so far, flat (``LayerState::Attn``); the next position."""
        return {"pos": 0, "layers": [{"k": [], "v": []} for _ in range(self.c["num_hidden_layers"])]}

    def embed(self, token):
        """Row ``token`` of the token table, the id clamped to the table (src/model.rs:334-339)."""
        table = self.w["model.embed_tokens.weight"]
        return table[min(int(token), table.shape[0] - 1)].copy()

    def window_of(self, il):
        """The layer's sliding window, if it has one (``c.swa[il]`` and ``c.n_swa``, src/model.rs:751-755; which
        layers slide: src/gguf.rs:511,529 from ``use_sliding_window``/``layer_types``/``max_window_layers``)."""
        c = self.c
        if not c.get("use_sliding_window"):
            return None
        kinds = c.get("layer_types")
        if kinds is not None:
            return c["sliding_window"] if kinds[il] == "sliding_attention" else None
        return c["sliding_window"] if il >= c.get("max_window_layers", 0) else None

    def attention(self, il, h, ls, pos):
        """src/model.rs:747-801 without gates, sinks or sparse cells (none of which qwen3 has)."""
        c, hd = self.c, self.hd
        nh, nkv = c["num_attention_heads"], c["num_key_value_heads"]
        p = f"model.layers.{il}.self_attn."
        win = self.window_of(il)
        cells = range(max(0, pos + 1 - win), pos + 1) if win else range(0, pos + 1)
        qg = self.mv(p + "q_proj.weight", h)
        qn, kn = self.w[p + "q_norm.weight"], self.w[p + "k_norm.weight"]
        q = np.concatenate([self.rope_neox(self.rms_norm(qg[i * hd:(i + 1) * hd], qn), pos) for i in range(nh)])
        kraw = self.mv(p + "k_proj.weight", h)
        v = self.mv(p + "v_proj.weight", h)
        k = np.concatenate([self.rope_neox(self.rms_norm(kraw[i * hd:(i + 1) * hd], kn), pos) for i in range(nkv)])
        ls["k"].append(k)                                   # kc.extend_from_slice(&k): row `pos` of the layer's cache
        ls["v"].append(v)
        scale = self.dt.type(1.0) / np.sqrt(self.dt.type(hd))
        out = np.zeros(nh * hd, dtype=self.dt)
        for i in range(nh):
            g = i // (nh // nkv)
            qh = q[i * hd:(i + 1) * hd]
            sc = np.array([self.fold(qh * ls["k"][t][g * hd:(g + 1) * hd]) * scale for t in cells], dtype=self.dt)
            pr = self.softmax(sc)
            oh = np.zeros(hd, dtype=self.dt)
            for t, pt in zip(cells, pr):                    # o += p * v, cell after cell
                oh = oh + pt * ls["v"][t][g * hd:(g + 1) * hd]
            out[i * hd:(i + 1) * hd] = oh
        return self.mv(p + "o_proj.weight", out)

    def dense_ffn(self, il, h):
        """a = silu(gate h) * (up h);  y = down a   (src/model.rs:803-811,818-820)."""
        p = f"model.layers.{il}.mlp."
        a = self.silu(self.mv(p + "gate_proj.weight", h)) * self.mv(p + "up_proj.weight", h)
        return self.mv(p + "down_proj.weight", a)

    def block(self, il, x, ls, pos):
        """x += attention(norm(x));  x += ffn(norm(x))   (src/model.rs:587-599)."""
        p = f"model.layers.{il}."
        x = x + self.attention(il, self.rms_norm(x, self.w[p + "input_layernorm.weight"]), ls, pos)
        return x + self.dense_ffn(il, self.rms_norm(x, self.w[p + "post_attention_layernorm.weight"]))

    def head(self, x):
        """Output norm, then the output matrix, or the token table when the file has none (src/model.rs:602-607)."""
        h = self.rms_norm(x, self.w["model.norm.weight"])
        name = "lm_head.weight" if "lm_head.weight" in self.w else "model.embed_tokens.weight"
        return self.mv(name, h)

    def step(self, st, token):
        """One token through every layer at the state's position; the position advances (src/model.rs:342-364)."""
        x = self.embed(token)
        pos = st["pos"]
        for il in range(self.c["num_hidden_layers"]):
            x = self.block(il, x, st["layers"][il], pos)
        st["pos"] = pos + 1
        return self.head(x)


def logits_of(cfg, tensors, tokens, dtype=np.float32):
    """Rows of logits for every token of a sequence fed one by one."""
    m = StepModel(cfg, tensors, dtype)
    st = m.new_state()
    return np.stack([m.step(st, t) for t in tokens])
