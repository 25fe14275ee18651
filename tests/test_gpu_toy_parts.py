"""A toy mixer with state of its own, a toy feed-forward and a toy architecture, all defined here:
they are registered, built, given random weights, stepped through the engine's step function in
portions and mixed batches, and compared with a plain loop - without a change to the package."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import random_tokens, rel_err

pytestmark = pytest.mark.gpu


def define_toy():
    from rustingstrata_b200.config import register_architecture
    from rustingstrata_b200.parts import (FeedForward, LayerCall, LayerSpec, Mixer, ModelSpec, PartSpec, StateNeed,
                                          TensorNeed, register_part)
    from rustingstrata_b200.kernels import ops

    @register_part("mixer", "toy_decay_sum", replace=True)
    class DecaySum(Mixer):
        """out_t = W s_t with s_t = decay * s_{t-1} + h_t: a recurrent mixer whose only memory is a
        fixed-size state per request (no cache pages).  Its forward loops over the batch on the host, so it
        tells the engine not to capture steps into CUDA graphs."""
        capturable = False

        def __init__(self, spec, runtime, position=None):
            super().__init__(spec, runtime)
            self.hidden, self.decay = int(spec.params["hidden"]), float(spec.params["decay"])

        def tensor_needs(self):
            return {self.spec.tensors["proj"]: TensorNeed((self.hidden, self.hidden))}

        def load(self, tensors):
            self.w = tensors[self.spec.tensors["proj"]]

        def state_need(self):
            return StateNeed(self.hidden)

        def forward(self, h, residual, ctx, call):
            hb = ctx.host
            for s in range(hb.n_seqs):                       # a request's tokens in order, state carried
                a, b = int(hb.q_start[s]), int(hb.q_start[s + 1])
                slot = int(hb.state_slots[s])
                st = call.state[slot]
                outs = []
                for t in range(a, b):
                    st.mul_(self.decay).add_(h[t].float())
                    outs.append(st.clone())
                o = torch.stack(outs).to(h.dtype)
                tmp = torch.zeros(b - a, self.hidden, device=h.device, dtype=torch.float32)
                ops.linear(o.contiguous(), self.w, tmp, b - a)
                residual[a:b] += tmp

    @register_part("feed_forward", "toy_scale", replace=True)
    class Scale(FeedForward):
        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.factor = float(spec.params["factor"])

        def forward(self, h, residual, ctx):
            residual[: ctx.n_tokens] += self.factor * h[: ctx.n_tokens].float()

    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d, where=""):
            return cls(dict(d))

    def build(cfg):
        d = cfg.d
        H, V = d["hidden_size"], d["vocab_size"]
        norm = lambda n: PartSpec("rmsnorm", {"width": H, "eps": d["eps"]}, {"weight": n})  # noqa: E731
        layers = []
        for i in range(d["layers"]):
            if i % 2 == 0:
                mixer = PartSpec("toy_decay_sum", {"hidden": H, "decay": d["decay"]}, {"proj": f"l{i}.proj"})
                pos = None
            else:                                            # the package's own attention beside the toy mixer
                mixer = PartSpec("paged_attention", {"hidden": H, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16,
                                                     "qk_norm": False, "window": None},
                                 {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
                pos = PartSpec("rope_neox", {"n_rot": 8, "base": 100.0})       # partial rotation
            ff = PartSpec("toy_scale", {"factor": 0.5}) if i == 0 else PartSpec(
                "gated_mlp", {"hidden": H, "intermediate": 40}, {k: f"l{i}.{k}" for k in ("gate_proj", "up_proj", "down_proj")})
            layers.append(LayerSpec.pre_norm(PartSpec("pre_norm", {"hidden": H}), mixer, norm(f"l{i}.n1"), ff, norm(f"l{i}.n2"), pos))
        return ModelSpec("toy", V, H, d["max_positions"], PartSpec("token_table", {"vocab": V, "width": H}, {"weight": "emb"}),
                         tuple(layers), tuple(LayerCall(i) for i in range(d["layers"])), norm("fn"),
                         PartSpec("linear", {"vocab": V, "width": H}, {"weight": "head"}))

    register_architecture("ToyDecayLM", ToyConfig, build, replace=True)


TOY = {"architectures": ["ToyDecayLM"], "vocab_size": 50, "hidden_size": 32, "layers": 3, "decay": 0.8, "eps": 1e-5,
       "max_positions": 128}


def plain_toy(w, toks):
    """The toy model as a plain loop over the whole sequence (float64)."""
    import plain_qwen3 as P
    d = TOY
    x = w["emb"][np.asarray(toks)]
    T = len(toks)
    for i in range(d["layers"]):
        h = P.rms_norm(x, w[f"l{i}.n1"], d["eps"])
        if i % 2 == 0:
            s, outs = np.zeros(d["hidden_size"]), []
            for t in range(T):
                s = d["decay"] * s + h[t]
                outs.append(s.copy())
            x = x + np.stack(outs) @ w[f"l{i}.proj"].T
        else:
            q = (h @ w[f"l{i}.q_proj"].T).reshape(T, 2, 16)
            k = (h @ w[f"l{i}.k_proj"].T).reshape(T, 1, 16)
            v = (h @ w[f"l{i}.v_proj"].T).reshape(T, 1, 16)
            q, k = P.rope_neox(q, np.arange(T), 8, 100.0), P.rope_neox(k, np.arange(T), 8, 100.0)
            x = x + P.attention_scores(q, k, v, 1).reshape(T, 32) @ w[f"l{i}.o_proj"].T
        h = P.rms_norm(x, w[f"l{i}.n2"], d["eps"])
        if i == 0:
            x = x + 0.5 * h
        else:
            x = x + (P.silu(h @ w[f"l{i}.gate_proj"].T) * (h @ w[f"l{i}.up_proj"].T)) @ w[f"l{i}.down_proj"].T
    return P.rms_norm(x, w["fn"], d["eps"]) @ w["head"].T


@pytest.mark.parametrize("dtype", ["float32"])
def test_toy_architecture_with_stateful_mixer(tmp_path, dtype):
    import plain_qwen3 as P
    from rustingstrata_b200.config import EngineConfig, unregister_architecture
    from rustingstrata_b200.engine import ModelRunner, StepEntry
    from rustingstrata_b200.models import manifest_for
    from rustingstrata_b200.parts import unregister_part
    from rustingstrata_b200.weights import write_random_model
    define_toy()
    try:
        d = str(tmp_path / "toy")
        m = manifest_for(TOY)
        assert "l0.proj" in m and "l1.q_proj" in m and "l2.proj" in m and "l0.gate_proj" not in m
        write_random_model(d, TOY, m, seed=3, std=0.15, norm_std=0.1)
        w = P.read_safetensors(os.path.join(d, "model.safetensors"))
        runner = ModelRunner.from_dir(d, EngineConfig(dtype=dtype, page_size=4, num_pages=24, max_seqs=4,
                                                      max_batch_tokens=128, max_logit_rows=128))
        assert sorted(runner.states) == [(0, "mixer"), (2, "mixer")] and len(runner.model.cache_groups) == 1   # two stateful calls, one cached
        toks = {r: random_tokens(50, n, 20 + i) for i, (r, n) in enumerate((("a", 40), ("b", 23), ("c", 31)))}
        ref = {r: plain_toy(w, t) for r, t in toks.items()}
        # a whole; b and c in portions, mixed with each other, b finishing first and its slot reused by d
        got = {r: {} for r in list(toks) + ["d"]}

        def step(entries):
            logits = runner.step([StepEntry(r, toks[r][s:s + n], list(range(n))) for r, s, n in entries]).cpu().numpy()
            runner.check_status()
            k = 0
            for r, s, n in entries:
                for i in range(n):
                    got[r][s + i] = logits[k]
                    k += 1
        step([("a", 0, 40)])
        step([("b", 0, 7), ("c", 0, 2)])
        step([("b", 7, 1), ("c", 2, 17)])
        step([("c", 19, 1), ("b", 8, 15)])
        runner.release("b")
        toks["d"], ref["d"] = toks["b"], ref["b"]
        step([("d", 0, 5), ("c", 20, 11)])                 # d takes b's state slot: it must start from zero
        step([("d", 5, 18)])
        for r in got:
            rows = np.stack([got[r][i] for i in range(len(toks[r]))])
            assert rel_err(rows, ref[r]) < 5e-6, r
        for r in ("a", "c", "d"):
            runner.release(r)
        runner.cache.check()
    finally:
        unregister_architecture("ToyDecayLM")
        unregister_part("mixer", "toy_decay_sum")
        unregister_part("feed_forward", "toy_scale")


# ----------------------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, again defined here only.

def define_routed():
    from rustingstrata_b200.config import register_architecture
    from rustingstrata_b200.parts import (FeedForward, LayerCall, LayerSpec, ModelSpec, PartSpec, PositionEncoding,
                                          TensorNeed, register_part)
    from rustingstrata_b200.kernels import ops

    @register_part("feed_forward", "toy_top1_of_n", replace=True)
    class TopOne(FeedForward):
        """Every token goes to the one expert its router logit (float32) is largest for; an expert is a matrix
        followed by SiLU.  The tokens of an expert are gathered, multiplied with the package's product and
        scattered back into the residual.  Which tokens go where is read back on the host, so steps of a model
        with this part are not captured into CUDA graphs."""
        capturable = False

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.hidden, self.n = int(spec.params["hidden"]), int(spec.params["experts"])

        def tensor_needs(self):
            needs = {self.spec.tensors["router"]: TensorNeed((self.n, self.hidden))}
            for e in range(self.n):
                needs[f"{self.spec.tensors['experts']}.{e}"] = TensorNeed((self.hidden, self.hidden))
            return needs

        def load(self, tensors):
            self.router = tensors[self.spec.tensors["router"]]
            self.experts = [tensors[f"{self.spec.tensors['experts']}.{e}"] for e in range(self.n)]

        def forward(self, h, residual, ctx):
            T = ctx.n_tokens
            logits = torch.zeros(T, self.n, device=h.device, dtype=torch.float32)
            ops.linear(h, self.router, logits, T)
            choice = logits.argmax(dim=1)
            for e in range(self.n):
                idx = torch.nonzero(choice == e).flatten()
                if idx.numel() == 0:
                    continue
                x = h[idx].contiguous()
                y = torch.zeros(idx.numel(), self.hidden, device=h.device, dtype=torch.float32)
                ops.linear(x, self.experts[e], y, idx.numel())
                residual[idx] += torch.nn.functional.silu(y)

    @register_part("position", "toy_squeezed_rope", replace=True)
    class SqueezedRope(PositionEncoding):
        """Rotation angles of position / squeeze: the same table layout as the package's rotary encoding, which is
        all the attention kernels ask of a position encoding."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.n_rot, self.base, self.squeeze = int(spec.params["n_rot"]), float(spec.params["base"]), float(spec.params["squeeze"])

        @property
        def cos_sin(self):
            return self.runtime.shared(("toy_squeezed_rope", self.n_rot, self.base, self.squeeze), self._table)

        def _table(self):
            half = self.n_rot // 2
            inv = np.power(self.base, -2.0 * np.arange(half, dtype=np.float64) / self.n_rot)
            theta = (np.arange(self.runtime.max_positions, dtype=np.float64) / self.squeeze)[:, None] * inv[None, :]
            return torch.from_numpy(np.concatenate([np.cos(theta), np.sin(theta)], axis=1).astype(np.float32)).to(self.runtime.device)

    class RoutedConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d, where=""):
            return cls(dict(d))

    def build(cfg):
        d = cfg.d
        H, V = d["hidden_size"], d["vocab_size"]
        norm = lambda n: PartSpec("rmsnorm", {"width": H, "eps": d["eps"]}, {"weight": n})  # noqa: E731
        layers = []
        for i in range(d["layers"]):
            mixer = PartSpec("paged_attention", {"hidden": H, "n_heads": 3, "n_kv_heads": 3, "head_dim": 16, "qk_norm": False,
                                                 "window": 9 if i == 1 else None},
                             {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
            pos = PartSpec("toy_squeezed_rope", {"n_rot": 16, "base": 30.0, "squeeze": 1.0 + i})
            ff = PartSpec("toy_top1_of_n", {"hidden": H, "experts": d["experts"]}, {"router": f"l{i}.router", "experts": f"l{i}.expert"})
            layers.append(LayerSpec(PartSpec("pre_norm", {"hidden": H}), {
                "mixer_norm": norm(f"l{i}.n1"), "mixer": mixer, "position": pos, "feed_forward_norm": norm(f"l{i}.n2"),
                "feed_forward": ff}))
        return ModelSpec("routed", V, H, d["max_positions"], PartSpec("token_table", {"vocab": V, "width": H}, {"weight": "emb"}),
                         tuple(layers), tuple(LayerCall(i) for i in range(d["layers"])), norm("fn"),
                         PartSpec("linear", {"vocab": V, "width": H}, {"weight": "head"}))

    register_architecture("ToyRoutedLM", RoutedConfig, build, replace=True)


ROUTED = {"architectures": ["ToyRoutedLM"], "vocab_size": 61, "hidden_size": 48, "layers": 2, "experts": 3, "eps": 1e-5,
          "max_positions": 96}


def plain_routed(w, toks):
    import plain_qwen3 as P
    d = ROUTED
    x = w["emb"][np.asarray(toks)]
    T = len(toks)
    for i in range(d["layers"]):
        h = P.rms_norm(x, w[f"l{i}.n1"], d["eps"])
        q = (h @ w[f"l{i}.q_proj"].T).reshape(T, 3, 16)
        k = (h @ w[f"l{i}.k_proj"].T).reshape(T, 3, 16)
        v = (h @ w[f"l{i}.v_proj"].T).reshape(T, 3, 16)
        pos = np.arange(T) / (1.0 + i)
        q, k = P.rope_neox(q, pos, 16, 30.0), P.rope_neox(k, pos, 16, 30.0)
        x = x + P.attention_scores(q, k, v, 3, window=9 if i == 1 else None).reshape(T, 48) @ w[f"l{i}.o_proj"].T
        h = P.rms_norm(x, w[f"l{i}.n2"], d["eps"])
        choice = np.argmax(h @ w[f"l{i}.router"].T, axis=1)
        y = np.stack([P.silu(h[t] @ w[f"l{i}.expert.{choice[t]}"].T) for t in range(T)])
        x = x + y
    return P.rms_norm(x, w["fn"], d["eps"]) @ w["head"].T


def test_toy_architecture_with_routed_feed_forward_and_its_own_position_encoding(tmp_path):
    import plain_qwen3 as P
    from rustingstrata_b200.config import EngineConfig, unregister_architecture
    from rustingstrata_b200.engine import ModelRunner, StepEntry
    from rustingstrata_b200.models import manifest_for
    from rustingstrata_b200.parts import unregister_part
    from rustingstrata_b200.weights import write_random_model
    define_routed()
    try:
        d = str(tmp_path / "routed")
        m = manifest_for(ROUTED)
        assert "l0.router" in m and "l1.expert.2" in m and "l0.gate_proj" not in m
        write_random_model(d, ROUTED, m, seed=9, std=0.2, norm_std=0.1)
        w = P.read_safetensors(os.path.join(d, "model.safetensors"))
        runner = ModelRunner.from_dir(d, EngineConfig(dtype="float32", page_size=4, num_pages=40, max_seqs=4,
                                                      max_batch_tokens=128, max_logit_rows=128))
        assert len(runner.model.cache_groups) == 2                     # all keys | a window of 9
        toks = {r: random_tokens(61, n, 40 + i) for i, (r, n) in enumerate((("a", 50), ("b", 37)))}
        ref = {r: plain_routed(w, t) for r, t in toks.items()}
        got = {r: {} for r in toks}

        def step(entries):
            logits = runner.step([StepEntry(r, toks[r][s:s + n], list(range(n))) for r, s, n in entries]).cpu().numpy()
            runner.check_status()
            k = 0
            for r, s, n in entries:
                for i in range(n):
                    got[r][s + i] = logits[k]
                    k += 1
        step([("a", 0, 21), ("b", 0, 2)])
        step([("a", 21, 1), ("b", 2, 30)])
        step([("a", 22, 28), ("b", 32, 1)])
        assert not runner.model.capturable
        for i in range(33, 37):
            step([("b", i, 1)])                                        # the same layout again and again: still run eagerly
        assert runner.graph_replays == 0
        for r in got:
            rows = np.stack([got[r][i] for i in range(len(toks[r]))])
            # a router logit that is a near-tie may fall the other way in float32; the seed is chosen so that none is
            assert rel_err(rows, ref[r]) < 5e-6, r
        for r in toks:
            runner.release(r)
        runner.cache.check()
    finally:
        unregister_architecture("ToyRoutedLM")
        unregister_part("feed_forward", "toy_top1_of_n")
        unregister_part("position", "toy_squeezed_rope")


# ----------------------------------------------------------------------------------------------------------
# Another arrangement of a layer (four norms, two mixers side by side) and a position encoding that follows a
# second stream of positions, again defined here only.

def define_sandwich():
    from rustingstrata_b200.config import register_architecture
    from rustingstrata_b200.parts import (Block, LayerCall, LayerSpec, Mixer, ModelSpec, PartSpec, PositionEncoding,
                                          StateNeed, TensorNeed, register_part)
    from rustingstrata_b200.kernels import ops

    @register_part("block", "toy_sandwich", replace=True)
    class Sandwich(Block):
        """x += post_a(attention(pre_a(x)) + count(pre_a(x)));  x += post_f(ff(pre_f(x))): a norm on either side of
        both halves (four norms), and two mixers in the first half - the package's attention and a toy that only
        keeps a per-request counter.  The halves write into a scratch stream first so that the post-norm can see
        their output alone."""
        roles = {"pre_a": "norm", "attention": "mixer", "count": "mixer", "post_a": "norm",
                 "pre_f": "norm", "ff": "feed_forward", "post_f": "norm"}
        optional = ("count",)

        def __init__(self, spec, runtime, parts):
            super().__init__(spec, runtime, parts)
            self.hidden = int(spec.params["hidden"])
            runtime.scratch("sandwich_h", runtime.max_batch_tokens, self.hidden)
            runtime.scratch("sandwich_y", runtime.max_batch_tokens, self.hidden, torch.float32)

        def forward(self, residual, ctx, call):
            T, p = ctx.n_tokens, self.parts
            h = self.runtime.get_scratch("sandwich_h")[:, : self.hidden]
            y = self.runtime.get_scratch("sandwich_y", torch.float32)[:, : self.hidden]
            self.norm_of_stream(p["pre_a"], residual, h, ctx)
            y[:T].zero_()
            p["attention"].forward(h, y, ctx, call.mixers["attention"])
            if "count" in p:
                p["count"].forward(h, y, ctx, call.mixers["count"])
            self.norm_of_stream(p["post_a"], y, h, ctx)                 # settles anything the mixers left owed to y
            residual[:T] += h[:T].float()
            self.norm_of_stream(p["pre_f"], residual, h, ctx)
            y[:T].zero_()
            p["ff"].forward(h, y, ctx)
            self.norm_of_stream(p["post_f"], y, h, ctx)
            residual[:T] += h[:T].float()

    @register_part("mixer", "toy_token_count", replace=True)
    class TokenCount(Mixer):
        """Adds gain * (tokens of the request seen so far, this one included) to every channel: its only memory is an
        int32 counter per request."""
        capturable = False

        def __init__(self, spec, runtime, position=None):
            super().__init__(spec, runtime)
            self.gain = float(spec.params["gain"])

        def state_need(self):
            return StateNeed(1, "int32")

        def forward(self, h, residual, ctx, call):
            hb = ctx.host
            assert call.state.dtype == torch.int32 and call.role == "count"
            for s in range(hb.n_seqs):
                a, b = int(hb.q_start[s]), int(hb.q_start[s + 1])
                st = call.state[int(hb.state_slots[s])]
                counts = st[0] + torch.arange(1, b - a + 1, device=st.device, dtype=torch.int32)
                residual[a:b] += self.gain * counts.float()[:, None]
                st += b - a

    @register_part("position", "toy_second_stream_rope", replace=True)
    class SecondStreamRope(PositionEncoding):
        """The package's rotation table, indexed by the request's own position stream (stream 1) instead of the
        token count: the step then carries two position values per token."""
        n_streams = 2
        stream = 1

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.n_rot, self.base = int(spec.params["n_rot"]), float(spec.params["base"])

        @property
        def cos_sin(self):
            return self.runtime.shared(("toy_second_stream_rope", self.n_rot, self.base), self._table)

        def _table(self):
            half = self.n_rot // 2
            inv = np.power(self.base, -2.0 * np.arange(half, dtype=np.float64) / self.n_rot)
            theta = np.arange(self.runtime.max_positions, dtype=np.float64)[:, None] * inv[None, :]
            return torch.from_numpy(np.concatenate([np.cos(theta), np.sin(theta)], axis=1).astype(np.float32)).to(self.runtime.device)

    class SandwichConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d, where=""):
            return cls(dict(d))

    def build(cfg):
        d = cfg.d
        H, V = d["hidden_size"], d["vocab_size"]
        norm = lambda n: PartSpec("rmsnorm", {"width": H, "eps": d["eps"]}, {"weight": n})  # noqa: E731
        layers = []
        for i in range(d["layers"]):
            att = PartSpec("paged_attention", {"hidden": H, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16, "qk_norm": False,
                                               "window": None}, {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
            parts = {"pre_a": norm(f"l{i}.pre_a"), "attention": att, "post_a": norm(f"l{i}.post_a"),
                     "pre_f": norm(f"l{i}.pre_f"), "post_f": norm(f"l{i}.post_f"),
                     "ff": PartSpec("gated_mlp", {"hidden": H, "intermediate": 24}, {k: f"l{i}.{k}" for k in ("gate_proj", "up_proj", "down_proj")}),
                     # layer 0 rotates by the token count, layer 1 by the second stream
                     "attention_position": PartSpec("rope_neox" if i == 0 else "toy_second_stream_rope", {"n_rot": 16, "base": 50.0})}
            if i == 1:
                parts["count"] = PartSpec("toy_token_count", {"gain": d["gain"]})
            layers.append(LayerSpec(PartSpec("toy_sandwich", {"hidden": H}), parts))
        return ModelSpec("sandwich", V, H, d["max_positions"], PartSpec("token_table", {"vocab": V, "width": H}, {"weight": "emb"}),
                         tuple(layers), tuple(LayerCall(i) for i in range(d["layers"])), norm("fn"),
                         PartSpec("linear", {"vocab": V, "width": H}, {"weight": "head"}))

    register_architecture("ToySandwichLM", SandwichConfig, build, replace=True)


SANDWICH = {"architectures": ["ToySandwichLM"], "vocab_size": 70, "hidden_size": 32, "layers": 2, "eps": 1e-5, "gain": 0.01,
            "max_positions": 160}


def plain_sandwich(w, toks, stream1):
    import plain_qwen3 as P
    d = SANDWICH
    x = w["emb"][np.asarray(toks)]
    T = len(toks)
    for i in range(d["layers"]):
        h = P.rms_norm(x, w[f"l{i}.pre_a"], d["eps"])
        q = (h @ w[f"l{i}.q_proj"].T).reshape(T, 2, 16)
        k = (h @ w[f"l{i}.k_proj"].T).reshape(T, 1, 16)
        v = (h @ w[f"l{i}.v_proj"].T).reshape(T, 1, 16)
        pos = np.arange(T) if i == 0 else np.asarray(stream1)
        q, k = P.rope_neox(q, pos, 16, 50.0), P.rope_neox(k, pos, 16, 50.0)
        y = P.attention_scores(q, k, v, 1).reshape(T, 32) @ w[f"l{i}.o_proj"].T
        if i == 1:
            y = y + d["gain"] * np.arange(1, T + 1)[:, None]
        x = x + P.rms_norm(y, w[f"l{i}.post_a"], d["eps"])
        h = P.rms_norm(x, w[f"l{i}.pre_f"], d["eps"])
        y = (P.silu(h @ w[f"l{i}.gate_proj"].T) * (h @ w[f"l{i}.up_proj"].T)) @ w[f"l{i}.down_proj"].T
        x = x + P.rms_norm(y, w[f"l{i}.post_f"], d["eps"])
    return P.rms_norm(x, w["fn"], d["eps"]) @ w["head"].T


def test_toy_block_with_four_norms_two_mixers_and_a_second_position_stream(tmp_path):
    import plain_qwen3 as P
    from rustingstrata_b200.config import EngineConfig, unregister_architecture
    from rustingstrata_b200.engine import ModelRunner, StepEntry, StepError
    from rustingstrata_b200.models import manifest_for
    from rustingstrata_b200.parts import unregister_part
    from rustingstrata_b200.weights import write_random_model
    define_sandwich()
    try:
        d = str(tmp_path / "sandwich")
        m = manifest_for(SANDWICH)
        assert {"l0.pre_a", "l0.post_a", "l0.pre_f", "l0.post_f", "l1.q_proj"} <= set(m)
        write_random_model(d, SANDWICH, m, seed=11, std=0.2, norm_std=0.1)
        w = P.read_safetensors(os.path.join(d, "model.safetensors"))
        runner = ModelRunner.from_dir(d, EngineConfig(dtype="float32", page_size=4, num_pages=40, max_seqs=3,
                                                      max_batch_tokens=128, max_logit_rows=128))
        assert runner.model.n_position_streams == 2
        assert sorted(runner.states) == [(1, "count")] and runner.states[(1, "count")].dtype == torch.int32
        assert sorted(runner.model.calls[1].mixers) == ["attention", "count"]
        toks = {r: random_tokens(70, n, 60 + i) for i, (r, n) in enumerate((("a", 45), ("b", 30)))}
        # the second stream: positions that stall and jump (as an encoding of rows and columns would), not the count
        stream1 = {"a": [(3 * t) % 41 + t // 7 for t in range(45)], "b": [100 - 2 * t for t in range(30)]}
        ref = {r: plain_sandwich(w, toks[r], stream1[r]) for r in toks}
        got = {r: {} for r in toks}

        def step(entries):
            logits = runner.step([StepEntry(r, toks[r][s:s + n], list(range(n)), [[p] for p in stream1[r][s:s + n]])
                                  for r, s, n in entries]).cpu().numpy()
            runner.check_status()
            k = 0
            for r, s, n in entries:
                for i in range(n):
                    got[r][s + i] = logits[k]
                    k += 1
        step([("a", 0, 19), ("b", 0, 2)])
        step([("a", 19, 1), ("b", 2, 27)])
        step([("b", 29, 1), ("a", 20, 25)])
        for r in got:
            rows = np.stack([got[r][i] for i in range(len(toks[r]))])
            assert rel_err(rows, ref[r]) < 5e-6, r
        with pytest.raises(StepError, match="stream_positions must be"):
            runner.step([StepEntry("c", [1, 2], [], [[1, 2], [3, 4]])])
        with pytest.raises(StepError, match="outside"):
            runner.step([StepEntry("c", [1, 2], [], [[1], [160]])])
        # without streams of its own a request's second stream is its token count: layer 1 then rotates like layer 0
        plain_count = plain_sandwich(w, toks["b"], list(range(30)))
        rows = runner.step([StepEntry("c", toks["b"], list(range(30)))]).cpu().numpy()
        assert rel_err(rows, plain_count) < 5e-6
        for r in ("a", "b", "c"):
            runner.release(r)
        runner.cache.check()
        # a layer description that does not fit its block is refused with the block's roles
        from rustingstrata_b200.parts import LayerSpec, PartSpec, Runtime
        from rustingstrata_b200.models.causal_lm import CausalLM
        arch_spec = runner.spec
        import dataclasses
        broken = dataclasses.replace(arch_spec, layers=(LayerSpec(PartSpec("toy_sandwich", {"hidden": 32}),
                                                                   {"pre_a": PartSpec("rmsnorm", {"width": 32, "eps": 1e-5}, {"weight": "x"}),
                                                                    "mixer": PartSpec("paged_attention", {})}),))
        with pytest.raises(ValueError, match="unknown roles: .'mixer'.*missing roles"):
            CausalLM(broken, Runtime(torch.float32, torch.device("cuda:0"), 8, 2, 2, 4, 160, 64))
    finally:
        unregister_architecture("ToySandwichLM")
        unregister_part("block", "toy_sandwich")
        unregister_part("mixer", "toy_token_count")
        unregister_part("position", "toy_second_stream_rope")


# ----------------------------------------------------------------------------------------------------------
# A position encoding that is no rotation: a bias on the attention scores, linear in the distance, defined here only.

def define_distance_bias():
    from rustingstrata_b200.config import register_architecture
    from rustingstrata_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec, PositionEncoding, register_part

    @register_part("position", "toy_distance_bias", replace=True)
    class DistanceBias(PositionEncoding):
        """score(q at i, k at j) += slope_h * (j - i) with slope_h = first / ratio^h: nothing is rotated, keys and queries
        enter the cache and the product as they are; the attention kernels add the bias."""
        chain_safe = True

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            n, first, ratio = int(spec.params["heads"]), float(spec.params["first"]), float(spec.params["ratio"])
            self._slopes = torch.tensor([first / ratio ** h for h in range(n)], dtype=torch.float32, device=runtime.device)

        @property
        def score_slopes(self):
            return self._slopes

    class BiasConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d, where=""):
            return cls(dict(d))

    def build(cfg):
        d = cfg.d
        H, V, nh = d["hidden_size"], d["vocab_size"], d["heads"]
        norm = lambda n: PartSpec("rmsnorm", {"width": H, "eps": d["eps"]}, {"weight": n})  # noqa: E731
        layers = []
        for i in range(d["layers"]):
            parts = {"mixer_norm": norm(f"l{i}.n1"), "feed_forward_norm": norm(f"l{i}.n2"),
                     "mixer": PartSpec("paged_attention", {"hidden": H, "n_heads": nh, "n_kv_heads": d["kv_heads"], "head_dim": d["head_dim"],
                                                           "qk_norm": False, "window": 37 if i == 1 else None},
                                       {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj")}),
                     "position": PartSpec("toy_distance_bias", {"heads": nh, "first": 0.5, "ratio": 2.0}),
                     "feed_forward": PartSpec("gated_mlp", {"hidden": H, "intermediate": d["ffn"]},
                                              {k: f"l{i}.{k}" for k in ("gate_proj", "up_proj", "down_proj")})}
            layers.append(LayerSpec(PartSpec("pre_norm", {"hidden": H}), parts))
        return ModelSpec("bias", V, H, d["max_positions"], PartSpec("token_table", {"vocab": V, "width": H}, {"weight": "emb"}),
                         tuple(layers), tuple(LayerCall(i) for i in range(d["layers"])), norm("fn"),
                         PartSpec("linear", {"vocab": V, "width": H}, {"weight": "head"}))

    register_architecture("ToyBiasLM", BiasConfig, build, replace=True)


BIAS = {"architectures": ["ToyBiasLM"], "vocab_size": 90, "hidden_size": 64, "layers": 2, "heads": 4, "kv_heads": 2, "head_dim": 64,
        "ffn": 96, "eps": 1e-5, "max_positions": 400}


def plain_bias(w, toks):
    import math
    import plain_qwen3 as P
    d = BIAS
    nh, nkv, hd, T = d["heads"], d["kv_heads"], d["head_dim"], len(toks)
    x = w["emb"][np.asarray(toks)]
    tq, tk = np.arange(T)[:, None], np.arange(T)[None, :]
    for i in range(d["layers"]):
        h = P.rms_norm(x, w[f"l{i}.n1"], d["eps"])
        q = (h @ w[f"l{i}.q_proj"].T).reshape(T, nh, hd)
        k = (h @ w[f"l{i}.k_proj"].T).reshape(T, nkv, hd)
        v = (h @ w[f"l{i}.v_proj"].T).reshape(T, nkv, hd)
        vis = tk <= tq
        if i == 1:
            vis &= tk > tq - 37
        o = np.zeros((T, nh, hd))
        for hh in range(nh):
            g = hh // (nh // nkv)
            s = (q[:, hh] @ k[:, g].T) / math.sqrt(hd) + (0.5 / 2.0 ** hh) * (tk - tq)
            o[:, hh] = P.softmax(np.where(vis, s, -np.inf)) @ v[:, g]
        x = x + o.reshape(T, nh * hd) @ w[f"l{i}.o_proj"].T
        h = P.rms_norm(x, w[f"l{i}.n2"], d["eps"])
        x = x + (P.silu(h @ w[f"l{i}.gate_proj"].T) * (h @ w[f"l{i}.up_proj"].T)) @ w[f"l{i}.down_proj"].T
    return P.rms_norm(x, w["fn"], d["eps"]) @ w["head"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_encoding_that_biases_scores_instead_of_rotating(tmp_path, dtype):
    """Head size 64 with pages of 16 is a shape the tensor-core attention kernels take; with a score bias the engine
    must run the CUDA-core kernels instead, in portions and in captured single-token steps across several splits."""
    import plain_qwen3 as P
    from rustingstrata_b200.config import EngineConfig, unregister_architecture
    from rustingstrata_b200.engine import ModelRunner, StepEntry
    from rustingstrata_b200.models import manifest_for
    from rustingstrata_b200.parts import unregister_part
    from rustingstrata_b200.weights import write_random_model
    define_distance_bias()
    try:
        d = str(tmp_path / "bias")
        write_random_model(d, BIAS, manifest_for(BIAS), seed=21, std=0.12, norm_std=0.1)
        w = P.read_safetensors(os.path.join(d, "model.safetensors"))
        runner = ModelRunner.from_dir(d, EngineConfig(dtype=dtype, page_size=16, num_pages=48, max_seqs=3,
                                                      max_batch_tokens=256, max_logit_rows=256))
        toks = {r: random_tokens(90, n, 70 + i) for i, (r, n) in enumerate((("a", 330), ("b", 90)))}
        ref = {r: plain_bias(w, t) for r, t in toks.items()}
        got = {r: {} for r in toks}

        def step(entries):
            logits = runner.step([StepEntry(r, toks[r][s:s + n], list(range(n))) for r, s, n in entries]).cpu().numpy()
            runner.check_status()
            k = 0
            for r, s, n in entries:
                for i in range(n):
                    got[r][s + i] = logits[k]
                    k += 1
        step([("a", 0, 200), ("b", 0, 3)])
        step([("a", 200, 110), ("b", 3, 60)])
        for i in range(20):
            step([("a", 310 + i, 1)] + ([("b", 63 + i, 1)] if True else []))
        for i in range(83, 90):
            step([("b", i, 1)])
        tol = 5e-6 if dtype == "float32" else 2e-2
        for r in got:
            rows = np.stack([got[r][i] for i in range(len(toks[r]))])
            assert rel_err(rows, ref[r]) < tol, r
        # the bias matters: without it the logits are far away
        assert runner.model.capturable and (runner.graph_replays > 10 or dtype == "float32")
        for r in toks:
            runner.release(r)
        runner.cache.check()
    finally:
        unregister_architecture("ToyBiasLM")
        unregister_part("position", "toy_distance_bias")
