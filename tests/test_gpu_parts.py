"""Each part alone against the plain implementation's function for it, and a toy mixer with state of
its own that is registered, built and stepped without touching the package."""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from helpers import TINY, TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def runtime(dtype, max_tokens=256, page_size=4, max_positions=512):
    from rustingstrata_b200.parts import Runtime
    return Runtime(DT[dtype], torch.device(DEV), max_tokens, 8, 64, page_size, max_positions, 1024)


def dev_tensors(w, names, dtype):
    return {n: torch.from_numpy(w[n]).to(DT[dtype]).to(DEV) for n in names}


def context(rt, q_lens, starts, tables, plans_for=()):
    """A StepContext for sequences with q_lens[i] new tokens starting at position starts[i]."""
    from rustingstrata_b200.parts import HostBatch, StepContext
    S, T = len(q_lens), int(sum(q_lens))
    q_lens = np.asarray(q_lens, np.int32)
    starts = np.asarray(starts, np.int32)
    q_start = np.zeros(S + 1, np.int32)
    q_start[1:] = np.cumsum(q_lens)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, q_lens)])
    seq = np.repeat(np.arange(S), q_lens)
    hb = HostBatch(T, S, q_lens, (starts + q_lens).astype(np.int32), q_start, np.arange(S, dtype=np.int32),
                   (starts == 0).astype(np.int32), rt.page_size, [t.shape[1] for t in tables])
    ctx = StepContext(T, S, 0, d(np.zeros(T)), d(pos), d(seq), d(q_start), d(hb.kv_lens), d(hb.state_slots),
                      d(np.zeros(1)), [d(t) for t in tables], torch.zeros(1, dtype=torch.int32, device=DEV), hb)
    for part in plans_for:
        plan = part.build_plan(hb)
        ctx.plans[part.plan_key()] = {k: (d(v) if isinstance(v, np.ndarray) else v) for k, v in plan.items()}
    return ctx


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(tiny_models, dtype):
    from rustingstrata_b200.parts import PartSpec, part_class
    cfg, w = P.read_model(tiny_models["B"])
    rt = runtime(dtype)
    name = "model.layers.1.input_layernorm.weight"
    part = part_class("norm", "rmsnorm")(PartSpec("rmsnorm", {"width": 96, "eps": cfg["rms_norm_eps"]}, {"weight": name}), rt)
    assert part.tensor_needs()[name].shape == (96,) and part.tensor_needs()[name].role == "norm"
    part.load(dev_tensors(w, [name], dtype))
    x = torch.randn(10, 96, device=DEV)
    out = torch.empty(10, 96, device=DEV, dtype=DT[dtype])
    part.forward(x, out, 10)
    assert rel_err(out.float().cpu().numpy(), P.rms_norm(x.double().cpu().numpy(), w[name], cfg["rms_norm_eps"])) < (
        1e-6 if dtype == "float32" else 5e-3)


def test_rotary_table_matches_the_formula():
    from rustingstrata_b200.parts import PartSpec, part_class
    rt = runtime("float32", max_positions=300)
    part = part_class("position", "rope_neox")(PartSpec("rope_neox", {"n_rot": 48, "base": 50000.0}), rt)
    tab = part.cos_sin.cpu().numpy()
    assert tab.shape == (300, 48)
    x = np.random.default_rng(0).standard_normal((300, 1, 48))
    want = P.rope_neox(x, np.arange(300), 48, 50000.0)
    c, s = tab[:, None, :24].astype(np.float64), tab[:, None, 24:].astype(np.float64)
    got = np.concatenate([x[..., :24] * c - x[..., 24:] * s, x[..., :24] * s + x[..., 24:] * c], -1)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-12)
    again = part_class("position", "rope_neox")(PartSpec("rope_neox", {"n_rot": 48, "base": 50000.0}), rt)
    assert again.cos_sin is part.cos_sin                   # one table per parameter set


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("A", 0), ("B", 1), ("C", 1)])
def test_attention_mixer_alone(tiny_models, name, layer, dtype):
    """The mixer fed the plain implementation's normed input, in two portions and a single token."""
    from rustingstrata_b200.parts import CallInfo
    from rustingstrata_b200.config import resolve_architecture
    from rustingstrata_b200.parts import part_class
    cfg, w = P.read_model(tiny_models[name])
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.config_class.from_dict(cfg))
    ls = spec.layers[layer]
    page = TINY[name]["page_size"]
    rt = runtime(dtype, page_size=page, max_positions=cfg["max_position_embeddings"])
    pos = part_class("position", ls.parts["position"].kind)(ls.parts["position"], rt)
    mixer = part_class("mixer", ls.parts["mixer"].kind)(ls.parts["mixer"], rt, position=pos)
    mixer.load(dev_tensors(w, mixer.tensor_needs(), dtype))
    T, H = 70, cfg["hidden_size"]
    h = np.random.default_rng(5).standard_normal((T, H))
    prefix = f"model.layers.{layer}."
    want = P.attention_mixer(h, w, prefix, cfg, np.arange(T), P.layer_window(cfg, layer))
    need = mixer.cache_need()
    assert need.window == P.layer_window(cfg, layer) and (need.n_kv_heads, need.head_dim) == (
        cfg["num_key_value_heads"], cfg["head_dim"])
    n_pages = 40
    cache = torch.zeros(n_pages, 2, need.n_kv_heads, page, need.head_dim, device=DEV, dtype=DT[dtype])
    table = np.random.default_rng(1).permutation(n_pages)[: (T + page - 1) // page][None].astype(np.int32)
    call = CallInfo(index=0, layer=layer, cache_group=0, cache=cache, writes_cache=True)
    got = np.zeros((T, H))
    for start, n in ((0, 41), (41, 28), (69, 1)):
        ctx = context(rt, [n], [start], [table], plans_for=[mixer])
        hd_ = torch.from_numpy(h[start:start + n]).to(DT[dtype]).to(DEV)
        hbuf = torch.zeros(rt.max_batch_tokens, H, device=DEV, dtype=DT[dtype])
        hbuf[:n] = hd_
        res = torch.zeros(rt.max_batch_tokens, H, device=DEV)
        mixer.forward(hbuf, res, ctx, call)
        assert ctx.status.item() == 0
        got[start:start + n] = res[:n].double().cpu().numpy()
    assert rel_err(got, want) < (3e-6 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_alone(tiny_models, dtype):
    from rustingstrata_b200.parts import PartSpec, part_class
    cfg, w = P.read_model(tiny_models["B"])
    rt = runtime(dtype)
    p = "model.layers.2."
    spec = PartSpec("gated_mlp", {"hidden": 96, "intermediate": 250, "activation": "silu"},
                    {k: p + f"mlp.{k}.weight" for k in ("gate_proj", "up_proj", "down_proj")})
    ff = part_class("feed_forward", "gated_mlp")(spec, rt)
    ff.load(dev_tensors(w, ff.tensor_needs(), dtype))
    h = np.random.default_rng(2).standard_normal((33, 96))
    hbuf = torch.zeros(rt.max_batch_tokens, 96, device=DEV, dtype=DT[dtype])
    hbuf[:33] = torch.from_numpy(h).to(DT[dtype]).to(DEV)
    base = torch.randn(rt.max_batch_tokens, 96, device=DEV)
    res = base.clone()
    ff.forward(hbuf, res, context(rt, [33], [0], [np.zeros((1, 1), np.int32)]))
    want = base[:33].double().cpu().numpy() + P.swiglu_ffn(hbuf[:33].double().cpu().numpy(), w, p)
    assert rel_err(res[:33].cpu().numpy(), want) < (3e-6 if dtype == "float32" else 1e-2)
    assert torch.equal(res[33:], base[33:])
    with pytest.raises(ValueError, match="activation"):
        part_class("feed_forward", "gated_mlp")(PartSpec("gated_mlp", {"hidden": 8, "intermediate": 8, "activation": "gelu"}), rt)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_head_and_block_alone(tiny_models, dtype):
    """One whole layer (block arrangement) and the two ends of the model against the plain functions."""
    from rustingstrata_b200.config import resolve_architecture
    from rustingstrata_b200.models import CausalLM
    from rustingstrata_b200.parts import CallInfo, LayerCallInfo
    cfg, w = P.read_model(tiny_models["A"])
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.config_class.from_dict(cfg))
    rt = runtime(dtype, page_size=4, max_positions=cfg["max_position_embeddings"])
    model = CausalLM(spec, rt)
    model.load(dev_tensors(w, model.tensor_needs(), dtype))
    toks = random_tokens(cfg["vocab_size"], 50, 9)
    ctx = context(rt, [50], [0], [np.arange(13, dtype=np.int32)[None]], plans_for=[model.blocks[0].mixer])
    ctx.token_ids = torch.tensor(toks, dtype=torch.int32, device=DEV)
    res = torch.zeros(rt.max_batch_tokens, 64, device=DEV)
    model.embedding.forward(ctx, res)
    x0 = P.embed(toks, w)
    np.testing.assert_array_equal(res[:50].cpu().numpy(), x0.astype(np.float32))
    cache = torch.zeros(16, 2, 2, 4, 16, device=DEV, dtype=DT[dtype])
    model.blocks[1].forward(res, ctx, LayerCallInfo(0, 1, {"mixer": CallInfo(0, 1, "mixer", 0, cache, True)}))
    want = P.block(x0, w, 1, cfg, np.arange(50), None)
    assert rel_err(res[:50].cpu().numpy(), want) < (2e-6 if dtype == "float32" else 1e-2)
    # head: tied to the token table in this configuration
    assert model.head.weight is model.embedding.weight
    rows = torch.tensor([49, 0, 7], dtype=torch.int32, device=DEV)
    hin = torch.empty(3, 64, device=DEV, dtype=DT[dtype])
    logits = torch.empty(3, cfg["vocab_size"], device=DEV)
    x = torch.from_numpy(want.astype(np.float32)).to(DEV)
    model.final_norm.forward(x, hin, 3, rows=rows)
    model.head.forward(hin, logits, 3)
    assert rel_err(logits.cpu().numpy(), P.head(want[[49, 0, 7]], w, cfg)) < (2e-6 if dtype == "float32" else 1e-2)


def test_run_order_may_repeat_a_layer_and_share_a_cache():
    """The order in which layers run is data: a layer named twice gets a cache per call, and a call
    may read an earlier call's cache instead of writing its own."""
    import dataclasses
    from rustingstrata_b200.config import resolve_architecture
    from rustingstrata_b200.models import CausalLM
    from rustingstrata_b200.parts import LayerCall
    cfg = TINY["A"]["config"]
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.config_class.from_dict(cfg))
    spec2 = dataclasses.replace(spec, order=(LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache=1)))
    m = CausalLM(spec2, runtime("float32"))
    assert len(m.cache_groups) == 1 and m.group_calls == [[(0, "mixer"), (1, "mixer"), (2, "mixer")]]
    assert [c.mixers["mixer"].writes_cache for c in m.calls] == [True, True, True, False]
    assert m._cache_slot[(3, "mixer")] == m._cache_slot[(1, "mixer")]
    with pytest.raises(ValueError, match="earlier entry"):
        CausalLM(dataclasses.replace(spec, order=(LayerCall(0, cache=1), LayerCall(1))), runtime("float32"))
    with pytest.raises(ValueError, match="names layer"):
        CausalLM(dataclasses.replace(spec, order=(LayerCall(5),)), runtime("float32"))
