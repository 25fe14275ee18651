"""safetensors reading/writing, the checkpoint loader's single error, random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from helpers import TINY, make_model_dir
from rustingstrata_b200.models import manifest_for
from rustingstrata_b200.weights import (SafetensorsError, SafetensorsWriter, WeightsError, bf16_bits_to_f32,
                                        f32_to_bf16_bits, index_model_dir, load_checkpoint, read_header,
                                        write_random_model)


def rewrite(model_dir, mutate):
    """Loads a model folder's tensors as raw arrays, lets ``mutate`` edit the dict, writes it back."""
    path = os.path.join(model_dir, "model.safetensors")
    hdr = read_header(path)
    with open(path, "rb") as f:
        blob = f.read()
    tensors = {n: (e.dtype, e.shape, blob[e.begin:e.end]) for n, e in hdr.items()}
    mutate(tensors)
    w = SafetensorsWriter(path, [(n, t[0], t[1]) for n, t in tensors.items()])
    for n, t in tensors.items():
        w.write(n, np.frombuffer(t[2], dtype=np.uint8))
    w.close()


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.1415927, 1e-30, 65504.0], dtype=np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    np.testing.assert_array_equal(bf16_bits_to_f32(f32_to_bf16_bits(x)), want)


def test_writer_reader_round_trip(tmp_path):
    p = str(tmp_path / "t.safetensors")
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.arange(5, dtype=np.int32)
    w = SafetensorsWriter(p, [("a", "F32", (3, 4)), ("b", "I32", (5,))], metadata={"k": "v"})
    w.write("a", a)
    w.write("b", b)
    w.close()
    h = read_header(p)
    assert h["a"].shape == (3, 4) and h["b"].dtype == "I32"
    with open(p, "rb") as f:
        blob = f.read()
    np.testing.assert_array_equal(np.frombuffer(blob[h["a"].begin:h["a"].end], dtype="<f4").reshape(3, 4), a)


def test_truncated_and_malformed_files_are_refused(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError, match="header length"):
        read_header(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)          # 8 of 16 data bytes
    with pytest.raises(SafetensorsError, match="outside the file"):
        read_header(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="needs 12"):
        read_header(p)


def test_random_model_is_a_function_of_seed_and_name(tmp_path):
    cfg = TINY["A"]["config"]
    m = manifest_for(cfg)
    write_random_model(str(tmp_path / "x"), cfg, m, seed=5)
    write_random_model(str(tmp_path / "y"), cfg, dict(reversed(list(m.items()))), seed=5)   # other order
    write_random_model(str(tmp_path / "z"), cfg, m, seed=6)
    x = load_checkpoint(str(tmp_path / "x"), m, torch.bfloat16)
    y = load_checkpoint(str(tmp_path / "y"), m, torch.bfloat16)
    z = load_checkpoint(str(tmp_path / "z"), m, torch.bfloat16)
    for n in m:
        assert torch.equal(x[n], y[n])
    assert not torch.equal(x["model.embed_tokens.weight"], z["model.embed_tokens.weight"])
    assert json.load(open(tmp_path / "x" / "config.json"))["hidden_size"] == 64
    e = x["model.embed_tokens.weight"].float()
    assert abs(float(e.std()) - 0.02) < 0.002 and abs(float(e.mean())) < 0.002
    assert torch.equal(x["model.norm.weight"].float(), torch.ones(64))


def test_manifest_names_shapes_and_tying():
    a, b = manifest_for(TINY["A"]["config"]), manifest_for(TINY["B"]["config"])
    assert "lm_head.weight" not in a and b["lm_head.weight"].shape == (515, 96)
    assert a["model.layers.1.self_attn.q_proj.weight"].shape == (64, 64)
    assert b["model.layers.2.self_attn.k_proj.weight"].shape == (64, 96)
    assert b["model.layers.0.self_attn.q_norm.weight"].shape == (32,)
    assert b["model.layers.0.mlp.down_proj.weight"].shape == (96, 250)
    assert len(a) == 1 + 2 * 11 + 1 and len(b) == 1 + 3 * 11 + 2


def test_kept_element_types(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "A")
    m = manifest_for(TINY["A"]["config"])

    def to_f32(ts):     # store one norm weight as F32: it must stay 32-bit in the bfloat16 engine
        n = "model.norm.weight"
        vals = bf16_bits_to_f32(np.frombuffer(ts[n][2], dtype="<u2")) * np.float32(1.0001)
        ts[n] = ("F32", ts[n][1], vals.astype("<f4").tobytes())
    rewrite(d, to_f32)
    t = load_checkpoint(d, m, torch.bfloat16)
    assert t["model.norm.weight"].dtype == torch.float32
    assert abs(float(t["model.norm.weight"][0]) - 1.0001) < 1e-7           # not rounded to bfloat16
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    t32 = load_checkpoint(d, m, torch.float32)
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["model.embed_tokens.weight"], t["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "B")
    m = manifest_for(TINY["B"]["config"])

    def damage(ts):
        del ts["model.layers.1.mlp.up_proj.weight"]
        del ts["lm_head.weight"]
        ts["model.layers.9.extra.weight"] = ("BF16", (2,), b"\0" * 4)
        dt, shape, raw = ts["model.layers.0.self_attn.q_norm.weight"]
        ts["model.layers.0.self_attn.q_norm.weight"] = (dt, (16,), raw[:32])
        ts["model.norm.weight"] = ("I32", (96,), b"\0" * 384)
    rewrite(d, damage)
    with pytest.raises(WeightsError) as ei:
        load_checkpoint(d, m, torch.bfloat16)
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.self_attn.q_norm.weight"]
    assert [w[0] for w in e.wrong_type] == ["model.norm.weight"]
    text = str(e)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "file [16] vs model [32]"):
        assert word in text


def test_model_prefix_is_optional(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "A")
    m = manifest_for(TINY["A"]["config"])
    ref = load_checkpoint(d, m, torch.bfloat16)

    def strip(ts):
        for n in list(ts):
            if n.startswith("model."):
                ts[n[len("model."):]] = ts.pop(n)
    rewrite(d, strip)
    got = load_checkpoint(d, m, torch.bfloat16)
    assert all(torch.equal(ref[n], got[n]) for n in m)


def test_sharded_model_dir(tmp_path):
    d = make_model_dir(str(tmp_path / "m"), "A")
    m = manifest_for(TINY["A"]["config"])
    ref = load_checkpoint(d, m, torch.bfloat16)
    path = os.path.join(d, "model.safetensors")
    hdr = read_header(path)
    blob = open(path, "rb").read()
    names = list(hdr)
    wm = {}
    for k, part in enumerate((names[:7], names[7:])):
        fn = f"model-{k + 1:05d}-of-00002.safetensors"
        w = SafetensorsWriter(os.path.join(d, fn), [(n, hdr[n].dtype, hdr[n].shape) for n in part])
        for n in part:
            w.write(n, np.frombuffer(blob[hdr[n].begin:hdr[n].end], dtype=np.uint8))
            wm[n] = fn
        w.close()
    os.remove(path)
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    assert set(index_model_dir(d)) == set(names)
    got = load_checkpoint(d, m, torch.bfloat16)
    assert all(torch.equal(ref[n], got[n]) for n in m)


def test_missing_files_give_a_clear_error(tmp_path):
    with pytest.raises(WeightsError, match="model.safetensors"):
        load_checkpoint(str(tmp_path), manifest_for(TINY["A"]["config"]), torch.bfloat16)
