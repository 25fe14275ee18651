"""The random-weights generator: a pure function of (seed, tensor name, element index), the same on the host and
on the device."""
import numpy as np
import pytest

from rustingstrata_b200.parts.spec import TensorNeed
from rustingstrata_b200.weights import random_init as R


def test_values_depend_on_seed_name_and_index_only():
    need = TensorNeed((300, 70))
    whole = R.draw_values(5, "model.layers.0.mlp.up_proj.weight", need, 0.02, 0.0)
    # any cut of the work gives the same elements
    parts = [R.draw_values(5, "model.layers.0.mlp.up_proj.weight", need, 0.02, 0.0, a, min(777, 21000 - a))
             for a in range(0, 21000, 777)]
    assert np.array_equal(np.concatenate(parts), whole)
    assert np.array_equal(np.concatenate(list(R.draw_tensor(5, "model.layers.0.mlp.up_proj.weight", need, 0.02, 0.0))), whole)
    # another name or another seed is another stream
    assert not np.array_equal(R.draw_values(5, "model.layers.1.mlp.up_proj.weight", need, 0.02, 0.0), whole)
    assert not np.array_equal(R.draw_values(6, "model.layers.0.mlp.up_proj.weight", need, 0.02, 0.0), whole)
    # the vectorised generator against the definition, element by element
    key, table = R.tensor_key(5, "model.layers.0.mlp.up_proj.weight"), R.normal_table()
    for i in (0, 1, 2, 69, 70, 20999):
        z = R.mix64(key + (i + 1) * R.GOLDEN)
        assert whole[i] == np.float32(0.0) + np.float32(0.02) * table[z >> 48]


def test_the_draws_look_normal():
    v = R.draw_values(0, "w", TensorNeed((1 << 20,)), 1.0, 0.0).astype(np.float64)
    assert abs(v.mean()) < 4e-3 and abs(v.std() - 1.0) < 4e-3
    assert abs(np.mean(v ** 3)) < 2e-2 and abs(np.mean(v ** 4) - 3.0) < 5e-2
    assert abs(np.mean(np.abs(v) < 1.0) - 0.6827) < 3e-3 and 4.0 < np.abs(v).max() < 4.4
    lag = np.corrcoef(v[:-1], v[1:])[0, 1]
    assert abs(lag) < 5e-3
    t = R.normal_table()
    assert t.shape == (65536,) and np.all(np.diff(t) > 0) and np.array_equal(t, -t[::-1])


def test_norm_scales_and_integer_tables():
    ones = R.draw_values(1, "model.norm.weight", TensorNeed((64,), "norm"), 0.02, 0.0)
    assert ones.dtype == np.float32 and np.all(ones == 1.0)
    n = R.draw_values(1, "model.norm.weight", TensorNeed((4096,), "norm"), 0.02, 0.1)
    assert abs(n.mean() - 1.0) < 1e-2 and abs(n.std() - 0.1) < 1e-2
    bits = R.draw_values(1, "table", TensorNeed((4096,), "int_table"), 0.02, 0.0)
    assert bits.dtype == np.int32 and set(np.unique(bits)) == {0, 1} and abs(bits.mean() - 0.5) < 0.05


def test_writing_a_model_folder_needs_no_kernel_library(tmp_path, monkeypatch):
    """``init-random`` is a host-side command: naming the tensors of a configuration and drawing them must not build
    or load a CUDA library (a part that asked a kernel about its tiling while it was being put together once did)."""
    from rustingstrata_b200.kernels import build
    from rustingstrata_b200.models import manifest_for

    def refuse(name, verbose=True):
        raise AssertionError(f"kernel library '{name}' asked for on a host-only path")
    monkeypatch.setattr(build, "compile_library", refuse)
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 96, "hidden_size": 64,
           "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
           "intermediate_size": 80, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 128,
           "tie_word_embeddings": False, "torch_dtype": "bfloat16"}
    m = manifest_for(cfg)
    assert len(m) == 3 + 2 * 11
    R.write_random_model(str(tmp_path / "m"), cfg, m, seed=1)
    assert (tmp_path / "m" / "model.safetensors").exists()


@pytest.mark.gpu
def test_host_and_device_draw_the_same_bits():
    import torch
    from rustingstrata_b200.kernels import ops
    from rustingstrata_b200.weights import f32_to_bf16_bits
    table = torch.from_numpy(R.normal_table().copy()).cuda()
    n = (1 << 20) + 37
    for name, need, std, norm_std in (("a.weight", TensorNeed((n,)), 0.02, 0.0), ("b.weight", TensorNeed((n,), "norm"), 0.02, 0.1),
                                      ("c.weight", TensorNeed((n,)), 0.37, 0.0)):
        host = R.draw_values(9, name, need, std, norm_std)
        scale, shift = R.scale_shift(need, std, norm_std)
        dev32 = torch.empty(n, dtype=torch.float32, device="cuda")
        ops.fill_random(dev32, R.tensor_key(9, name), table, scale, shift)
        assert np.array_equal(dev32.cpu().numpy().view(np.uint32), host.view(np.uint32)), name
        dev16 = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        ops.fill_random(dev16, R.tensor_key(9, name), table, scale, shift)
        assert np.array_equal(dev16.view(torch.int16).cpu().numpy().view(np.uint16), f32_to_bf16_bits(host)), name
        # a later part of the stream drawn on its own
        part = torch.empty(1000, dtype=torch.float32, device="cuda")
        ops.fill_random(part, R.tensor_key(9, name), table, scale, shift, first=12345)
        assert np.array_equal(part.cpu().numpy(), host[12345:13345])
    bits = torch.empty(4096, dtype=torch.int32, device="cuda")
    ops.fill_random(bits, R.tensor_key(9, "t"), None, 0.0, 0.0)
    assert np.array_equal(bits.cpu().numpy(), R.draw_values(9, "t", TensorNeed((4096,), "int_table"), 0.0, 0.0))


@pytest.mark.gpu
def test_a_written_folder_and_the_device_drawn_model_are_the_same_model(tmp_path):
    """``init-random`` (host generator, file) and ``Engine(config, random_seed=...)`` (device generator, no file)
    give the same logits to the bit, in both precisions."""
    import torch
    from helpers import TINY, make_model_dir, random_tokens
    from rustingstrata_b200 import Engine
    from rustingstrata_b200.engine import StepEntry
    t = TINY["B"]
    folder = make_model_dir(str(tmp_path / "B"), "B")
    toks = random_tokens(t["config"]["vocab_size"], 40, 3)
    for dtype in ("float32", "bfloat16"):
        kw = dict(dtype=dtype, page_size=16, max_tokens=256, max_batch_tokens=64, max_seqs=2)
        a = Engine(folder, **kw).step_raw([StepEntry("x", toks, list(range(40)))])
        b = Engine(t["config"], random_seed=t["seed"], random_std=t["std"], random_norm_std=t["norm_std"], **kw
                   ).step_raw([StepEntry("x", toks, list(range(40)))])
        assert torch.equal(a, b), dtype
