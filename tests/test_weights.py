"""Safetensors reading and writing, the one weights error, random model folders."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny
from pulsarlm_b200 import models  # noqa: F401
from pulsarlm_b200.config.registry import read_model_config, read_model_dir
from pulsarlm_b200.models.model import tensor_needs_of
from pulsarlm_b200.weights.loader import WeightsError, load_checked
from pulsarlm_b200.weights.random_init import write_random_model
from pulsarlm_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, model_files, write_safetensors

CPU = torch.device("cpu")


def needs_of(cfg):
    arch, typed = read_model_config(cfg)
    return tensor_needs_of(arch.describe(typed))


def test_reader_reads_what_the_safetensors_package_wrote(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
               "h": torch.randn(2, 2).half()}
    save_file(tensors, str(tmp_path / "x.safetensors"), metadata={"format": "pt"})
    f = SafetensorsFile(str(tmp_path / "x.safetensors"))
    assert sorted(f.names()) == sorted(tensors)
    for name, t in tensors.items():
        assert f.dtype(name) == t.dtype and f.shape(name) == tuple(t.shape)
        assert torch.equal(f.tensor(name), t)


def test_writer_is_read_by_the_safetensors_package(tmp_path):
    tensors = {"w": torch.randn(4, 6).to(torch.bfloat16), "v": torch.randn(5), "empty": torch.zeros(0, 3)}
    write_safetensors(str(tmp_path / "y.safetensors"), tensors, metadata={"k": "v"})
    back = load_file(str(tmp_path / "y.safetensors"))
    assert set(back) == set(tensors)
    for name, t in tensors.items():
        assert torch.equal(back[name], t)


def test_truncated_file_is_refused(tmp_path):
    path = tmp_path / "z.safetensors"
    write_safetensors(str(path), {"w": torch.randn(8, 8)})
    data = path.read_bytes()
    path.write_bytes(data[:-16])
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(path))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = tiny.TINY_B
    w = tiny.random_weights(cfg, 1)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["lm_head.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    w["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(32, 96)
    w["model.norm.weight"] = torch.zeros(97)
    tiny.write_model_dir(str(tmp_path), cfg, w)
    with pytest.raises(WeightsError) as error:
        load_checked(str(tmp_path), needs_of(cfg), torch.float32, CPU)
    e = error.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [n for n, _, _ in e.wrong_shape] == ["model.layers.2.self_attn.k_proj.weight", "model.norm.weight"]
    text = str(e)
    for word in ("lm_head.weight", "q_proj.bias", "[32, 96]", "[64, 96]", "[97]"):
        assert word in text


def test_tied_checkpoint_may_carry_a_head_copy_but_untied_must(tmp_path):
    cfg = tiny.TINY_A
    w = tiny.random_weights(cfg, 1)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    tiny.write_model_dir(str(tmp_path), cfg, w)
    loaded = load_checked(str(tmp_path), needs_of(cfg), torch.float32, CPU)
    assert "lm_head.weight" not in loaded


def test_dtype_rules(tmp_path):
    cfg = tiny.TINY_A
    w = tiny.random_weights(cfg, 1, torch.bfloat16)
    w["model.norm.weight"] = w["model.norm.weight"].float()
    tiny.write_model_dir(str(tmp_path), cfg, w)
    as_bf16 = load_checked(str(tmp_path), needs_of(cfg), torch.bfloat16, CPU)
    assert as_bf16["model.norm.weight"].dtype == torch.float32  # stored in 32-bit, stays so
    assert as_bf16["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16
    assert as_bf16["model.embed_tokens.weight"].dtype == torch.bfloat16
    as_f32 = load_checked(str(tmp_path), needs_of(cfg), torch.float32, CPU)
    assert all(t.dtype == torch.float32 for t in as_f32.values())
    assert torch.equal(as_f32["model.embed_tokens.weight"], w["model.embed_tokens.weight"].float())


def test_random_model_folder_loads_and_is_seeded(tmp_path):
    a = write_random_model(str(tmp_path / "a"), tiny.TINY_B, seed=5, dtype=torch.float32)
    b = write_random_model(str(tmp_path / "b"), tiny.TINY_B, seed=5, dtype=torch.float32)
    c = write_random_model(str(tmp_path / "c"), tiny.TINY_B, seed=6, dtype=torch.float32)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    arch, cfg, text = read_model_dir(a)
    assert text == json.loads(json.dumps(tiny.TINY_B))
    wa, wb, wc = (load_checked(d, needs_of(tiny.TINY_B), torch.float32, CPU) for d in (a, b, c))
    assert all(torch.equal(wa[n], wb[n]) for n in wa)
    assert not torch.equal(wa["lm_head.weight"], wc["lm_head.weight"])
    assert abs(float(wa["lm_head.weight"].std()) - 0.02) < 0.002
    assert abs(float(wa["model.norm.weight"].mean()) - 1.0) < 0.02


def test_sharded_folder(tmp_path):
    cfg = tiny.TINY_A
    w = tiny.random_weights(cfg, 1)
    names = sorted(w)
    half = len(names) // 2
    save_file({n: w[n] for n in names[:half]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({n: w[n] for n in names[half:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert len(model_files(str(tmp_path))) == 2
    loaded = load_checked(str(tmp_path), needs_of(cfg), torch.float32, CPU)
    assert all(torch.equal(loaded[n], w[n]) for n in w)


def test_random_values_are_a_function_of_seed_name_and_index():
    """The counter-based generator: a tensor's values do not depend on its length, on
    other tensors or on the order of drawing; noise is centred with unit variance; the
    bfloat16 form is the float32 form rounded once."""
    from pulsarlm_b200.weights.random_init import fill_random

    a = fill_random(torch.empty(200000), 7, "layers.0.w", 0.02)
    assert torch.equal(a[:1000], fill_random(torch.empty(1000), 7, "layers.0.w", 0.02))
    assert not torch.equal(a[:1000], fill_random(torch.empty(1000), 8, "layers.0.w", 0.02))
    other = fill_random(torch.empty(200000), 7, "layers.1.w", 0.02)
    assert abs(float(torch.corrcoef(torch.stack([a, other]))[0, 1])) < 0.01
    assert abs(float(a.mean())) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    assert 2.7 < float(((a / 0.02) ** 4).mean()) < 3.1          # close to a normal's 3
    assert float(a.abs().max()) < 0.02 * 4.9                     # sum of eight uniforms: bounded
    half = fill_random(torch.empty(1000, dtype=torch.bfloat16), 7, "layers.0.w", 0.02)
    assert torch.equal(half, a[:1000].to(torch.bfloat16))
    scale = fill_random(torch.empty(4096), 7, "norm", 0.02, 1.0)
    assert abs(float(scale.mean()) - 1.0) < 2e-3 and abs(float(scale.std()) - 0.02) < 2e-3
