"""Configuration and the architecture registry (cases after
pulsarlm/tests/test_engine_model.py:262-327)."""

import copy
import json

import pytest

import tiny
from pulsarlm_b200 import models  # noqa: F401
from pulsarlm_b200.config.base import ConfigError
from pulsarlm_b200.config.llama import LlamaConfig
from pulsarlm_b200.config.registry import find_architecture, read_model_config, register_architecture
from pulsarlm_b200.models.model import tensor_needs_of


def test_reads_every_key():
    cfg = LlamaConfig.from_text(tiny.TINY_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 6, 2)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 256, 1000)
    assert cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False and cfg.max_position_embeddings == 512
    s = cfg.rope.llama3_scaling
    assert cfg.rope.theta == 500000.0 and (s.factor, s.low_freq_factor, s.high_freq_factor) == (8.0, 1.0, 4.0)
    assert s.original_max_position_embeddings == 64


def test_head_dim_defaults_to_hidden_over_heads():
    text = dict(tiny.TINY_A)
    del text["head_dim"]
    assert LlamaConfig.from_text(text).head_dim == 64 // 4


def test_rope_parameters_layout_and_plain_rope():
    text = copy.deepcopy(tiny.TINY_B)
    scaling = text.pop("rope_scaling")
    theta = text.pop("rope_theta")
    text["rope_parameters"] = {**scaling, "rope_theta": theta}
    assert LlamaConfig.from_text(text).rope == LlamaConfig.from_text(tiny.TINY_B).rope
    legacy = copy.deepcopy(tiny.TINY_B)
    legacy["rope_scaling"] = {"type": "llama3", **{k: v for k, v in scaling.items() if k != "rope_type"}}
    assert LlamaConfig.from_text(legacy).rope == LlamaConfig.from_text(tiny.TINY_B).rope
    assert LlamaConfig.from_text(tiny.TINY_A).rope.llama3_scaling is None


@pytest.mark.parametrize("change,word", [
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "yarn"),
    ({"rope_scaling": {"type": "dynamic", "factor": 2.0}}, "dynamic"),
    ({"attention_bias": True}, "bias"),
    ({"mlp_bias": True}, "bias"),
    ({"hidden_act": "gelu"}, "gelu"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rms_norm_eps": "small"}, "rms_norm_eps"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
])
def test_rejections(change, word):
    text = {**tiny.TINY_A, **change}
    with pytest.raises(ConfigError) as error:
        LlamaConfig.from_text(text)
    assert word in str(error.value)


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "intermediate_size",
                                 "vocab_size", "rms_norm_eps", "rope_theta"])
def test_missing_key_is_named(key):
    text = dict(tiny.TINY_A)
    del text[key]
    with pytest.raises(ConfigError) as error:
        LlamaConfig.from_text(text)
    assert key in str(error.value)


def test_round_trip_through_to_text():
    for text in (tiny.TINY_A, tiny.TINY_B, tiny.TINY_C):
        cfg = LlamaConfig.from_text(text)
        assert LlamaConfig.from_text(json.loads(json.dumps(cfg.to_text()))) == cfg


def test_registry_by_architecture_and_model_type():
    assert find_architecture(tiny.TINY_A).name == "LlamaForCausalLM"
    assert find_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError) as error:
        find_architecture({"architectures": ["MambaForCausalLM"]})
    assert "MambaForCausalLM" in str(error.value) and "LlamaForCausalLM" in str(error.value)


def test_registering_another_architecture():
    from pulsarlm_b200.models.llama import describe_llama

    def describe(cfg):
        spec = describe_llama(cfg)
        spec.order = spec.order + [spec.order[-1]]  # the last layer runs twice
        return spec

    register_architecture("TwiceLastForCausalLM", LlamaConfig.from_text, describe, replace=True)
    arch, cfg = read_model_config({**tiny.TINY_A, "architectures": ["TwiceLastForCausalLM"]})
    assert arch.describe(cfg).order == [0, 1, 1]
    with pytest.raises(ValueError):
        register_architecture("TwiceLastForCausalLM", LlamaConfig.from_text, describe)


def test_spec_names_every_checkpoint_tensor():
    for text in (tiny.TINY_A, tiny.TINY_B):
        arch, cfg = read_model_config(text)
        needs = tensor_needs_of(arch.describe(cfg))
        required = {n: need.shape for n, need in needs.items() if not need.optional}
        assert required == tiny.tensor_shapes(text)


def test_a_layer_may_only_read_a_cache_it_can_see_whole():
    """A layer that reads another layer's cache must have that layer's kv heads and head
    size, and a window no wider than the owner's: pages behind the owner's window are
    given back while the request runs."""
    import torch

    from pulsarlm_b200.models.llama import describe_llama
    from pulsarlm_b200.models.model import Model

    def model_with(reader: dict, owner: dict) -> Model:
        spec = describe_llama(LlamaConfig.from_text(tiny.TINY_A))
        spec.layers[0].mixer.params.update(owner)
        spec.layers[1].mixer.params.update({"cache_from": 0, **reader})
        return Model(spec, torch.float32, torch.device("cpu"))

    assert model_with({}, {}).cache_sources() == [None, 0]
    assert model_with({"window": 8}, {"window": 24}).cache_sources() == [None, 0]
    assert model_with({"window": 8}, {}).cache_sources() == [None, 0]
    with pytest.raises(ValueError, match="keeps a window of 8 only"):
        model_with({}, {"window": 8}).cache_sources()
    with pytest.raises(ValueError, match="keeps a window of 8 only"):
        model_with({"window": 9}, {"window": 8}).cache_sources()
    with pytest.raises(ValueError, match="kv heads of size"):
        model_with({"n_kv_heads": 2}, {}).cache_sources()
    with pytest.raises(ValueError, match="kv heads of size"):
        model_with({"head_dim": 32}, {}).cache_sources()
