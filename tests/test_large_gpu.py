"""The engine at the Llama-3.1-8B layer sizes (two layers, the full 128,256-token
vocabulary, llama3 RoPE scaling at its real parameters) against the plain
implementation, in float32 and bfloat16: sizes at which an index that overflows, a
tile that is dropped at the end of a wide matrix or a RoPE angle that loses
precision would show. The prompt is cut into a long portion, a short one and
single tokens, beside a second request."""

import pytest
import torch

import plain_llama
from harness import TOLERANCE

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2,
    "hidden_size": 4096,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "intermediate_size": 14336,
    "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
}

# Two more layer shapes of the family (two layers each): small heads, a tied and very
# wide vocabulary; and one kv head per query head, a width that is no power of two.
CONFIG_1B = dict(CONFIG, hidden_size=2048, head_dim=64, intermediate_size=8192, tie_word_embeddings=True,
                 rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 8192})
CONFIG_13B = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2,
    "hidden_size": 5120,
    "num_attention_heads": 40,
    "num_key_value_heads": 40,
    "intermediate_size": 13824,
    "vocab_size": 32000,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
}


@pytest.fixture(scope="module")
def weights():
    import tiny

    return tiny.random_weights(CONFIG, seed=3, dtype=torch.bfloat16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_llama_8b_layer_sizes(weights, dtype):
    run_shape(CONFIG, weights, dtype)


@pytest.mark.parametrize("config", [CONFIG_1B, CONFIG_13B], ids=["llama-3.2-1b", "llama-2-13b"])
def test_other_layer_sizes_of_the_family(config):
    import tiny

    run_shape(config, tiny.random_weights(config, seed=5, dtype=torch.bfloat16), "bfloat16")


def run_shape(CONFIG, weights, dtype):
    from pulsarlm_b200 import models  # noqa: F401
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.config.registry import read_model_config
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.models.model import Model
    from pulsarlm_b200.weights.loader import check_tensors

    device = torch.device("cuda:0")
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    arch, cfg = read_model_config(CONFIG)
    model = Model(arch.describe(cfg), torch_dtype, device)
    model.load(check_tensors("test", model.tensor_needs(), weights, torch_dtype, device))
    runner = ModelRunner(model, CacheManager(model.cache_needs(), 16, 32, 2, torch_dtype, device))

    gen = torch.Generator().manual_seed(1)
    a = torch.randint(0, CONFIG["vocab_size"], (150,), generator=gen).tolist()
    b = torch.randint(0, CONFIG["vocab_size"], (41,), generator=gen).tolist()
    want = [0, 63, 129]
    rows = {}
    out = runner.step([StepEntry("a", a[:130], want)])
    rows.update({("a", w): out[i] for i, w in enumerate(want)})
    out = runner.step([StepEntry("b", b[:38], [37]), StepEntry("a", a[130:147], [16])])
    rows[("b", 37)], rows[("a", 146)] = out[0], out[1]
    for i in range(147, 150):
        out = runner.step([StepEntry("a", a[i:i + 1], [0]), StepEntry("b", b[i - 109:i - 108], [0])])
        rows[("a", i)], rows[("b", i - 109)] = out[0], out[1]
    runner.check_status()

    ref = {"a": plain_llama.forward(CONFIG, weights, a, dtype=torch.float32),
           "b": plain_llama.forward(CONFIG, weights, b, dtype=torch.float32)}
    for (request, position), got in rows.items():
        err = plain_llama.max_relative_error(got.cpu(), ref[request][position])
        assert err < TOLERANCE[dtype], (request, position, err)


@pytest.mark.parametrize("config", [CONFIG, CONFIG_13B], ids=["llama-3.1-8b", "llama-2-13b"])
def test_a_short_portion_after_a_long_history(config):
    """1,100 tokens of a prompt in one step, then 100 beside another request's single
    token: one tile of queries over 1,200 keys, which the attention part splits over the
    keys (checked below), in both arrangements of the kernel (two heads of a kv head per
    CTA; one head per CTA). A small vocabulary keeps the plain implementation quick."""
    import tiny
    from pulsarlm_b200 import models  # noqa: F401
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.config.registry import read_model_config
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry
    from pulsarlm_b200.models.model import Model
    from pulsarlm_b200.parts.attention import prefill_splits
    from pulsarlm_b200.weights.loader import check_tensors

    config = dict(config, vocab_size=2048)
    weights = tiny.random_weights(config, seed=7, dtype=torch.bfloat16)
    device = torch.device("cuda:0")
    arch, cfg = read_model_config(config)
    model = Model(arch.describe(cfg), torch.bfloat16, device)
    model.load(check_tensors("test", model.tensor_needs(), weights, torch.bfloat16, device))
    runner = ModelRunner(model, CacheManager(model.cache_needs(), 16, 96, 2, torch.bfloat16, device))
    heads, kv_heads = config["num_attention_heads"], config["num_key_value_heads"]
    ctas = heads // 2 if (heads // kv_heads) % 2 == 0 else heads
    assert prefill_splits(ctas, 1200, 100, heads, plain_llama.head_dim_of(config), device) > 1

    gen = torch.Generator().manual_seed(2)
    a = torch.randint(0, 2048, (1200,), generator=gen).tolist()
    b = torch.randint(0, 2048, (31,), generator=gen).tolist()
    runner.step([StepEntry("a", a[:1100], []), StepEntry("b", b[:30], [])])
    out = runner.step([StepEntry("a", a[1100:], [0, 63, 99]), StepEntry("b", b[30:], [0])])
    runner.check_status()
    ref_a = plain_llama.forward(config, weights, a, dtype=torch.float32)
    ref_b = plain_llama.forward(config, weights, b, dtype=torch.float32)
    for got, expected in ((out[0], ref_a[1100]), (out[1], ref_a[1163]), (out[2], ref_a[1199]), (out[3], ref_b[30])):
        assert plain_llama.max_relative_error(got.cpu(), expected) < TOLERANCE["bfloat16"]
