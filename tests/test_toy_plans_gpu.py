"""A toy mixer that plans every step on the host: it returns an array of its own from
`plan_step`, finds it on the device in `batch.plans`, and works in eager steps, in
captured decode steps (where the array is refreshed before every replay; replays it
names a variant for get a capture of their own) and through the engine's pipelined
decoding, without a change to the package's files."""

import numpy as np
import pytest
import torch

import plain_llama
import tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
GAINS = (0.5, 1.0, 1.75)


def gain_of(position: int) -> float:
    return GAINS[(position // 7) % 3]


def register_toy():
    from pulsarlm_b200.config.llama import LlamaConfig
    from pulsarlm_b200.config.registry import register_architecture
    from pulsarlm_b200.models.llama import describe_llama
    from pulsarlm_b200.parts.registry import Part, register_part
    from pulsarlm_b200.parts.spec import PartSpec, TensorNeed

    @register_part("mixer", "toy_gain", replace=True)
    class ToyGain(Part):
        """out[t] = gain(position of t) * (h[t] W^T), the gain looked up on the host per
        token and staged as a float32 array: a stand-in for the chunk boundaries or
        expert offsets a real part would plan."""

        planned = 0  # how often plan_step ran (the test reads it)
        regimes: set = set()  # which variants of a captured step plan_step was asked for

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.hidden = spec.params["hidden_size"]

        @classmethod
        def tensor_needs(cls, spec):
            h = spec.params["hidden_size"]
            return {spec.tensors["w"]: TensorNeed((h, h))}

        def load(self, tensors):
            self.w = tensors[self.spec.tensors["w"]]

        def cache_need(self):
            return None

        def plan_key(self):
            return ("toy_gain",)

        def plan_variant(self, step):
            # a capture of its own for replays in which some request is past 40 tokens (a stand-in
            # for a part that changes kernels with the lengths)
            return "long" if max(step.context_lens) > 40 else None

        def plan_step(self, step):
            type(self).planned += 1
            if step.fixed_shape:
                type(self).regimes.add(step.variants.get(self.plan_key()))
            gains = np.empty(step.n_tokens, dtype=np.float32)
            for e in range(step.n_entries):
                first = step.context_lens[e] - step.query_lens[e]
                for j in range(step.query_lens[e]):
                    gains[step.first_rows[e] + j] = gain_of(first + j)
            return {"gains": gains, "note": "kept as planned first"}

        def forward(self, h, batch):
            plan = batch.plans[self.plan_key()]
            assert plan["note"] == "kept as planned first" and plan["gains"].dtype == torch.float32
            return ((h.float() @ self.w.float().T) * plan["gains"][:, None]).to(h.dtype)

    def describe(cfg):
        spec = describe_llama(cfg)
        spec.layers[1].mixer = PartSpec("toy_gain", {"hidden_size": cfg.hidden_size},
                                        {"w": "model.layers.1.toy.w.weight"})
        return spec

    register_architecture("ToyGainForCausalLM", LlamaConfig.from_text, describe, replace=True)
    return ToyGain


def plain_toy(cfg, w, tokens):
    wd = {k: v.double() for k, v in w.items()}
    x = plain_llama.embed(wd["model.embed_tokens.weight"], torch.tensor(tokens))
    eps = cfg["rms_norm_eps"]
    pos = torch.arange(len(tokens))
    gains = torch.tensor([gain_of(p) for p in range(len(tokens))], dtype=torch.float64)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, wd[p + "input_layernorm.weight"], eps)
        if layer == 1:
            x = x + (h @ wd[p + "toy.w.weight"].T) * gains[:, None]
        else:
            x = x + plain_llama.attention_block(h, wd, p, cfg, pos)
        h = plain_llama.rms_norm(x, wd[p + "post_attention_layernorm.weight"], eps)
        x = x + plain_llama.swiglu_mlp(h, wd[p + "mlp.gate_proj.weight"], wd[p + "mlp.up_proj.weight"],
                                       wd[p + "mlp.down_proj.weight"])
    return plain_llama.rms_norm(x, wd["model.norm.weight"], eps) @ wd["lm_head.weight"].T


def test_a_part_that_plans_its_steps_on_the_host(tmp_path):
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry

    toy = register_toy()
    cfg = dict(tiny.TINY_B, architectures=["ToyGainForCausalLM"])
    w = tiny.random_weights(cfg, 4)
    for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
        del w[f"model.layers.1.self_attn.{name}.weight"]
    w["model.layers.1.toy.w.weight"] = torch.randn(96, 96, generator=torch.Generator().manual_seed(2)) / 10
    model = load_model(tiny.write_model_dir(str(tmp_path), cfg, w), "float32", DEV)
    assert [type(n).__name__ for n in model.cache_needs()] == ["KVCacheNeed", "NoneType", "KVCacheNeed"]

    # eager steps: portions of two requests and single tokens beside them
    runner = ModelRunner(model, CacheManager(model.cache_needs(), tiny.PAGE_B, 12, 3, torch.float32, DEV))
    assert runner.graphs_allowed and any(key == ("toy_gain",) for key, _ in runner._planners)
    a, b = tiny.random_tokens(cfg, 50, 1), tiny.random_tokens(cfg, 33, 2)
    got = {"a": [], "b": []}
    plan = [[("a", a[:7])], [("a", a[7:20]), ("b", b[:5])], [("b", b[5:6]), ("a", a[20:21])],
            [("a", a[21:50]), ("b", b[6:33])]]
    for step in plan:
        logits = runner.step([StepEntry(r, t, list(range(len(t)))) for r, t in step]).cpu()
        at = 0
        for r, t in step:
            got[r].append(logits[at : at + len(t)])
            at += len(t)
    runner.check_status()
    for r, tokens in (("a", a), ("b", b)):
        assert plain_llama.max_relative_error(torch.cat(got[r]), plain_toy(cfg, w, tokens)) < 1e-4, r

    # through the engine: captured, pipelined decode steps whose gains change from replay to replay
    engine = Engine(model, n_pages=12, page_size=tiny.PAGE_B, max_requests=3, stop_ids=[], record_logits=True,
                    prefill_tokens_per_step=16)
    before = toy.planned
    requests = [engine.submit(p, sampling=SamplingParams(temperature=0.0), max_tokens=30, ignore_eos=True)
                for p in (a[:11], b[:20])]
    while any(not r.finished for r in requests):
        engine.step()
    engine.sync()
    engine.runner.check_status()
    assert engine.runner.graph_steps >= 29 and engine.lookahead
    # replays before and after a request passed 40 tokens ran captures of their own
    assert toy.regimes == {None, "long"} and {len(key) for key in engine.runner._graphs} == {2, 3}
    assert toy.planned - before >= engine.runner.steps  # every step was planned, the replays too
    for request in requests:
        sequence = list(request.prompt) + list(request.output)
        reference = plain_toy(cfg, w, sequence[:-1])[len(request.prompt) - 1:]
        assert plain_llama.max_relative_error(torch.stack(request.logits), reference) < 1e-4
        assert list(request.output) == [int(row.argmax()) for row in request.logits]
