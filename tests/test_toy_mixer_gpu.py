"""A toy mixer with a state of its own, defined here, is registered, built and
stepped without a change to the package's files: the state lives in the cache
manager's per-request slots and is carried across steps and portions."""

import pytest
import torch

import tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def register_toy():
    from pulsarlm_b200.config.llama import LlamaConfig
    from pulsarlm_b200.config.registry import register_architecture
    from pulsarlm_b200.models.llama import describe_llama
    from pulsarlm_b200.parts.registry import Part, register_part
    from pulsarlm_b200.parts.spec import PartSpec, StateNeed, TensorNeed

    @register_part("mixer", "toy_decay", replace=True)
    class ToyDecay(Part):
        """state' = decay * state + h W_in^T per token, in order; out = state' W_out^T.
        A running sum with decay: the smallest mixer whose output at a token depends
        on every earlier token through a state of fixed size."""

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.hidden, self.width, self.decay = spec.params["hidden_size"], spec.params["width"], spec.params["decay"]
            self.binding = None

        @classmethod
        def tensor_needs(cls, spec):
            h, n = spec.params["hidden_size"], spec.params["width"]
            return {spec.tensors["in"]: TensorNeed((n, h)), spec.tensors["out"]: TensorNeed((h, n))}

        def load(self, tensors):
            self.w_in = tensors[self.spec.tensors["in"]].float()
            self.w_out = tensors[self.spec.tensors["out"]].float()

        def cache_need(self):
            return StateNeed((self.width,), "float32")

        def bind_cache(self, binding):
            self.binding = binding

        def forward(self, h, batch):
            # Plain torch on the device: the point of this test is the framework's
            # plumbing (registry, slots, batches), not this mixer's speed.
            u = h.float() @ self.w_in.T
            out = torch.empty_like(u)
            entry = batch.entry.long()
            slots = batch.slots.long()
            for e in range(batch.n_entries):
                rows = torch.nonzero(entry == e).flatten()
                state = self.binding.states[slots[e]]
                for r in rows.tolist():  # rows of an entry are in position order
                    state.mul_(self.decay).add_(u[r])
                    out[r] = state
            return (out @ self.w_out.T).to(h.dtype)

    def describe(cfg):
        spec = describe_llama(cfg)
        layer = spec.layers[1]
        layer.mixer = PartSpec("toy_decay", {"hidden_size": cfg.hidden_size, "width": 24, "decay": 0.9},
                               {"in": "model.layers.1.toy.in.weight", "out": "model.layers.1.toy.out.weight"})
        return spec

    register_architecture("ToyDecayForCausalLM", LlamaConfig.from_text, describe, replace=True)


def plain_toy(cfg, w, tokens):
    import plain_llama

    wd = {k: v.double() for k, v in w.items()}
    x = plain_llama.embed(wd["model.embed_tokens.weight"], torch.tensor(tokens))
    eps = cfg["rms_norm_eps"]
    pos = torch.arange(len(tokens))
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, wd[p + "input_layernorm.weight"], eps)
        if layer == 1:
            u = h @ wd[p + "toy.in.weight"].T
            state = torch.zeros(24, dtype=torch.float64)
            rows = []
            for t in range(len(tokens)):
                state = 0.9 * state + u[t]
                rows.append(state)
            x = x + torch.stack(rows) @ wd[p + "toy.out.weight"].T
        else:
            x = x + plain_llama.attention_block(h, wd, p, cfg, pos)
        h = plain_llama.rms_norm(x, wd[p + "post_attention_layernorm.weight"], eps)
        x = x + plain_llama.swiglu_mlp(h, wd[p + "mlp.gate_proj.weight"], wd[p + "mlp.up_proj.weight"],
                                       wd[p + "mlp.down_proj.weight"])
    return plain_llama.rms_norm(x, wd["model.norm.weight"], eps) @ wd["lm_head.weight"].T


def test_toy_mixer_registers_builds_and_steps(tmp_path):
    import plain_llama
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry

    register_toy()
    cfg = dict(tiny.TINY_B, architectures=["ToyDecayForCausalLM"])
    w = tiny.random_weights(cfg, 2)
    for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
        del w[f"model.layers.1.self_attn.{name}.weight"]
    gen = torch.Generator().manual_seed(1)
    w["model.layers.1.toy.in.weight"] = torch.randn(24, 96, generator=gen) / 10
    w["model.layers.1.toy.out.weight"] = torch.randn(96, 24, generator=gen) / 5
    folder = tiny.write_model_dir(str(tmp_path), cfg, w)

    model = load_model(folder, "float32", DEV)  # the registry finds the architecture by config.json
    needs = model.cache_needs()
    assert type(needs[1]).__name__ == "StateNeed" and type(needs[0]).__name__ == "KVCacheNeed"
    cache = CacheManager(needs, tiny.PAGE_B, 12, 3, torch.float32, DEV)
    runner = ModelRunner(model, cache)
    assert not runner.graphs_allowed

    a = tiny.random_tokens(cfg, 50, 1)
    b = tiny.random_tokens(cfg, 33, 2)
    got = {"a": [], "b": []}
    # a and b interleaved, in portions and single tokens; b starts later and reuses nothing of a's state
    plan = [[("a", a[:7])], [("a", a[7:20]), ("b", b[:5])], [("b", b[5:6]), ("a", a[20:21])],
            [("a", a[21:50]), ("b", b[6:33])]]
    for step in plan:
        entries = [StepEntry(r, t, list(range(len(t)))) for r, t in step]
        logits = runner.step(entries).cpu()
        at = 0
        for r, t in step:
            got[r].append(logits[at : at + len(t)])
            at += len(t)
    runner.check_status()
    for r, tokens in (("a", a), ("b", b)):
        err = plain_llama.max_relative_error(torch.cat(got[r]), plain_toy(cfg, w, tokens))
        assert err < 1e-4, (r, err)
    # a finished request's slot is zeroed for the next one
    runner.end("a")
    c = tiny.random_tokens(cfg, 9, 3)
    logits = runner.step([StepEntry("c", c, list(range(9)))]).cpu()
    assert cache.slot("c") == 0
    assert plain_llama.max_relative_error(logits, plain_toy(cfg, w, c)) < 1e-4


def test_a_state_mixer_that_says_so_steps_in_captured_graphs(tmp_path):
    """The same toy mixer with a single-token step that makes no host round trip
    (`captures_state_steps`): the engine captures its decode steps. The capture's warm-up
    run works on a copy of the states, rows that pad a step to its size update the padding
    slot, and pipelined steps advance a state once each: the tokens generated with graphs
    and lookahead equal those of eager steps and of the plain implementation."""
    import plain_llama
    from pulsarlm_b200 import Engine, SamplingParams
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.parts.registry import part_class, register_part

    register_toy()
    eager_class = part_class("mixer", "toy_decay")

    @register_part("mixer", "toy_decay", replace=True)
    class ToyDecayCapturable(eager_class):
        def captures_state_steps(self):
            return True

        def forward(self, h, batch):
            if int(batch.n_decode) != h.shape[0]:
                return super().forward(h, batch)  # prompt portions: the loop over an entry's tokens
            # one token per entry: state[slot] = decay * state[slot] + u, for all entries at once
            u = h.float() @ self.w_in.T
            slots = batch.slots.long()
            states = self.binding.states
            new = states[slots] * self.decay + u
            states[slots] = new
            return (new @ self.w_out.T).to(h.dtype)

    cfg = dict(tiny.TINY_B, architectures=["ToyDecayForCausalLM"])
    w = tiny.random_weights(cfg, 2)
    for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
        del w[f"model.layers.1.self_attn.{name}.weight"]
    gen = torch.Generator().manual_seed(1)
    w["model.layers.1.toy.in.weight"] = torch.randn(24, 96, generator=gen) / 10
    w["model.layers.1.toy.out.weight"] = torch.randn(96, 24, generator=gen) / 5
    folder = tiny.write_model_dir(str(tmp_path), cfg, w)
    model = load_model(folder, "float32", DEV)
    prompts = [tiny.random_tokens(cfg, n, 10 + n) for n in (9, 30, 4)]  # three requests: steps padded to four rows
    greedy = SamplingParams(temperature=0.0)
    results = {}
    for name, options in (("graphs", {}), ("eager", {"cuda_graphs": False})):
        engine = Engine(model, n_pages=24, page_size=tiny.PAGE_B, max_requests=3, stop_ids=[], **options)
        assert engine.runner.graphs_allowed
        results[name] = engine.generate(prompts, greedy, max_tokens=12, ignore_eos=True)
        assert (engine.runner.graph_steps > 0) == (name == "graphs")
        # a second round on the same engine: slots are zeroed at hand-out, the padding slot is nobody's
        assert engine.generate(prompts, greedy, max_tokens=12, ignore_eos=True) == results[name]
    assert results["graphs"] == results["eager"]
    for prompt, out in zip(prompts, results["graphs"]):
        logits = plain_toy(cfg, w, list(prompt) + list(out))
        for i, token in enumerate(out):
            row = logits[len(prompt) - 1 + i]
            assert float(row.max() - row[token]) <= 1e-4 * float(row.abs().max()), (i, token)
