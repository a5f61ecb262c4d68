"""Two more toy parts, defined here and registered without a change to the package's
files: a feed-forward that routes every token to one of three small experts, and a
position encoding of its own (rotates only the first half of each head, at
frequencies that are no powers of a base). They stand in one model beside the
package's parts, are stepped in portions and single tokens, and are compared with a
plain restatement of the same layers."""

import math

import pytest
import torch

import plain_llama
import tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
EXPERTS, EXPERT_WIDTH = 3, 40


def toy_frequencies(rotary_dim):
    return [1.0 / (3.0 + 1.7 * j) for j in range(rotary_dim // 2)]


def register_toys():
    from pulsarlm_b200.config.llama import LlamaConfig
    from pulsarlm_b200.config.registry import register_architecture
    from pulsarlm_b200.models.llama import describe_llama
    from pulsarlm_b200.parts.registry import Part, register_part
    from pulsarlm_b200.parts.spec import PartSpec, TensorNeed

    @register_part("feed_forward", "toy_routed", replace=True)
    class ToyRouted(Part):
        """Router logits h R^T in float32; the token goes to the expert with the largest
        logit (the lower index on a tie) and its output is scaled by that expert's
        softmax probability: out = p_e * relu(h A_e^T) B_e^T."""

        @classmethod
        def tensor_needs(cls, spec):
            h, n, width = spec.params["hidden_size"], spec.params["experts"], spec.params["width"]
            t = spec.tensors
            return {t["router"]: TensorNeed((n, h)), t["a"]: TensorNeed((n * width, h)),
                    t["b"]: TensorNeed((n * h, width))}

        def load(self, tensors):
            p, t = self.spec.params, self.spec.tensors
            self.router = tensors[t["router"]].float()
            self.a = tensors[t["a"]].float().view(p["experts"], p["width"], p["hidden_size"])
            self.b = tensors[t["b"]].float().view(p["experts"], p["hidden_size"], p["width"])

        def forward(self, h, batch):
            x = h.float()
            probabilities = torch.softmax(x @ self.router.T, dim=-1)
            chosen = probabilities.argmax(dim=-1)
            inner = torch.relu(torch.einsum("th,twh->tw", x, self.a[chosen]))
            out = torch.einsum("tw,thw->th", inner, self.b[chosen])
            return (out * probabilities.gather(1, chosen[:, None])).to(h.dtype)

    @register_part("position", "toy_half", replace=True)
    class ToyHalf(Part):
        """Rotates pairs (j, j + head_dim / 4) of the first half of a head by
        pos / (3 + 1.7 j) radians; the second half passes through."""

        def __init__(self, spec, ctx):
            super().__init__(spec, ctx)
            self.rotary_dim = int(spec.params["head_dim"]) // 2
            self.inv_freq = torch.tensor(toy_frequencies(self.rotary_dim), dtype=torch.float64, device=ctx.device)

        def table(self):
            return self.inv_freq, self.rotary_dim

    def describe(cfg):
        spec = describe_llama(cfg)
        for i, layer in enumerate(spec.layers):
            if i != 1:  # layer 1 keeps the package's rope; the others get the toy encoding
                layer.mixer.params["position"] = PartSpec("toy_half", {"head_dim": cfg.head_dim})
        p = "model.layers.0.mlp."
        spec.layers[0].feed_forward = PartSpec(
            "toy_routed", {"hidden_size": cfg.hidden_size, "experts": EXPERTS, "width": EXPERT_WIDTH},
            {"router": p + "router.weight", "a": p + "experts_a.weight", "b": p + "experts_b.weight"})
        return spec

    register_architecture("ToyRoutedForCausalLM", LlamaConfig.from_text, describe, replace=True)


def rotate_first_half(x, positions):
    """x [T, heads, hd]: the toy encoding, in the dtype of x."""
    hd = x.shape[-1]
    rot = hd // 2
    angles = positions.to(torch.float64)[:, None] * torch.tensor(toy_frequencies(rot), dtype=torch.float64)[None, :]
    cos, sin = angles.cos().to(x.dtype)[:, None, :], angles.sin().to(x.dtype)[:, None, :]
    a, b = x[..., : rot // 2], x[..., rot // 2 : rot]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rot:]], dim=-1)


def plain_toys(cfg, w, tokens, chosen_out=None):
    wd = {k: v.double() for k, v in w.items()}
    x = plain_llama.embed(wd["model.embed_tokens.weight"], torch.tensor(tokens))
    eps, hidden = cfg["rms_norm_eps"], cfg["hidden_size"]
    n_heads, n_kv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], plain_llama.head_dim_of(cfg)
    pos = torch.arange(len(tokens))
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, wd[p + "input_layernorm.weight"], eps)
        if layer == 1:
            x = x + plain_llama.attention_block(h, wd, p, cfg, pos)
        else:
            q = (h @ wd[p + "self_attn.q_proj.weight"].T).view(len(tokens), n_heads, hd)
            k = (h @ wd[p + "self_attn.k_proj.weight"].T).view(len(tokens), n_kv, hd)
            v = (h @ wd[p + "self_attn.v_proj.weight"].T).view(len(tokens), n_kv, hd)
            o = plain_llama.causal_attention(rotate_first_half(q, pos), rotate_first_half(k, pos), v,
                                             1.0 / math.sqrt(hd))
            x = x + o.reshape(len(tokens), n_heads * hd) @ wd[p + "self_attn.o_proj.weight"].T
        h = plain_llama.rms_norm(x, wd[p + "post_attention_layernorm.weight"], eps)
        if layer == 0:
            probabilities = torch.softmax(h @ wd[p + "mlp.router.weight"].T, dim=-1)
            chosen = probabilities.argmax(dim=-1)
            if chosen_out is not None:
                top = torch.topk(h @ wd[p + "mlp.router.weight"].T, 2, dim=-1).values
                chosen_out.append((chosen, float((top[:, 0] - top[:, 1]).min())))
            a = wd[p + "mlp.experts_a.weight"].view(EXPERTS, EXPERT_WIDTH, hidden)
            b = wd[p + "mlp.experts_b.weight"].view(EXPERTS, hidden, EXPERT_WIDTH)
            rows = [probabilities[t, e] * (torch.relu(h[t] @ a[e].T) @ b[e].T) for t, e in enumerate(chosen.tolist())]
            x = x + torch.stack(rows)
        else:
            x = x + plain_llama.swiglu_mlp(h, wd[p + "mlp.gate_proj.weight"], wd[p + "mlp.up_proj.weight"],
                                           wd[p + "mlp.down_proj.weight"])
    head = wd["lm_head.weight"] if "lm_head.weight" in wd else wd["model.embed_tokens.weight"]
    return plain_llama.rms_norm(x, wd["model.norm.weight"], eps) @ head.T


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", None)])
def test_toy_feed_forward_and_position_register_build_and_step(tmp_path, dtype, tolerance):
    from harness import TOLERANCE
    from pulsarlm_b200.cache.manager import CacheManager
    from pulsarlm_b200.engine.loading import load_model
    from pulsarlm_b200.engine.runner import ModelRunner, StepEntry

    register_toys()
    cfg = dict(tiny.TINY_B, architectures=["ToyRoutedForCausalLM"])
    w = tiny.random_weights(cfg, 4)
    for name in ("gate_proj", "up_proj", "down_proj"):
        del w[f"model.layers.0.mlp.{name}.weight"]
    gen = torch.Generator().manual_seed(5)
    hidden = cfg["hidden_size"]
    w["model.layers.0.mlp.router.weight"] = torch.randn(EXPERTS, hidden, generator=gen)
    w["model.layers.0.mlp.experts_a.weight"] = torch.randn(EXPERTS * EXPERT_WIDTH, hidden, generator=gen) / 8
    w["model.layers.0.mlp.experts_b.weight"] = torch.randn(EXPERTS * hidden, EXPERT_WIDTH, generator=gen) / 8
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}  # what the engine will hold
    folder = tiny.write_model_dir(str(tmp_path), cfg, w)

    model = load_model(folder, dtype, DEV)
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    runner = ModelRunner(model, CacheManager(model.cache_needs(), tiny.PAGE_B, 16, 3, torch_dtype, DEV))

    # Routing is a step function of the router's logits: take prompts whose logits leave
    # a clear margin between the first and the second expert at every token, so that
    # rounding in the engine cannot choose another expert than the plain implementation.
    for seed in range(1, 200):
        a = tiny.random_tokens(cfg, 60, seed)
        b = tiny.random_tokens(cfg, 21, seed + 1000)
        routed = []
        want = {"a": plain_toys(cfg, w, a, routed), "b": plain_toys(cfg, w, b, routed)}
        if min(routed[0][1], routed[1][1]) > 0.25:
            break
    else:
        pytest.fail("no prompt with a clear routing margin among the seeds tried")
    assert len(set(routed[0][0].tolist())) == EXPERTS  # the prompt reaches every expert
    got = {"a": [], "b": []}
    plan = [[("a", a[:33])], [("a", a[33:35]), ("b", b[:20])], [("b", b[20:21]), ("a", a[35:36])],
            [("a", a[36:60])]]
    for step in plan:
        logits = runner.step([StepEntry(r, t, list(range(len(t)))) for r, t in step]).cpu()
        at = 0
        for r, t in step:
            got[r].append(logits[at : at + len(t)])
            at += len(t)
    runner.check_status()
    for r in ("a", "b"):
        err = plain_llama.max_relative_error(torch.cat(got[r]), want[r])
        assert err < (tolerance or TOLERANCE["bfloat16"]), (r, err)
