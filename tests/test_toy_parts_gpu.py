"""A feed-forward with routing and a position encoding of another kind, both defined here, registered,
built from a config.json and stepped, without a change to the framework's files.

The toy feed-forward sends every token to the one of three small experts that its router prefers
(router logits and softmax in 32-bit) and scales the expert's output by the router's probability.
The toy position encoding is not rotary: it adds sin / cos of position-dependent angles to q and k
(the attention part then takes its unfused path: norm, `apply`, cache write).
"""
import math
from dataclasses import dataclass

import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

TOY = {
    "architectures": ["ToyRoutedForCausalLM"], "vocab_size": 157, "hidden_size": 40, "num_hidden_layers": 3,
    "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 56,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False, "torch_dtype": "float32",
    "max_position_embeddings": 128,
    "routed_layers": [0, 2], "n_experts": 3, "expert_size": 24, "additive_position_layers": [1], "position_scale": 0.5,
}


def additive_position(x, positions, scale):
    """x[T, H, D] + scale * [sin(p w_0), cos(p w_0), sin(p w_1), ...] with w_i = 1 / 50^(2i/D)."""
    D = x.shape[-1]
    i = torch.arange(D // 2, dtype=torch.float64)
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] / (50.0 ** (2 * i / D))[None, :]
    enc = torch.stack([ang.sin(), ang.cos()], dim=-1).reshape(len(positions), D)
    return x + scale * enc[:, None, :].to(device=x.device, dtype=x.dtype)


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from imp_b200 import register_architecture, register_part, write_model_folder
    from imp_b200.architectures.qwen3 import qwen3_plan
    from imp_b200.config.model_config import Qwen3Config
    from imp_b200.config.registry import config_from_dict, unregister_architecture
    from imp_b200.parts.base import FeedForward, PositionEncoding
    from imp_b200.parts.plan import PartSpec, TensorSpec
    from imp_b200.parts.registry import unregister_part

    class ToyRouted(FeedForward):
        """y_t = p_t[e] * W2[e] relu(W1[e] x_t), e = argmax of the router's logits, p = softmax of them."""

        @classmethod
        def tensor_specs(cls, params):
            d, f, n = params["hidden_size"], params["expert_size"], params["n_experts"]
            specs = {"router": TensorSpec((n, d))}
            for e in range(n):
                specs[f"w1_{e}"] = TensorSpec((f, d))
                specs[f"w2_{e}"] = TensorSpec((d, f))
            return specs

        def forward(self, x, ctx):
            n = self.params["n_experts"]
            logits = x.float() @ self.tensors["router"].float().T          # routing in 32-bit
            prob = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            out = torch.zeros_like(x)
            for e in range(n):
                rows = (choice == e).nonzero(as_tuple=True)[0]
                if rows.numel() == 0:
                    continue
                hid = torch.relu(x[rows].float() @ self.tensors[f"w1_{e}"].float().T)
                y = (hid @ self.tensors[f"w2_{e}"].float().T) * prob[rows, e:e + 1]
                out[rows] = y.to(x.dtype)
            return out

    class ToyAdditivePosition(PositionEncoding):
        def apply(self, q, k, ctx):
            pos = ctx.positions.tolist()
            q.copy_(additive_position(q.float(), pos, self.params["scale"]).to(q.dtype))
            k.copy_(additive_position(k.float(), pos, self.params["scale"]).to(k.dtype))

    class ToyConfig(Qwen3Config):
        pass

    def toy_plan(cfg):
        plan = qwen3_plan(cfg)
        x = cfg.extra
        for i in x["routed_layers"]:
            names = {"router": f"model.layers.{i}.moe.router.weight"}
            for e in range(x["n_experts"]):
                names[f"w1_{e}"] = f"model.layers.{i}.moe.experts.{e}.w1.weight"
                names[f"w2_{e}"] = f"model.layers.{i}.moe.experts.{e}.w2.weight"
            plan.layers[i].feed_forward = PartSpec(
                "toy_routed", {"hidden_size": cfg.hidden_size, "expert_size": x["expert_size"], "n_experts": x["n_experts"]},
                names)
        for i in x["additive_position_layers"]:
            plan.layers[i].mixer.params = dict(plan.layers[i].mixer.params,
                                               position=PartSpec("toy_additive", {"scale": x["position_scale"]}))
        return plan

    register_part("feed_forward", "toy_routed", ToyRouted)
    register_part("position", "toy_additive", ToyAdditivePosition)
    register_architecture("ToyRoutedForCausalLM", ToyConfig, toy_plan)
    folder = str(tmp_path_factory.mktemp("toy_routed"))
    write_model_folder(folder, config_from_dict(TOY), seed=13, std=0.15)
    yield folder
    unregister_architecture("ToyRoutedForCausalLM")
    unregister_part("feed_forward", "toy_routed")
    unregister_part("position", "toy_additive")


def plain_logits(folder, ids):
    """Whole-sequence computation, written out from the plain parts."""
    cfg = P.read_config(folder)
    w = P.read_weights(folder)
    T = len(ids)
    pos = list(range(T))
    Hq, Hkv, D, eps = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["eps"]
    h = P.embedding(w["model.embed_tokens.weight"], ids)
    for layer in range(TOY["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        x = P.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        q = P.rmsnorm((x @ w[p + "self_attn.q_proj.weight"].T).view(T, Hq, D), w[p + "self_attn.q_norm.weight"], eps)
        k = P.rmsnorm((x @ w[p + "self_attn.k_proj.weight"].T).view(T, Hkv, D), w[p + "self_attn.k_norm.weight"], eps)
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(T, Hkv, D)
        if layer in TOY["additive_position_layers"]:
            q, k = additive_position(q, pos, TOY["position_scale"]), additive_position(k, pos, TOY["position_scale"])
        else:
            q, k = P.rope(q, pos, cfg["theta"]), P.rope(k, pos, cfg["theta"])
        h = h + P.attention(q, k, v).reshape(T, Hq * D) @ w[p + "self_attn.o_proj.weight"].T
        x = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        if layer in TOY["routed_layers"]:
            logits = x @ w[p + "moe.router.weight"].T
            prob = torch.softmax(logits, dim=-1)
            y = torch.zeros_like(x)
            for t in range(T):
                e = int(logits[t].argmax())
                hid = torch.relu(w[p + f"moe.experts.{e}.w1.weight"] @ x[t])
                y[t] = prob[t, e] * (w[p + f"moe.experts.{e}.w2.weight"] @ hid)
            h = h + y
        else:
            h = h + P.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.rmsnorm(h, w["model.norm.weight"], eps) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(toy_folder, dtype):
    from imp_b200 import Engine, EngineConfig, GenerateParams, StepEntry
    eng = Engine.from_folder(toy_folder, EngineConfig(compute_dtype=dtype, kv_block_size=8, max_batch_size=3,
                                                      max_seq_len=128, kv_cache_tokens=512, max_batch_tokens=64))
    layers = eng.model.plan_json()["layers"]
    assert [l["parts"]["feed_forward"]["kind"] for l in layers] == ["toy_routed", "swiglu", "toy_routed"]
    assert [l["parts"]["mixer"]["params"]["position"]["kind"] for l in layers] == ["rotary", "toy_additive", "rotary"]

    def step(entries):
        return torch.from_numpy(eng.step_tokens(entries))

    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, TOY["vocab_size"], (37,), generator=g).tolist()
    b = torch.randint(0, TOY["vocab_size"], (11,), generator=g).tolist()
    ref_a, ref_b = plain_logits(toy_folder, a), plain_logits(toy_folder, b)
    if dtype == "float32":
        def check(got, want, what):
            err = (got - want).abs()
            assert (err <= 2e-4 + 2e-4 * want.abs()).all(), f"{what}: max error {err.max():.3g}"
    else:
        # in bfloat16 a token near a tie of its router may go to another expert: compare where the choice is clear
        def check(got, want, what):
            scale = float(want.abs().max())
            bad = ((got - want).abs() > 0.04 * scale + 0.04 * want.abs()).any(dim=-1)
            assert bad.float().mean() <= 0.15, f"{what}: {int(bad.sum())} of {bad.numel()} rows differ"
    whole = step([StepEntry("a", a, list(range(len(a))))])
    eng.end("a")
    check(whole, ref_a, "whole")
    rows_a, rows_b, ia, ib = [], [], 0, 0
    for n in (6, 2, 13, 1, 15):
        entries = [StepEntry("a2", a[ia:ia + n], list(range(n)))]
        if ib < len(b):
            entries.append(StepEntry("b", [b[ib]], [0]))
        lg = step(entries)
        rows_a.append(lg[:n])
        if ib < len(b):
            rows_b.append(lg[n:])
            ib += 1
        ia += n
    eng.end("a2")
    while ib < len(b):
        rows_b.append(step([StepEntry("b", [b[ib]], [0])]))
        ib += 1
    eng.end("b")
    check(torch.cat(rows_a), ref_a, "portions")
    check(torch.cat(rows_b), ref_b, "token by token")
    if dtype == "float32":
        ids = list(a[:5])
        want = []
        for _ in range(6):
            tok = int(torch.argmax(plain_logits(toy_folder, ids)[-1]))
            want.append(tok)
            ids.append(tok)
        assert eng.generate([a[:5]], GenerateParams(max_tokens=6, temperature=0.0))[0] == want
    eng.check_invariants()
    assert eng.free_pages() == eng.num_pages
