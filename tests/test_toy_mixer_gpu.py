"""A mixer with state of its own, a layer that is run twice and a layer that reads another layer's
cache, all defined here, registered, built from a config.json, stepped and generated with, without
a change to the framework's files.

The toy mixer is a causal running mean: y_t = W * mean(x_0 .. x_t).  Its state lives in the cache
manager's fixed-size state slots, as two tensors of different types per request and run position:
the running sum (a float32 vector) and the number of tokens seen (one int32).
"""
import math
from dataclasses import dataclass

import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

TOY = {
    "architectures": ["ToyMeanForCausalLM"], "vocab_size": 211, "hidden_size": 48, "num_hidden_layers": 4,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 72,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": True, "torch_dtype": "float32",
    "max_position_embeddings": 256,
    "toy_layers": [1], "shared_cache": {"2": 0}, "run_order": [0, 1, 2, 3, 1],
}


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from imp_b200 import register_architecture, register_part, write_model_folder
    from imp_b200.architectures.qwen3 import qwen3_plan
    from imp_b200.cache.manager import StateSpec
    from imp_b200.config.model_config import Qwen3Config
    from imp_b200.config.registry import config_from_dict, unregister_architecture
    from imp_b200.parts.base import Mixer
    from imp_b200.parts.plan import PartSpec, TensorSpec
    from imp_b200.parts.registry import unregister_part

    class ToyMean(Mixer):
        @classmethod
        def tensor_specs(cls, params):
            return {"w": TensorSpec((params["hidden_size"], params["hidden_size"]))}

        @classmethod
        def cache_spec(cls, params):
            return StateSpec(tensors=(("sum", (params["hidden_size"],), "float32"), ("count", (1,), "int32")))

        def forward(self, x, ctx, cache):
            w = self.tensors["w"].float()
            out = torch.empty_like(x)
            total, count = cache.states
            assert total.dtype == torch.float32 and count.dtype == torch.int32
            t0 = 0
            for n, start, slot, fresh in zip(ctx.q_lens, ctx.starts, ctx.slots, ctx.fresh):
                seen = int(count[slot, 0])
                assert seen == start and (seen == 0) == fresh      # a fresh request's state starts at zero
                sums = torch.cumsum(x[t0:t0 + n].float(), 0) + total[slot]
                if cache.writes:
                    total[slot] = sums[-1]
                    count[slot, 0] = seen + n
                counts = torch.arange(seen + 1, seen + n + 1, device=x.device, dtype=torch.float32)
                out[t0:t0 + n] = ((sums / counts[:, None]) @ w.T).to(x.dtype)
                t0 += n
            return out

    class ToyConfig(Qwen3Config):
        pass

    def toy_plan(cfg):
        plan = qwen3_plan(cfg)
        for i in cfg.extra["toy_layers"]:
            plan.layers[i].mixer = PartSpec("toy_mean", {"hidden_size": cfg.hidden_size},
                                            {"w": f"model.layers.{i}.toy.w"})
        for i, src in cfg.extra["shared_cache"].items():
            plan.layers[int(i)].cache_from = int(src)
        plan.order = list(cfg.extra["run_order"])
        return plan

    register_part("mixer", "toy_mean", ToyMean)
    register_architecture("ToyMeanForCausalLM", ToyConfig, toy_plan)
    folder = str(tmp_path_factory.mktemp("toy"))
    write_model_folder(folder, config_from_dict(TOY), seed=11, std=0.1)
    yield folder
    unregister_architecture("ToyMeanForCausalLM")
    unregister_part("mixer", "toy_mean")


def plain_toy_logits(folder, ids):
    """Whole-sequence computation of the toy model, written out by hand from the plain parts."""
    cfg = P.read_config(folder)
    w = P.read_weights(folder)
    T = len(ids)
    pos = list(range(T))
    Hq, Hkv, D, eps = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["eps"]
    h = P.embedding(w["model.embed_tokens.weight"], ids)
    kv_of_layer = {}
    for layer in TOY["run_order"]:
        p = f"model.layers.{layer}."
        x = P.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        if layer in TOY["toy_layers"]:
            counts = torch.arange(1, T + 1, dtype=x.dtype)[:, None]
            a = (torch.cumsum(x, 0) / counts) @ w[p + "toy.w"].T
        else:
            q = P.rope(P.rmsnorm((x @ w[p + "self_attn.q_proj.weight"].T).view(T, Hq, D),
                                 w[p + "self_attn.q_norm.weight"], eps), pos, cfg["theta"])
            if str(layer) in TOY["shared_cache"]:
                k, v = kv_of_layer[TOY["shared_cache"][str(layer)]]
            else:
                k = P.rope(P.rmsnorm((x @ w[p + "self_attn.k_proj.weight"].T).view(T, Hkv, D),
                                     w[p + "self_attn.k_norm.weight"], eps), pos, cfg["theta"])
                v = (x @ w[p + "self_attn.v_proj.weight"].T).view(T, Hkv, D)
                kv_of_layer[layer] = (k, v)
            a = P.attention(q, k, v).reshape(T, Hq * D) @ w[p + "self_attn.o_proj.weight"].T
        h = h + a
        x = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + P.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.rmsnorm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_built_and_stepped(toy_folder, dtype):
    from imp_b200 import Engine, EngineConfig, GenerateParams, StepEntry
    eng = Engine.from_folder(toy_folder, EngineConfig(compute_dtype=dtype, kv_block_size=4, max_batch_size=3,
                                                      max_seq_len=128, kv_cache_tokens=512, max_batch_tokens=64))
    # run positions 0 and 3 own pages, position 2 reads position 0's, positions 1 and 4 own state
    info = eng.info()
    assert [s["kind"] if s else None for s in info["model"]["cache_specs"]] == ["paged", "state", None, "paged", "state"]
    assert info["model"]["cache_position"] == [0, 1, 0, 3, 4]
    assert len(info["cache"]["paged"]) == 1 and len(info["cache"]["state"]) == 1
    assert info["cache"]["state"][0]["layers"] == [1, 4] and len(info["cache"]["state"][0]["tensors"]) == 2
    assert not info["model"]["graph_safe"], "a part written in Python keeps CUDA graphs off for its model"
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, TOY["vocab_size"], (29,), generator=g).tolist()
    b = torch.randint(0, TOY["vocab_size"], (13,), generator=g).tolist()
    ref_a, ref_b = plain_toy_logits(toy_folder, a), plain_toy_logits(toy_folder, b)
    scale = float(ref_a.abs().max())
    atol, rtol = (2e-4, 2e-4) if dtype == "float32" else (0.03 * scale, 0.03)

    def check(got, want, what):
        err = (got - want).abs()
        assert (err <= atol + rtol * want.abs()).all(), f"{what}: max error {err.max():.3g}"

    def step(entries):
        return torch.from_numpy(eng.step_tokens(entries))

    whole = step([StepEntry("a", a, list(range(29)))])
    eng.end("a")
    check(whole, ref_a, "whole")
    # portions of a beside single tokens of b; a's slot is reused after it ends
    rows_a, rows_b, ia, ib = [], [], 0, 0
    for n in (5, 2, 9, 1, 12):
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
        # greedy generation through the scheduler, state slots and all
        ids = list(a[:6])
        want = []
        for _ in range(8):
            tok = int(torch.argmax(plain_toy_logits(toy_folder, ids)[-1]))
            want.append(tok)
            ids.append(tok)
        assert eng.generate([a[:6], b[:3]], GenerateParams(max_tokens=8, temperature=0.0))[0] == want
    eng.check_invariants()
    assert eng.free_pages() == eng.num_pages and eng.info()["cache"]["free_slots"] == 3
