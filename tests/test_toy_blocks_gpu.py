"""Two block arrangements that the library does not have, defined here, registered, built from a
config.json and stepped, without a change to the framework's files:

  * a sandwich-norm block: norms before AND after both branches (six part slots, four norms of its own
    around a mixer and a feed-forward);
  * a parallel-residual block: one norm feeds the mixer and the feed-forward side by side (three slots).

A layer is a block kind plus the parts in the slots that block declares, so a plan can carry any number
of norms per layer; the blocks here run the library's own attention, SwiGLU and RMSNorm parts through
their handles.  One model mixes both with the library's pre-norm block, layer by layer.
"""
import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

TOY = {
    "architectures": ["ToyBlocksForCausalLM"], "vocab_size": 173, "hidden_size": 56, "num_hidden_layers": 4,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 88,
    "rms_norm_eps": 2e-5, "rope_theta": 20000.0, "tie_word_embeddings": True, "torch_dtype": "float32",
    "max_position_embeddings": 128,
    "block_kinds": ["toy_sandwich", "toy_parallel", "prenorm", "toy_sandwich"],
}


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from imp_b200 import register_architecture, register_part, write_model_folder
    from imp_b200.architectures.qwen3 import qwen3_plan
    from imp_b200.config.model_config import Qwen3Config
    from imp_b200.config.registry import config_from_dict, unregister_architecture
    from imp_b200.parts.base import Block
    from imp_b200.parts.plan import LayerSpec, PartSpec
    from imp_b200.parts.registry import unregister_part

    class SandwichBlock(Block):
        """h += post1(mixer(pre1(h))); h += post2(ffn(pre2(h))); the second sum is left pending."""

        @classmethod
        def part_slots(cls, params):
            return [("pre_mixer_norm", "norm"), ("mixer", "mixer"), ("post_mixer_norm", "norm"),
                    ("pre_ffn_norm", "norm"), ("feed_forward", "feed_forward"), ("post_ffn_norm", "norm")]

        def forward(self, h, pending, ctx, cache):
            p = self.parts
            x = p["pre_mixer_norm"].add_norm(h, pending)                  # adds what the block before left pending
            a = p["mixer"].forward(x, ctx, cache)
            h.add_(p["post_mixer_norm"].add_norm(a.float(), None).float())
            x = p["pre_ffn_norm"].add_norm(h, None)
            f = p["feed_forward"].forward(x, ctx)
            return p["post_ffn_norm"].add_norm(f.float(), None)

    class ParallelBlock(Block):
        """h += mixer(norm(h)) + ffn(norm(h)): one norm, both branches from the same activations."""

        @classmethod
        def part_slots(cls, params):
            return [("norm", "norm"), ("mixer", "mixer"), ("feed_forward", "feed_forward")]

        def forward(self, h, pending, ctx, cache):
            p = self.parts
            x = p["norm"].add_norm(h, pending)
            a = p["mixer"].forward(x, ctx, cache)
            f = p["feed_forward"].forward(x, ctx)
            return (a.float() + f.float()).to(a.dtype)

    class ToyConfig(Qwen3Config):
        pass

    def toy_plan(cfg):
        plan = qwen3_plan(cfg)
        for i, kind in enumerate(cfg.extra["block_kinds"]):
            base = plan.layers[i]
            pre = f"model.layers.{i}."

            def norm(name):
                return PartSpec("rmsnorm", dict(base.mixer_norm.params), {"weight": pre + name + ".weight"})

            if kind == "toy_sandwich":
                plan.layers[i] = LayerSpec("toy_sandwich", {
                    "pre_mixer_norm": base.mixer_norm, "mixer": base.mixer, "post_mixer_norm": norm("post_attention_norm"),
                    "pre_ffn_norm": norm("pre_feedforward_layernorm"), "feed_forward": base.feed_forward,
                    "post_ffn_norm": norm("post_feedforward_layernorm")})
            elif kind == "toy_parallel":
                plan.layers[i] = LayerSpec("toy_parallel", {"norm": base.mixer_norm, "mixer": base.mixer,
                                                            "feed_forward": base.feed_forward})
        return plan

    register_part("block", "toy_sandwich", SandwichBlock)
    register_part("block", "toy_parallel", ParallelBlock)
    register_architecture("ToyBlocksForCausalLM", ToyConfig, toy_plan)
    folder = str(tmp_path_factory.mktemp("toy_blocks"))
    write_model_folder(folder, config_from_dict(TOY), seed=17, std=0.1)
    yield folder
    unregister_architecture("ToyBlocksForCausalLM")
    unregister_part("block", "toy_sandwich")
    unregister_part("block", "toy_parallel")


def plain_logits(folder, ids):
    cfg, w = P.read_config(folder), P.read_weights(folder)
    T, pos = len(ids), list(range(len(ids)))
    Hq, Hkv, D, eps = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["eps"]

    def attn(x, p):
        q = P.rope(P.rmsnorm((x @ w[p + "self_attn.q_proj.weight"].T).view(T, Hq, D), w[p + "self_attn.q_norm.weight"], eps), pos, cfg["theta"])
        k = P.rope(P.rmsnorm((x @ w[p + "self_attn.k_proj.weight"].T).view(T, Hkv, D), w[p + "self_attn.k_norm.weight"], eps), pos, cfg["theta"])
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(T, Hkv, D)
        return P.attention(q, k, v).reshape(T, Hq * D) @ w[p + "self_attn.o_proj.weight"].T

    def ffn(x, p):
        return P.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    h = P.embedding(w["model.embed_tokens.weight"], ids)
    for i, kind in enumerate(TOY["block_kinds"]):
        p = f"model.layers.{i}."
        if kind == "toy_sandwich":
            h = h + P.rmsnorm(attn(P.rmsnorm(h, w[p + "input_layernorm.weight"], eps), p), w[p + "post_attention_norm.weight"], eps)
            h = h + P.rmsnorm(ffn(P.rmsnorm(h, w[p + "pre_feedforward_layernorm.weight"], eps), p),
                              w[p + "post_feedforward_layernorm.weight"], eps)
        elif kind == "toy_parallel":
            x = P.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
            h = h + attn(x, p) + ffn(x, p)
        else:
            h = h + attn(P.rmsnorm(h, w[p + "input_layernorm.weight"], eps), p)
            h = h + ffn(P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps), p)
    return P.rmsnorm(h, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


def test_the_plan_carries_what_each_block_declares(toy_folder):
    from imp_b200 import Model
    m = Model.load(toy_folder)
    layers = m.plan_json()["layers"]
    assert [l["block"] for l in layers] == TOY["block_kinds"]
    assert [len(l["parts"]) for l in layers] == [6, 3, 4, 6]
    names = set(m.tensor_info())
    assert "model.layers.0.post_feedforward_layernorm.weight" in names and "model.layers.3.post_attention_norm.weight" in names
    # the parallel block has one norm: the checkpoint holds no second one for that layer, the pre-norm layer does
    assert "model.layers.1.post_attention_layernorm.weight" not in names and "model.layers.2.post_attention_layernorm.weight" in names


def test_a_block_without_its_part_or_with_a_stray_one_is_a_plan_error():
    from imp_b200 import ConfigError, config_from_dict, plan_for, register_architecture, register_part, unregister_architecture
    from imp_b200.architectures.qwen3 import qwen3_plan
    from imp_b200.config.model_config import Qwen3Config
    from imp_b200.parts.base import Block
    from imp_b200.parts.registry import unregister_part

    class OneNorm(Block):
        @classmethod
        def part_slots(cls, params):
            return [("norm", "norm"), ("mixer", "mixer")]

    def plan_missing(cfg):
        plan = qwen3_plan(cfg)
        plan.layers[0].block = "toy_one_norm"          # its slots are norm and mixer; the layer brings four others
        return plan

    register_part("block", "toy_one_norm", OneNorm)
    register_architecture("ToyBrokenForCausalLM", Qwen3Config, plan_missing)
    try:
        with pytest.raises(ConfigError, match="slot 'norm'"):
            plan_for(config_from_dict(dict(TOY, architectures=["ToyBrokenForCausalLM"])))
    finally:
        unregister_architecture("ToyBrokenForCausalLM")
        unregister_part("block", "toy_one_norm")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sandwich_and_parallel_blocks_match_the_plain_computation(toy_folder, dtype):
    from imp_b200 import Engine, EngineConfig, GenerateParams, StepEntry
    eng = Engine.from_folder(toy_folder, EngineConfig(compute_dtype=dtype, kv_block_size=8, max_batch_size=3, max_seq_len=128,
                                                      kv_cache_tokens=512, max_batch_tokens=64))
    g = torch.Generator().manual_seed(6)
    a = torch.randint(0, TOY["vocab_size"], (33,), generator=g).tolist()
    b = torch.randint(0, TOY["vocab_size"], (9,), generator=g).tolist()
    ref_a, ref_b = plain_logits(toy_folder, a), plain_logits(toy_folder, b)
    scale = float(ref_a.abs().max())
    atol, rtol = (2e-4, 2e-4) if dtype == "float32" else (0.03 * scale, 0.03)

    def check(got, want, what):
        err = (got - want).abs()
        assert (err <= atol + rtol * want.abs()).all(), f"{what}: max error {err.max():.3g}"

    def step(entries):
        return torch.from_numpy(eng.step_tokens(entries))

    check(step([StepEntry("a", a, list(range(len(a))))]), ref_a, "whole")
    eng.end("a")
    rows_a, rows_b, ia, ib = [], [], 0, 0
    for n in (4, 2, 11, 1, 15):
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
        ids, want = list(a[:6]), []
        for _ in range(6):
            want.append(int(torch.argmax(plain_logits(toy_folder, ids)[-1])))
            ids.append(want[-1])
        assert eng.generate([a[:6]], GenerateParams(max_tokens=6, temperature=0.0))[0] == want
    info = eng.info()
    assert not info["model"]["graph_safe"] and info["graph_replays"] == 0
    # a pending sum may stay unsummed only where the next normaliser is the library's own norm (blocks written in Python sum anyway)
    assert info["model"]["defer_pending"] == [False, True, False, True]
    eng.check_invariants()
    assert eng.free_pages() == eng.num_pages
