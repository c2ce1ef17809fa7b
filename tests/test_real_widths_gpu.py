"""The engine at the layer widths of three real models, two layers each and a reduced, odd vocabulary,
against the plain implementation: the shapes at which the tensor-memory GEMMs (single CTAs, CTA pairs,
swap-AB), the weight-streaming GEMM with 32-row tiles and the tensor-memory attention run in the
benchmarks, here checked for their numbers.

  8b    hidden 4096, 32 query / 8 kv heads of 128, inner 12288, separate head
  0.6b  hidden 1024 (not heads x head size), 16 / 8 heads of 128: two query heads a kv head, inner 3072, tied head
  14b   hidden 5120, 40 / 8 heads of 128: FIVE query heads a kv head (an odd group for the attention kernels
        that take one or two heads of a group per CTA), inner 17408 = 68 x 256 (a ragged last tile column
        for the CTA-pair product)
"""
import shutil

import numpy as np
import pytest
import torch

from plain.qwen3_plain import PlainModel

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 32003, "hidden_size": 4096, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    "max_position_embeddings": 1024,
}
SHAPES = {
    "8b": WIDE,
    "0.6b": dict(WIDE, vocab_size=30011, hidden_size=1024, num_attention_heads=16, intermediate_size=3072, tie_word_embeddings=True),
    "14b": dict(WIDE, vocab_size=15013, hidden_size=5120, num_attention_heads=40, intermediate_size=17408),
}
ALL_SHAPES = pytest.mark.parametrize("wide", list(SHAPES), indirect=True)
ONLY_8B = pytest.mark.parametrize("wide", ["8b"], indirect=True)


@pytest.fixture(scope="module")
def wide(request, tmp_path_factory):
    from imp_b200.config.registry import config_from_dict
    from imp_b200.weights.random_init import write_model_folder
    config = SHAPES[request.param]
    folder = str(tmp_path_factory.mktemp("wide"))
    write_model_folder(folder, config_from_dict(config), seed=3, std=0.02)
    g = torch.Generator().manual_seed(8)
    ids = {name: torch.randint(0, config["vocab_size"], (n,), generator=g).tolist()
           for name, n in (("a", 300), ("b", 140), ("c", 33))}
    plain = PlainModel(folder)
    ref = {name: plain.logits(v) for name, v in ids.items()}
    del plain
    yield folder, ids, ref
    shutil.rmtree(folder, ignore_errors=True)


def run(eng, ids, plan):
    """plan: list of steps, each a list of (request, n tokens); returns {request: logits of all its rows}."""
    from imp_b200 import StepEntry
    done = {k: 0 for k in ids}
    rows = {k: [] for k in ids}
    for step in plan:
        entries = [StepEntry(r, ids[r][done[r]:done[r] + n], list(range(n))) for r, n in step]
        lg = torch.from_numpy(eng.step_tokens(entries))
        at = 0
        for r, n in step:
            rows[r].append(lg[at:at + n])
            at += n
            done[r] += n
    for r in ids:
        if done[r]:
            assert done[r] == len(ids[r])
            eng.end(r)
    return {r: torch.cat(v) for r, v in rows.items() if v}


def engine(folder, dtype):
    from imp_b200 import Engine, EngineConfig
    return Engine.from_folder(folder, EngineConfig(compute_dtype=dtype, kv_block_size=16, max_batch_size=24, max_seq_len=512,
                                                   kv_cache_tokens=24 * 512, max_batch_tokens=640))


@ALL_SHAPES
def test_bfloat16_at_real_widths(wide):
    folder, ids, ref = wide
    eng = engine(folder, "bfloat16")

    def check(got, what):
        for r, lg in got.items():
            want = ref[r]
            scale = float(want.abs().max())
            err = (lg - want).abs()
            assert (err <= 0.03 * scale + 0.03 * want.abs()).all(), f"{what}, request {r}: max error {float(err.max()):.3g} of {scale:.3g}"
            # the most likely token agrees wherever it is clearly ahead
            top2 = torch.topk(want, 2, dim=-1).values
            clear = (top2[:, 0] - top2[:, 1]) > 0.1 * scale
            assert (lg.argmax(-1)[clear] == want.argmax(-1)[clear]).all(), f"{what}, request {r}: argmax differs"

    # whole prompts: 300 rows on CTA pairs, 140 on single CTAs, 33 on the swap-AB kernel; attention in 128-token tiles
    check(run(eng, ids, [[("a", 300)], [("b", 140)], [("c", 33)]]), "whole")
    # portions beside decode tokens: 130 + 100 + the rest of a; b and c token by token for a while, then in portions
    plan = [[("a", 130), ("b", 1), ("c", 1)], [("a", 100), ("b", 1), ("c", 1)], [("b", 70), ("c", 31), ("a", 1)]]
    plan += [[("a", 1), ("b", 1)] for _ in range(20)]
    plan += [[("a", 49), ("b", 48)]]
    check(run(eng, ids, plan), "portions and decode")
    # one step of 320 tokens over three sequences, then the rest: the fused q,k,v epilogue (norm, rotation, page write)
    # of the wide products in a mixed batch, where a tile of rows holds the end of one sequence and the start of another
    check(run(eng, ids, [[("a", 200), ("b", 100), ("c", 20)], [("c", 13), ("a", 100), ("b", 40)]]), "a mixed step of 320 tokens")
    # twenty sequences decoding together (the swap-AB kernel's shape in decode): twenty copies of c, last 3 tokens
    many = {f"c{i}": ids["c"] for i in range(20)}
    from imp_b200 import StepEntry
    eng.step_tokens([StepEntry(r, v[:30], []) for r, v in list(many.items())[:10]])
    eng.step_tokens([StepEntry(r, v[:30], []) for r, v in list(many.items())[10:]])
    for t in range(30, 33):
        lg = torch.from_numpy(eng.step_tokens([StepEntry(r, [v[t]], [0]) for r, v in many.items()]))
        want = ref["c"][t]
        scale = float(want.abs().max())
        assert ((lg - want[None]).abs() <= 0.03 * scale + 0.03 * want.abs()[None]).all(), f"20-way decode at position {t}"
        assert (lg - lg[0:1]).abs().max() <= 0.02 * scale        # the same sequence twenty times: the same logits
    for r in many:
        eng.end(r)
    eng.check_invariants()
    assert eng.free_pages() == eng.num_pages
    assert eng.info()["fallback_calls"] == 0, "a matrix product fell back to the plain kernel"


@ONLY_8B
def test_keys_do_not_depend_on_which_product_kernel_wrote_them(wide):
    """512 tokens whole (q,k,v with norm, rotation and page write in the epilogue of the CTA-pair product), as two
    portions of 256 (the same kernel, the second portion over cached keys) and as four of 128 (a product that writes
    bfloat16, then the separate norm-and-rotation kernel).  All three round the product to bfloat16 before the norm,
    so the logits of the last rows differ by accumulation order only."""
    folder, ids, ref = wide
    from imp_b200 import StepEntry
    eng = engine(folder, "bfloat16")
    g = torch.Generator().manual_seed(21)
    d = torch.randint(0, SHAPES["8b"]["vocab_size"], (512,), generator=g).tolist()
    want = PlainModel(folder).logits(d)[-8:]
    scale = float(want.abs().max())
    got = {}
    for name, cut in (("whole", [512]), ("halves", [256, 256]), ("quarters", [128] * 4)):
        at = 0
        for n in cut:
            last = at + n == 512
            lg = eng.step_tokens([StepEntry(name, d[at:at + n], list(range(n - 8, n)) if last else [])])
            at += n
        got[name] = torch.from_numpy(lg)
        eng.end(name)
        err = (got[name] - want).abs()
        assert (err <= 0.03 * scale + 0.03 * want.abs()).all(), f"{name}: max error {float(err.max()):.3g} of {scale:.3g}"
    for name in ("halves", "quarters"):
        diff = float((got[name] - got["whole"]).abs().max())
        assert diff <= 0.01 * scale, f"{name} against whole: {diff:.3g} of {scale:.3g}"
    assert eng.info()["fallback_calls"] == 0


@ALL_SHAPES
def test_float32_at_real_widths_is_exact_under_cutting(wide):
    folder, ids, ref = wide
    eng = engine(folder, "float32")
    small = {"b": ids["b"], "c": ids["c"]}
    whole = run(eng, small, [[("b", 140)], [("c", 33)]])
    for r, lg in whole.items():
        err = (lg - ref[r]).abs()
        assert (err <= 2e-3 + 2e-3 * ref[r].abs()).all(), f"request {r}: max error {float(err.max()):.3g}"
    cut = run(eng, small, [[("b", 70), ("c", 2)], [("b", 69), ("c", 30)], [("b", 1), ("c", 1)]])
    for r in small:
        assert np.array_equal(whole[r].numpy(), cut[r].numpy()), f"request {r}: logits depend on the cut"


@ONLY_8B
def test_a_norm_that_knows_nothing_of_unsummed_branches_gets_tensors(wide, tmp_path, monkeypatch):
    """Products of few rows leave their K-split partial sums to the norm that reads them next, but only to a norm
    that says it takes them.  Here the second norm of layer 1 and the final norm are a norm defined in this test
    (the same formula, in torch): it must be handed plain tensors, the built-in norms around it still get unsummed
    branches, and the logits are those of the built-in model (the random weights depend on seed and tensor name
    only)."""
    from dataclasses import dataclass

    from imp_b200 import Engine, EngineConfig, StepEntry, register_architecture, register_part, write_model_folder
    from imp_b200.architectures.qwen3 import qwen3_plan
    from imp_b200.config.model_config import Qwen3Config
    from imp_b200.config.registry import config_from_dict, unregister_architecture
    from imp_b200.parts.base import Norm
    from imp_b200.parts.plan import PartSpec, TensorSpec
    from imp_b200.parts.registry import unregister_part

    seen = {"toy": 0}

    class TorchRMSNorm(Norm):
        @classmethod
        def tensor_specs(cls, params):
            return {"weight": TensorSpec((params["size"],), role="norm", init="one_plus_normal")}

        def add_norm(self, h, branch, rows=None):
            assert branch is None or isinstance(branch, torch.Tensor), type(branch)
            seen["toy"] += 1
            v = h if branch is None else h + branch.float()
            if rows is None:
                if branch is not None:
                    h.copy_(v)
            else:
                v = v[rows.long()]
            y = v * torch.rsqrt((v * v).mean(dim=-1, keepdim=True) + self.params["eps"]) * self.tensors["weight"].float()
            return y.to(branch.dtype if branch is not None else torch.bfloat16)

    class ToyNormConfig(Qwen3Config):
        pass

    def plan_with_toy_norms(cfg):
        plan = qwen3_plan(cfg)
        last = plan.layers[-1]
        last.ffn_norm = PartSpec("torch_rms", last.ffn_norm.params, last.ffn_norm.tensors)
        plan.final_norm = PartSpec("torch_rms", plan.final_norm.params, plan.final_norm.tensors)
        return plan

    register_part("norm", "torch_rms", TorchRMSNorm)
    register_architecture("ToyNormForCausalLM", ToyNormConfig, plan_with_toy_norms)
    try:
        folder = str(tmp_path / "toy_norm")
        write_model_folder(folder, config_from_dict(dict(WIDE, architectures=["ToyNormForCausalLM"])), seed=3, std=0.02)
        eng = Engine.from_folder(folder, EngineConfig(compute_dtype="bfloat16", kv_block_size=16, max_batch_size=24,
                                                      max_seq_len=512, kv_cache_tokens=24 * 512, max_batch_tokens=640))
        model = eng.info()["model"]
        assert model["mixer_defer_out"] == [True, False] and model["defer_pending"] == [True, False]
        assert not model["graph_safe"]
        _, ids, ref = wide
        c = ids["c"]
        many = [f"c{i}" for i in range(20)]
        eng.step_tokens([StepEntry(r, c[:30], []) for r in many[:10]])
        eng.step_tokens([StepEntry(r, c[:30], []) for r in many[10:]])
        seen["toy"] = 0
        before = eng.info()["split_norm_calls"]
        for t in range(30, 33):
            lg = torch.from_numpy(eng.step_tokens([StepEntry(r, [c[t]], [0]) for r in many]))
            want = ref["c"][t]
            scale = float(want.abs().max())
            assert ((lg - want[None]).abs() <= 0.03 * scale + 0.03 * want.abs()[None]).all(), f"position {t}"
        # three steps: the own norm ran twice a step, and the two built-in norms before it got unsummed branches
        assert seen["toy"] == 6 and eng.info()["split_norm_calls"] - before == 6
        for r in many:
            eng.end(r)
    finally:
        unregister_architecture("ToyNormForCausalLM")
        unregister_part("norm", "torch_rms")
