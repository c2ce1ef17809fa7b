"""A part written in CUDA against the C extension interface alone (tests/c_ext/toy_c_rmsnorm.cu: no Python in it),
compiled here with nvcc, loaded beside the engine's library and registered through imp_register_part: a model whose
plan names the kind for some of its norms loads, steps and matches the plain computation in both precisions."""
import ctypes
import json
import os
import subprocess

import pytest
import torch

from plain.qwen3_plain import PlainModel

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CFG = {
    "architectures": ["ToyCNormForCausalLM"], "vocab_size": 197, "hidden_size": 72, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 120, "rms_norm_eps": 3e-6,
    "rope_theta": 40000.0, "tie_word_embeddings": False, "torch_dtype": "bfloat16", "max_position_embeddings": 256,
}


@pytest.fixture(scope="module")
def c_part(tmp_path_factory):
    from imp_b200 import capi
    lib = capi.load()                                   # the engine's library: the extension links against it
    lib_path = capi.loaded_library_path()
    out = str(tmp_path_factory.mktemp("c_ext") / "libtoy_c_rmsnorm.so")
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-I", os.path.join(ROOT, "include"), os.path.join(HERE, "c_ext", "toy_c_rmsnorm.cu"), "-o", out,
           "-L", os.path.dirname(lib_path), "-l:" + os.path.basename(lib_path), "-Xlinker", "-rpath=" + os.path.dirname(lib_path)]
    p = subprocess.run(cmd, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-2000:]
    ext = ctypes.CDLL(out)
    assert ext.toy_c_register() == 0
    assert "toy_c_rmsnorm" in json.loads(lib.imp_known_parts(b"norm").decode())
    yield ext
    assert ext.toy_c_unregister() == 0


@pytest.fixture(scope="module")
def folder(c_part, tmp_path_factory):
    from imp_b200 import register_architecture, write_model_folder
    from imp_b200.architectures.qwen3 import qwen3_plan
    from imp_b200.config.model_config import Qwen3Config
    from imp_b200.config.registry import config_from_dict, unregister_architecture
    from imp_b200.parts.plan import PartSpec

    class ToyCConfig(Qwen3Config):
        pass

    def plan(cfg):
        p = qwen3_plan(cfg)

        def c_norm(spec):
            return PartSpec("toy_c_rmsnorm", spec.params, spec.tensors)
        p.layers[0].ffn_norm = c_norm(p.layers[0].ffn_norm)
        p.layers[1].mixer_norm = c_norm(p.layers[1].mixer_norm)
        p.layers[2].mixer_norm = c_norm(p.layers[2].mixer_norm)
        p.layers[2].ffn_norm = c_norm(p.layers[2].ffn_norm)
        p.final_norm = c_norm(p.final_norm)
        return p

    register_architecture("ToyCNormForCausalLM", ToyCConfig, plan)
    path = str(tmp_path_factory.mktemp("toy_c_model"))
    write_model_folder(path, config_from_dict(CFG), seed=23, std=0.08)
    yield path
    unregister_architecture("ToyCNormForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_norm_written_in_c_runs_inside_the_model(folder, dtype):
    from imp_b200 import Engine, EngineConfig, GenerateParams, StepEntry
    eng = Engine.from_folder(folder, EngineConfig(compute_dtype=dtype, kv_block_size=8, max_batch_size=3, max_seq_len=128,
                                                  kv_cache_tokens=512, max_batch_tokens=64))
    kinds = [part["kind"] for layer in eng.model.plan_json()["layers"] for slot, part in layer["parts"].items() if "norm" in slot]
    assert kinds.count("toy_c_rmsnorm") == 4
    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, CFG["vocab_size"], (41,), generator=g).tolist()
    b = torch.randint(0, CFG["vocab_size"], (12,), generator=g).tolist()
    plain = PlainModel(folder)
    ref_a, ref_b = plain.logits(a), plain.logits(b)
    scale = float(ref_a.abs().max())
    atol, rtol = (2e-4, 2e-4) if dtype == "float32" else (0.03 * scale, 0.03)

    def check(got, want, what):
        err = (torch.from_numpy(got) - want).abs()
        assert (err <= atol + rtol * want.abs()).all(), f"{what}: max error {err.max():.3g}"

    check(eng.step_tokens([StepEntry("a", a, list(range(len(a))))]), ref_a, "whole")
    eng.end("a")
    # portions of one request beside single tokens of another; the final norm (in C) gathers the wanted rows
    rows_a, rows_b, ia, ib = [], [], 0, 0
    for n in (5, 2, 17, 1, 16):
        entries = [StepEntry("a2", a[ia:ia + n], list(range(n)))]
        if ib < len(b):
            entries.append(StepEntry("b", [b[ib]], [0]))
        lg = eng.step_tokens(entries)
        rows_a.append(lg[:n])
        if ib < len(b):
            rows_b.append(lg[n:])
            ib += 1
        ia += n
    check(__import__("numpy").concatenate(rows_a), ref_a, "portions")
    check(__import__("numpy").concatenate(rows_b), ref_b[:ib], "token by token")
    eng.end("a2")
    eng.end("b")
    if dtype == "float32":
        assert eng.generate([a[:7]], GenerateParams(max_tokens=5, temperature=0.0))[0] == plain.generate(a[:7], 5)
    info = eng.info()
    assert not info["model"]["graph_safe"] and info["graph_replays"] == 0      # a part outside the library: no captured graphs
    eng.check_invariants()
    assert eng.free_pages() == eng.num_pages
