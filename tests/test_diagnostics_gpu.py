"""The two debugging switches of the forward pass, on tiny configuration A, each in a process of its own
(the switches are read once per process):

  IMP_B200_PROFILE=1        event timers between named stages, CUDA graphs off;
  IMP_B200_DEBUG_FORWARD=1  statistics of every stage's tensor and the ten largest logits.

The stage lists must name the embedding, every layer's mixer and feed-forward, the final norm and the head, in
running order; the timers must add up to the step's device time; the statistics and the top logits must be
those of the plain implementation.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import json, sys
from imp_b200 import Engine, EngineConfig, StepEntry
folder, page, ids = sys.argv[1], int(sys.argv[2]), json.loads(sys.argv[3])
eng = Engine.from_folder(folder, EngineConfig(compute_dtype="float32", kv_block_size=page, max_batch_size=2, max_seq_len=512,
                                              kv_cache_tokens=1024, max_batch_tokens=512))
timed = []
for rep in range(5):                       # the same prompt five times: the averaged timers and the step's own time
    eng.timer_start()
    eng.step_tokens([StepEntry("r%d" % rep, ids, [len(ids) - 1])])
    timed.append(eng.timer_stop())
    eng.end("r%d" % rep)
info = eng.info()
print("RESULT " + json.dumps({"timed_ms": timed, "model": info["model"], "graph_replays": info["graph_replays"]}))
"""


def run(folder, page, ids, **env):
    full = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), **env)
    p = subprocess.run([sys.executable, "-c", SCRIPT, folder, str(page), json.dumps(ids)], env=full, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):]), p.stderr


def stage_names(n_layers):
    names = ["embedding"]
    for i in range(n_layers):
        names += [f"layer{i}.mixer", f"layer{i}.feed_forward"]
    return names + ["final_norm", "head"]


def test_profile_timers_name_every_stage_and_add_up_to_the_step(model_folders):
    folder, cd, page = model_folders["A"]
    ids = torch.randint(0, cd["vocab_size"], (384,), generator=torch.Generator().manual_seed(1)).tolist()
    out, err = run(folder, page, ids, IMP_B200_PROFILE="1")
    prof = out["model"]["profile"]
    assert [s["stage"] for s in prof["stages"]] == stage_names(cd["num_hidden_layers"])
    assert prof["steps"] == 5 and out["graph_replays"] == 0
    assert all(s["ms"] > 0 for s in prof["stages"])
    total = sum(s["ms"] for s in prof["stages"])
    assert abs(total - prof["ms_per_step"]) <= 1e-3 * prof["ms_per_step"]
    # the stages lie inside the step's own device time (events around batch upload, forward pass and the copy of the logits)
    assert prof["last_step_ms"] <= out["timed_ms"][-1] * 1.001
    # a model that is not asked to profile reports nothing and prints nothing
    plain_out, plain_err = run(folder, page, ids)
    assert "profile" not in plain_out["model"] and "[profile]" not in plain_err


def test_profile_timers_cover_the_step_where_the_device_is_the_limit(tmp_path):
    """On the tiny model a step is a few launches long and the time around the forward pass (batch upload, copy of the
    logits) is a third of it.  At a width where the device works for milliseconds the stages must hold the step's time
    to within a tenth."""
    from imp_b200.config.registry import config_from_dict
    from imp_b200.weights.random_init import write_model_folder
    cd = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 2003, "hidden_size": 1024, "num_hidden_layers": 3,
          "num_attention_heads": 8, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 3072, "rms_norm_eps": 1e-6,
          "rope_theta": 1000000.0, "tie_word_embeddings": True, "torch_dtype": "bfloat16", "max_position_embeddings": 512}
    folder = str(tmp_path / "medium")
    write_model_folder(folder, config_from_dict(cd), seed=4, std=0.02)
    ids = torch.randint(0, cd["vocab_size"], (512,), generator=torch.Generator().manual_seed(3)).tolist()
    out, _ = run(folder, 16, ids, IMP_B200_PROFILE="1")
    prof = out["model"]["profile"]
    assert [s["stage"] for s in prof["stages"]] == stage_names(3)
    step_ms, staged_ms = out["timed_ms"][-1], prof["last_step_ms"]
    assert staged_ms <= step_ms * 1.001 and staged_ms >= 0.9 * step_ms, f"stages {staged_ms:.4f} ms of a step of {step_ms:.4f} ms"
    layers = [s["ms"] for s in prof["stages"] if s["stage"].startswith("layer")]
    assert sum(layers) >= 0.8 * prof["ms_per_step"]                   # the time is in the layers, not in the head of 2003 rows


def test_debug_forward_statistics_are_those_of_the_plain_computation(model_folders):
    folder, cd, page = model_folders["A"]
    ids = torch.randint(0, cd["vocab_size"], (40,), generator=torch.Generator().manual_seed(2)).tolist()
    out, err = run(folder, page, ids, IMP_B200_DEBUG_FORWARD="1")
    stages = out["model"]["debug_stages"]
    assert [s["stage"] for s in stages] == stage_names(cd["num_hidden_layers"])
    assert all(s["nan"] == 0 for s in stages)
    assert err.count("[debug_forward] ") >= 5 * (len(stages) + 1)            # printed at every step, with the top logits

    # the same quantities from the plain implementation: embedding rows, each branch's output, normalised last row, logits
    cfg, w = P.read_config(folder), P.read_weights(folder)
    T, pos = len(ids), list(range(len(ids)))
    Hq, Hkv, D, eps = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["eps"]
    want = {}
    h = P.embedding(w["model.embed_tokens.weight"], ids)
    want["embedding"] = h
    for i in range(cfg["layers"]):
        p = f"model.layers.{i}."
        x = P.rmsnorm(h, w[p + "input_layernorm.weight"], eps)
        q = P.rope(P.rmsnorm((x @ w[p + "self_attn.q_proj.weight"].T).view(T, Hq, D), w[p + "self_attn.q_norm.weight"], eps), pos, cfg["theta"])
        k = P.rope(P.rmsnorm((x @ w[p + "self_attn.k_proj.weight"].T).view(T, Hkv, D), w[p + "self_attn.k_norm.weight"], eps), pos, cfg["theta"])
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(T, Hkv, D)
        a = P.attention(q, k, v).reshape(T, Hq * D) @ w[p + "self_attn.o_proj.weight"].T
        want[f"layer{i}.mixer"] = a
        h = h + a
        f = P.swiglu_mlp(P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps), w[p + "mlp.gate_proj.weight"],
                         w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        want[f"layer{i}.feed_forward"] = f
        h = h + f
    last = P.rmsnorm(h[-1:], w["model.norm.weight"], eps)
    want["final_norm"] = last
    logits = last @ w["model.embed_tokens.weight"].T
    want["head"] = logits
    for s in stages:
        t = want[s["stage"]].double()
        scale = float(t.abs().max())
        assert s["shape"] == str(list(t.shape)), (s["stage"], s["shape"])
        for key, value in (("min", float(t.min())), ("max", float(t.max())), ("mean", float(t.mean())), ("l2", float(t.norm()))):
            assert abs(s[key] - value) <= 2e-4 * max(scale, abs(value)) + 1e-6, (s["stage"], key, s[key], value)
    top = out["model"]["debug_top_logits"]
    order = torch.argsort(logits[0], descending=True, stable=True)[:10].tolist()
    assert [t["token"] for t in top] == order
    assert all(abs(t["logit"] - float(logits[0, t["token"]])) <= 2e-4 for t in top)
