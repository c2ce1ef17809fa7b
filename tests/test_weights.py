"""safetensors reading and writing, binding by name, and the one error that lists every mismatch."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from imp_b200.config.registry import config_from_dict, plan_for
from imp_b200.weights.loader import WeightError, device_dtype, load_weights
from imp_b200.weights.random_init import random_tensors, tensor_seed, write_model_folder
from imp_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, save_safetensors


def test_round_trip_all_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "e": torch.empty(0, 4)}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c", "e"] and f.metadata == {"k": "v"}
    for k in t:
        assert f.tensor(k).dtype == t[k].dtype and torch.equal(f.tensor(k), t[k])
    # the library reader agrees with the file this writer made
    from safetensors import safe_open
    with safe_open(p, framework="pt") as g:
        assert torch.equal(g.get_tensor("a"), t["a"])


def test_truncated_and_malformed_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, {"a": torch.randn(64, 64)})
    data = open(p, "rb").read()
    open(p, "wb").write(data[:-100])
    with pytest.raises(SafetensorsError, match="'a'.*outside"):
        SafetensorsFile(p)
    open(p, "wb").write(data[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10) + b"not json!!")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16"):
        SafetensorsFile(p)


def test_random_weights_depend_on_seed_and_name_only():
    plan = plan_for(config_from_dict(TINY_A))
    a = random_tensors(plan, seed=3, std=0.02, dtype=torch.float32)
    b = random_tensors(plan, seed=3, std=0.02, dtype=torch.float32)
    c = random_tensors(plan, seed=4, std=0.02, dtype=torch.float32)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert tensor_seed(3, "x") != tensor_seed(3, "y")
    w = a["model.layers.0.mlp.gate_proj.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = a["model.layers.1.input_layernorm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.01 and 0.003 < n.std().item() < 0.03


def test_folder_loads_and_keeps_storage_precision(model_folders):
    fa, cda, _ = model_folders["A"]   # stored float32
    fb, cdb, _ = model_folders["B"]   # stored bfloat16
    wa = load_weights(fa, plan_for(config_from_dict(cda)), torch.bfloat16, "cpu")
    wb = load_weights(fb, plan_for(config_from_dict(cdb)), torch.bfloat16, "cpu")
    assert all(t.dtype == torch.float32 for t in wa.values())      # a tensor stored in 32-bit stays so
    assert all(t.dtype == torch.bfloat16 for t in wb.values())
    wb32 = load_weights(fb, plan_for(config_from_dict(cdb)), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in wb32.values())
    k = "model.layers.0.self_attn.q_proj.weight"
    assert torch.equal(wb32[k], wb[k].float())
    assert device_dtype(torch.int64, "int_table", torch.bfloat16) == torch.int32
    assert device_dtype(torch.float16, "matrix", torch.bfloat16) == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY_B)
    plan = plan_for(cfg)
    t = random_tensors(plan, seed=0, dtype=torch.bfloat16)
    del t["model.layers.1.self_attn.q_norm.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192, dtype=torch.bfloat16)
    t["model.layers.2.mlp.up_proj.weight"] = torch.zeros(96, 200, dtype=torch.bfloat16)
    cfg.save(str(tmp_path))
    save_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError) as ei:
        load_weights(str(tmp_path), plan, torch.bfloat16, "cpu")
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.q_norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(e.wrong_shape) == 1 and "up_proj" in e.wrong_shape[0] and "[200, 96]" in e.wrong_shape[0]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shapes", "q_norm", "q_proj.bias", "[96, 200]"):
        assert word in msg


def test_tied_config_refuses_a_separate_head(tmp_path):
    cfg = config_from_dict(TINY_A)
    t = random_tensors(plan_for(cfg), seed=0, dtype=torch.float32)
    t["lm_head.weight"] = torch.zeros(256, 64)
    cfg.save(str(tmp_path))
    save_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError, match="unexpected.*lm_head"):
        load_weights(str(tmp_path), plan_for(cfg), torch.float32, "cpu")


def test_sharded_folder(tmp_path):
    cfg = config_from_dict(TINY_A)
    plan = plan_for(cfg)
    t = random_tensors(plan, seed=5, dtype=torch.float32)
    names = sorted(t)
    half = len(names) // 2
    save_safetensors(str(tmp_path / "m-1.safetensors"), {k: t[k] for k in names[:half]})
    save_safetensors(str(tmp_path / "m-2.safetensors"), {k: t[k] for k in names[half:]})
    wm = {k: ("m-1.safetensors" if i < half else "m-2.safetensors") for i, k in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    w = load_weights(str(tmp_path), plan, torch.float32, "cpu")
    assert all(torch.equal(w[k], t[k]) for k in names)


def test_no_weights_file(tmp_path):
    with pytest.raises(SafetensorsError, match="model.safetensors"):
        load_weights(str(tmp_path), plan_for(config_from_dict(TINY_A)), torch.float32, "cpu")
