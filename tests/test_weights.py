"""Checkpoints through the library's loader: the safetensors container, binding by name, the one
error that lists every mismatch, element types on the device, and random weights by (seed, name).
Files are written here with the test folder's own safetensors writer (tests/safetensors_io.py)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from imp_b200 import Model, WeightError, config_from_dict, plan_for, write_model_folder
from imp_b200.capi import ConfigError, SafetensorsError
from safetensors_io import SafetensorsFile, save_safetensors


def folder_tensors(folder):
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return {k: f.tensor(k).clone() for k in f.names()}


def write_folder(tmp_path, cfg, tensors):
    cfg.save(str(tmp_path))
    save_safetensors(str(tmp_path / "model.safetensors"), tensors)
    return str(tmp_path)


def test_the_library_writes_a_file_other_readers_accept(tmp_path):
    write_model_folder(str(tmp_path), config_from_dict(TINY_B), seed=2, std=0.05)
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    plan = plan_for(config_from_dict(TINY_B)).expected_tensors()
    assert sorted(f.names()) == sorted(plan)
    for k, spec in plan.items():
        assert tuple(f.tensor(k).shape) == tuple(spec.shape) and f.tensor(k).dtype == torch.bfloat16
    from safetensors import safe_open
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as g:
        assert torch.equal(g.get_tensor("model.norm.weight"), f.tensor("model.norm.weight"))
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen3ForCausalLM"]


def test_truncated_and_malformed_files(tmp_path):
    cfg = config_from_dict(TINY_A)
    write_model_folder(str(tmp_path), cfg, seed=1)
    p = str(tmp_path / "model.safetensors")
    data = open(p, "rb").read()
    open(p, "wb").write(data[:-100])
    with pytest.raises(SafetensorsError, match="'model.norm.weight'.*outside"):
        Model.load(str(tmp_path))
    open(p, "wb").write(data[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        Model.load(str(tmp_path))
    open(p, "wb").write(struct.pack("<Q", 10) + b"not json!!")
    with pytest.raises(SafetensorsError, match="JSON"):
        Model.load(str(tmp_path))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16"):
        Model.load(str(tmp_path))


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    cfg = config_from_dict(TINY_A)
    a = folder_tensors(write_model_folder(str(tmp_path / "a"), cfg, seed=3, std=0.02))
    b = folder_tensors(write_model_folder(str(tmp_path / "b"), cfg, seed=3, std=0.02))
    c = folder_tensors(write_model_folder(str(tmp_path / "c"), cfg, seed=4, std=0.02))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    # another model with a tensor of the same name and shape gets the same values: only (seed, name) count
    d3 = dict(TINY_A, num_hidden_layers=3)
    d = folder_tensors(write_model_folder(str(tmp_path / "d"), config_from_dict(d3), seed=3, std=0.02))
    assert torch.equal(a["model.layers.1.mlp.up_proj.weight"], d["model.layers.1.mlp.up_proj.weight"])
    assert not torch.equal(a["model.layers.0.mlp.up_proj.weight"], a["model.layers.1.mlp.up_proj.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = a["model.layers.1.input_layernorm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.01 and 0.003 < n.std().item() < 0.03
    big = torch.cat([t.flatten() for k, t in a.items() if "proj" in k]) / 0.02
    assert abs(big.abs().gt(2.0).float().mean().item() - 0.0455) < 0.01     # a normal distribution's tails


def test_folder_loads_and_keeps_storage_precision(model_folders):
    fa, _, _ = model_folders["A"]   # stored float32
    fb, _, _ = model_folders["B"]   # stored bfloat16
    a16, b16 = Model.load(fa).tensor_info("bfloat16"), Model.load(fb).tensor_info("bfloat16")
    assert all(t["stored"] == "F32" and t["device"] == "float32" for t in a16.values())     # stored in 32-bit stays so
    assert all(t["stored"] == "BF16" and t["device"] == "bfloat16" for t in b16.values())
    assert all(t["device"] == "float32" for t in Model.load(fb).tensor_info("float32").values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY_B)
    t = folder_tensors(write_model_folder(str(tmp_path / "src"), cfg, seed=0))
    del t["model.layers.1.self_attn.q_norm.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192, dtype=torch.bfloat16)
    t["model.layers.2.mlp.up_proj.weight"] = torch.zeros(96, 200, dtype=torch.bfloat16)
    (tmp_path / "m").mkdir()
    with pytest.raises(WeightError) as ei:
        Model.load(write_folder(tmp_path / "m", cfg, t))
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.q_norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(e.wrong_shape) == 1 and "up_proj" in e.wrong_shape[0] and "[200, 96]" in e.wrong_shape[0]
    msg = str(e)
    for word in ("missing", "unexpected", "wrong shapes", "q_norm", "q_proj.bias", "[96, 200]"):
        assert word in msg


def test_wrong_element_types_are_errors(tmp_path):
    cfg = config_from_dict(TINY_A)
    t = folder_tensors(write_model_folder(str(tmp_path / "src"), cfg, seed=0))
    t["model.layers.0.mlp.up_proj.weight"] = t["model.layers.0.mlp.up_proj.weight"].to(torch.int32)
    t["model.norm.weight"] = torch.ones(64, dtype=torch.int64)
    (tmp_path / "m").mkdir()
    with pytest.raises(WeightError, match="wrong element types") as ei:
        Model.load(write_folder(tmp_path / "m", cfg, t))
    assert len(ei.value.wrong_type) == 2 and any("up_proj" in w and "I32" in w for w in ei.value.wrong_type)
    assert any("model.norm.weight" in w and "I64" in w for w in ei.value.wrong_type)
    assert not ei.value.missing and not ei.value.unexpected and not ei.value.wrong_shape
    # half precision is a floating-point type: converted, not refused
    t = folder_tensors(str(tmp_path / "src"))
    t["model.norm.weight"] = t["model.norm.weight"].to(torch.float16)
    (tmp_path / "h").mkdir()
    info = Model.load(write_folder(tmp_path / "h", cfg, t)).tensor_info("bfloat16")
    assert info["model.norm.weight"] == {"stored": "F16", "device": "bfloat16", "shape": [64], "role": "norm"}


def test_tied_checkpoint_may_carry_a_separate_head_and_nothing_else(tmp_path):
    """Published tied checkpoints of this family store lm_head.weight too; it is not read.  Any other
    stray tensor is still an error."""
    cfg = config_from_dict(TINY_A)
    t = folder_tensors(write_model_folder(str(tmp_path / "src"), cfg, seed=0))
    t["lm_head.weight"] = torch.zeros(256, 64)
    (tmp_path / "m").mkdir()
    m = Model.load(write_folder(tmp_path / "m", cfg, t))
    assert "lm_head.weight" not in m.tensor_info() and m.plan_json()["ignored_tensors"] == ["lm_head.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    (tmp_path / "n").mkdir()
    with pytest.raises(WeightError, match="unexpected.*q_proj.bias") as ei:
        Model.load(write_folder(tmp_path / "n", cfg, t))
    assert ei.value.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    # an untied configuration needs its head
    cfg_b = config_from_dict(TINY_B)
    tb = folder_tensors(write_model_folder(str(tmp_path / "srcb"), cfg_b, seed=0))
    del tb["lm_head.weight"]
    (tmp_path / "b").mkdir()
    with pytest.raises(WeightError, match="missing.*lm_head"):
        Model.load(write_folder(tmp_path / "b", cfg_b, tb))


def test_sharded_folder(tmp_path):
    cfg = config_from_dict(TINY_A)
    t = folder_tensors(write_model_folder(str(tmp_path / "src"), cfg, seed=5))
    names = sorted(t)
    half = len(names) // 2
    cfg.save(str(tmp_path))
    save_safetensors(str(tmp_path / "m-1.safetensors"), {k: t[k] for k in names[:half]})
    save_safetensors(str(tmp_path / "m-2.safetensors"), {k: t[k] for k in names[half:]})
    wm = {k: ("m-1.safetensors" if i < half else "m-2.safetensors") for i, k in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    assert sorted(Model.load(str(tmp_path)).tensor_info()) == names
    os.remove(tmp_path / "m-2.safetensors")
    with pytest.raises(SafetensorsError, match="m-2.safetensors"):
        Model.load(str(tmp_path))


def test_no_weights_file(tmp_path):
    config_from_dict(TINY_A).save(str(tmp_path))
    with pytest.raises(SafetensorsError, match="model.safetensors"):
        Model.load(str(tmp_path))
    with pytest.raises(ConfigError, match="config.json"):
        Model.load(str(tmp_path / "nowhere"))
