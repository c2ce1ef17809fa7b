"""The C API called as a C program would call it: raw ctypes on the exported symbols, no wrapper
classes.  Argument and error-code checks in the style of the reference's tests/test_e2e.cpp:18-90
(defaults, error strings, null arguments, missing files), then the calls a program makes to load a
model, create a context, generate, step token by token, and replay tokens for logits."""
import ctypes
import json
import os
import subprocess
import sys
from ctypes import POINTER, byref, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

import pytest

from conftest import TINY_A
from imp_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    return capi.load()


def message(lib):
    return lib.imp_error_message().decode()


def test_header_and_library_agree_on_the_entry_points(lib):
    """Every function the two public headers declare is exported, and nothing the bindings use is undeclared."""
    import re
    declared = set()
    for name in ("imp.h", "imp_parts.h"):
        text = open(os.path.join(ROOT, "include", "imp_b200", name)).read()
        declared |= set(re.findall(r"IMP_EXPORT[^;(]*?\b(imp_\w+)\s*\(", text))
    assert len(declared) > 60
    for fn in declared:
        assert hasattr(lib, fn), f"{fn} is declared in the headers but not exported"
    for fn in capi._SIGNATURES:
        assert fn in declared, f"{fn} is bound in capi.py but not declared in a public header"


def test_defaults_and_error_strings(lib):
    c = lib.imp_config_default()
    # src/api/imp_api.cpp:35-72: batch 32, context 4096, no chunking, graphs on
    assert (c.device_id, c.max_batch_size, c.max_seq_len, c.prefill_chunk_size, c.enable_cuda_graphs) == (0, 32, 4096, 0, 1)
    assert (c.kv_block_size, c.max_batch_tokens, c.compute_dtype, c.lookahead) == (16, 2048, capi.COMPUTE_BF16, 1)
    p = lib.imp_generate_params_default()
    # src/api/imp_api.cpp:76-102
    assert (round(p.temperature, 3), round(p.top_p, 3), p.top_k, p.max_tokens, p.seed) == (0.7, 0.9, 40, 256, -1)
    assert (p.min_p, p.typical_p, p.repetition_penalty, round(p.dry_base, 3), p.dry_allowed_length) == (0.0, 1.0, 1.0, 1.75, 2)
    assert (p.mirostat, p.mirostat_tau, round(p.mirostat_eta, 3), p.ignore_eos) == (0, 5.0, 0.1, 0)
    assert lib.imp_error_string(capi.IMP_SUCCESS) == b"success"
    texts = {lib.imp_error_string(code) for code in range(-8, 1)}
    assert len(texts) == 9 and b"unknown error" not in texts
    assert lib.imp_error_string(-99) == b"unknown error"
    assert lib.imp_version().decode().count(".") == 2


def test_null_arguments_are_errors_not_crashes(lib):
    h = c_void_p()
    assert lib.imp_model_load(None, byref(h)) == capi.IMP_ERROR_INVALID_ARG and "null" in message(lib)
    assert lib.imp_model_load(b"/nowhere", None) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_model_random(None, 0, 0.02, 0.01, byref(h)) == capi.IMP_ERROR_INVALID_ARG
    cfg = lib.imp_config_default()
    assert lib.imp_context_create(None, byref(cfg), byref(h)) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_context_reset(None) == capi.IMP_ERROR_INVALID_ARG
    n = c_int(0)
    assert lib.imp_step(None, None, 0, byref(n)) == capi.IMP_ERROR_INVALID_ARG
    rid = c_int64(0)
    assert lib.imp_submit(None, None, 0, None, byref(rid)) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_step_tokens(None, None, 0, None, 0) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_generate(None, None, 0, None, None, 0, None) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_prefill(None, None, 0, None) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_decode_step(None, None) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_register_part(None, None, None) == capi.IMP_ERROR_INVALID_ARG
    assert lib.imp_cache_create(None, 4, 4, 1, 0, byref(h)) == capi.IMP_ERROR_INVALID_ARG
    # freeing nothing is allowed, getters on nothing answer nothing
    lib.imp_model_free(None)
    lib.imp_context_free(None)
    assert lib.imp_model_vocab_size(None) == 0 and lib.imp_model_arch(None) == b"" and lib.imp_has_work(None) == 0


def test_model_errors_have_their_codes(lib, tmp_path):
    h = c_void_p()
    assert lib.imp_model_load(str(tmp_path / "nowhere").encode(), byref(h)) == capi.IMP_ERROR_FILE_NOT_FOUND
    assert "config.json" in message(lib) and not h.value
    (tmp_path / "config.json").write_text("{broken")
    assert lib.imp_model_load(str(tmp_path).encode(), byref(h)) == capi.IMP_ERROR_INVALID_MODEL and "JSON" in message(lib)
    bad = dict(TINY_A, head_dim=24)
    assert lib.imp_model_random(json.dumps(bad).encode(), 0, 0.02, 0.01, byref(h)) == capi.IMP_ERROR_INVALID_MODEL
    assert "multiple of 16" in message(lib)
    unknown = dict(TINY_A, architectures=["NoSuchModel"])
    assert lib.imp_model_random(json.dumps(unknown).encode(), 0, 0.02, 0.01, byref(h)) == capi.IMP_ERROR_INVALID_MODEL
    assert "Qwen3ForCausalLM" in message(lib)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert lib.imp_model_load(str(tmp_path).encode(), byref(h)) == capi.IMP_ERROR_FILE_NOT_FOUND       # no weights file
    assert "model.safetensors" in message(lib)
    assert lib.imp_model_random(json.dumps(TINY_A).encode(), 0, -1.0, 0.01, byref(h)) == capi.IMP_ERROR_INVALID_ARG
    # a good one: the getters answer from config.json
    assert lib.imp_model_random(json.dumps(TINY_A).encode(), 3, 0.05, 0.01, byref(h)) == capi.IMP_SUCCESS and message(lib) == ""
    assert lib.imp_model_arch(h) == b"Qwen3ForCausalLM"
    assert (lib.imp_model_n_layers(h), lib.imp_model_d_model(h), lib.imp_model_vocab_size(h), lib.imp_model_max_seq_len(h)) == \
        (2, 64, 256, 512)
    plan = json.loads(lib.imp_model_plan_json(h).decode())
    assert plan["layers"][0]["block"] == "prenorm" and set(plan["layers"][0]["parts"]) == {"mixer_norm", "mixer", "ffn_norm", "feed_forward"}
    # a context needs a sound configuration (checked before any device is touched)
    ctx = c_void_p()
    cfg = lib.imp_config_default()
    cfg.max_batch_tokens, cfg.max_batch_size = 8, 64
    assert lib.imp_context_create(h, byref(cfg), byref(ctx)) == capi.IMP_ERROR_INVALID_ARG and "max_batch_tokens" in message(lib)
    cfg = lib.imp_config_default()
    cfg.compute_dtype = 7
    assert lib.imp_context_create(h, byref(cfg), byref(ctx)) == capi.IMP_ERROR_INVALID_ARG and not ctx.value
    lib.imp_model_free(h)


@pytest.fixture
def context(lib, model_folders):
    folder, cd, page = model_folders["A"]
    model, ctx = c_void_p(), c_void_p()
    assert lib.imp_model_load(folder.encode(), byref(model)) == 0, message(lib)
    cfg = lib.imp_config_default()
    cfg.compute_dtype, cfg.kv_block_size, cfg.kv_cache_max_blocks = capi.COMPUTE_FP32, page, 32
    cfg.max_batch_size, cfg.max_seq_len, cfg.max_batch_tokens = 4, 64, 32
    assert lib.imp_context_create(model, byref(cfg), byref(ctx)) == 0, message(lib)
    yield ctx, folder
    lib.imp_context_free(ctx)
    lib.imp_model_free(model)


def ints(values):
    return (c_int32 * max(len(values), 1))(*values)


@pytest.mark.gpu
def test_generate_prefill_decode_and_replay_through_raw_calls(lib, context):
    from plain.qwen3_plain import PlainModel
    ctx, folder = context
    plain = PlainModel(folder)
    prompt = [5, 17, 3, 200, 9]
    want = plain.generate(prompt, 7)
    p = lib.imp_generate_params_default()
    p.temperature, p.max_tokens = 0.0, 7
    out, n = ints([0] * 16), c_int(0)
    assert lib.imp_generate(ctx, ints(prompt), len(prompt), byref(p), out, 16, byref(n)) == 0, message(lib)
    assert list(out[:n.value]) == want
    # the reference's token-level pair: prefill samples the first token, decode steps hand tokens out one by one
    assert lib.imp_prefill(ctx, ints(prompt), len(prompt), byref(p)) == 0, message(lib)
    tok, got = c_int32(-1), []
    while lib.imp_decode_step(ctx, byref(tok)) == 0:
        got.append(tok.value)
    assert got == want and "ended" in message(lib)
    assert lib.imp_context_reset(ctx) == 0
    assert lib.imp_decode_step(ctx, byref(tok)) == capi.IMP_ERROR_INVALID_ARG and "imp_prefill" in message(lib)
    # submit + step: two requests share the steps; outputs name their request
    a, b = c_int64(-1), c_int64(-1)
    assert lib.imp_submit(ctx, ints(prompt), len(prompt), byref(p), byref(a)) == 0
    assert lib.imp_submit(ctx, ints(prompt[:2]), 2, byref(p), byref(b)) == 0 and a.value != b.value
    outs, tokens = (capi.ImpStepOutput * 8)(), {a.value: [], b.value: []}
    while lib.imp_has_work(ctx):
        assert lib.imp_step(ctx, outs, 8, byref(n)) == 0, message(lib)
        for o in outs[:n.value]:
            tokens[o.id].append(o.token)
    assert tokens[a.value] == want and tokens[b.value] == plain.generate(prompt[:2], 7)
    info = capi.ImpRequestInfo()
    assert lib.imp_request_info(ctx, a, byref(info)) == 0
    assert (info.status, info.finish_reason, info.n_prompt, info.n_output) == (2, 2, 5, 7)     # finished by length
    assert lib.imp_request_release(ctx, a) == 0 and lib.imp_request_info(ctx, a, byref(info)) == capi.IMP_ERROR_INVALID_ARG
    # replaying tokens for logits: a portion, then two tokens beside a new request
    import numpy as np
    V = 256
    lg = np.zeros((3, V), dtype=np.float32)
    e = (capi.ImpStepEntry * 2)()
    e[0].id, e[0].tokens, e[0].n_tokens, e[0].want, e[0].n_want = 7, ints(prompt[:3]), 3, ints([2]), 1
    assert lib.imp_step_tokens(ctx, e, 1, lg.ctypes.data_as(c_void_p), lg.size) == 0, message(lib)
    first = lg[0].copy()
    e[0].tokens, e[0].n_tokens, e[0].want, e[0].n_want = ints(prompt[3:]), 2, ints([0, 1]), 2
    e[1].id, e[1].tokens, e[1].n_tokens, e[1].want, e[1].n_want = 8, ints(prompt[:3]), 3, ints([2]), 1
    assert lib.imp_step_tokens(ctx, e, 2, lg.ctypes.data_as(c_void_p), lg.size) == 0, message(lib)
    ref = plain.logits(prompt).numpy()
    assert np.abs(first - ref[2]).max() < 1e-4 and np.abs(lg[:2] - ref[3:5]).max() < 1e-4
    assert np.array_equal(lg[2], first), "the same tokens give the same bits, whatever else is in the batch"
    assert lib.imp_step_tokens(ctx, e, 2, lg.ctypes.data_as(c_void_p), 10) == capi.IMP_ERROR_INVALID_ARG and "too small" in message(lib)
    assert lib.imp_end(ctx, 7) == 0 and lib.imp_end(ctx, 8) == 0
    assert lib.imp_end(ctx, 7) == capi.IMP_ERROR_INVALID_ARG and "twice" in message(lib)


@pytest.mark.gpu
def test_request_errors_through_raw_calls(lib, context):
    ctx, _ = context
    p = lib.imp_generate_params_default()
    rid = c_int64(-1)
    assert lib.imp_submit(ctx, ints([1, 2, 256]), 3, byref(p), byref(rid)) == capi.IMP_ERROR_INVALID_ARG and "vocabulary" in message(lib)
    assert lib.imp_submit(ctx, ints([]), 0, byref(p), byref(rid)) == capi.IMP_ERROR_INVALID_ARG
    long_prompt = [1] * 64                                     # max_seq_len is 64: no room for a token
    assert lib.imp_submit(ctx, ints(long_prompt), 64, byref(p), byref(rid)) == capi.IMP_ERROR_INVALID_ARG
    assert "max_seq_len" in message(lib)
    p.max_tokens = 0
    assert lib.imp_submit(ctx, ints([1]), 1, byref(p), byref(rid)) == capi.IMP_ERROR_INVALID_ARG and "max_tokens" in message(lib)
    p = lib.imp_generate_params_default()
    p.top_k = -1
    assert lib.imp_submit(ctx, ints([1]), 1, byref(p), byref(rid)) == capi.IMP_ERROR_INVALID_ARG and "top_k" in message(lib)
    assert lib.imp_cancel(ctx, 12345) == capi.IMP_ERROR_INVALID_ARG
    assert not lib.imp_has_work(ctx)
    info = json.loads(lib.imp_context_info_json(ctx).decode())
    assert info["cache"]["free_pages"] == info["cache"]["num_pages"] == 32 and info["workspace_bytes"] > 0


@pytest.mark.gpu
def test_the_entry_point_generates_without_torch(model_folders):
    """The product path is the library behind ctypes: a fresh interpreter that loads a model, generates and
    replays never imports torch."""
    folder, cd, page = model_folders["B"]
    code = f"""
import sys
sys.path.insert(0, {ROOT!r})
from imp_b200 import Engine, EngineConfig, GenerateParams, StepEntry
eng = Engine.from_folder({folder!r}, EngineConfig(kv_block_size={page}, max_batch_size=2, max_seq_len=128, kv_cache_tokens=512,
                                                  max_batch_tokens=64))
out = eng.generate([[1, 2, 3], [4, 5]], GenerateParams(max_tokens=5, temperature=0.0))
lg = eng.step_tokens([StepEntry("a", [1, 2, 3], [2])])
assert len(out) == 2 and len(out[0]) == 5 and lg.shape == (1, {cd["vocab_size"]})
assert "torch" not in sys.modules, "torch was imported on the product path"
print("ok", out[0])
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.startswith("ok"), r.stderr[-2000:]
