"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache.

It rests on the formulas of kekzl/imp's sources (cited per function by the
file's path within that project).  The reference's model code is CUDA-only and
cannot be built as a project here (it needs CUDA >= 13.1, CMakeLists.txt:15, and
fetches dependencies from the network, :44-68), so no whole-model output of the
reference exists; but its kernel files compile one by one, and
tests/golden/reference_anchor.json holds what they gave on a B200 for tiny
inputs.  tests/test_reference_anchor.py pins the per-part functions below
(rmsnorm, rope, the q/k norm before the rotation, the SwiGLU activation,
embedding, attention, the greedy tie rule) on those outputs; the order of the
parts inside a layer and the tied head rest on reading.

One function per part.  Nothing here is shared with the engine: this file
reads config.json and model.safetensors by itself and computes on the CPU in
float32 (or float64 with `dtype=torch.float64`).
"""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open


# ------------------------------------------------------------------ files
def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    cfg = {
        "layers": c["num_hidden_layers"],
        "hidden": c["hidden_size"],
        "heads": heads,
        "kv_heads": c.get("num_key_value_heads", heads),
        "head_dim": c.get("head_dim") or c["hidden_size"] // heads,
        "inter": c["intermediate_size"],
        "vocab": c["vocab_size"],
        "theta": float(c.get("rope_theta", 10000.0)),
        "eps": float(c["rms_norm_eps"]),
        "tied": bool(c.get("tie_word_embeddings", False)),
        "windows": [0] * c["num_hidden_layers"],
    }
    lt = c.get("layer_types")
    if lt is not None:
        cfg["windows"] = [int(c["sliding_window"]) if t == "sliding_attention" else 0 for t in lt]
    elif c.get("use_sliding_window"):
        first = c.get("max_window_layers") or 0
        cfg["windows"] = [int(c["sliding_window"]) if i >= first else 0 for i in range(cfg["layers"])]
    return cfg


def read_weights(model_dir, dtype=torch.float32):
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(dtype)
    return out


# ------------------------------------------------------------------ parts
def embedding(table, ids):
    """h[t] = E[id[t]], no scale (src/graph/executor_forward.cu:2786-2797)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rmsnorm(x, w, eps):
    """x * rsqrt(mean(x^2) + eps) * w over the last axis (src/compute/layernorm.cu:50-82)."""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rope(x, positions, theta):
    """Rotate pairs (i, i + D/2) of x[T, H, D] by pos * theta^(-2i/D)
    (src/compute/rope.cu:84-101: freq = 1/theta^(2i/D); x_i' = x_i cos - x_{i+D/2} sin,
    x_{i+D/2}' = x_i sin + x_{i+D/2} cos; neox pairing)."""
    T, H, D = x.shape
    half = D // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = 1.0 / (theta ** (2.0 * i / D))
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * freq[None, :]
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention(q, k, v, window=0):
    """Causal grouped-query attention over one whole sequence.

    q[T, Hq, D], k/v[T, Hkv, D]; s_ij = q_i.k_j / sqrt(D); masked when j > i or
    i - j >= window (window > 0) (src/compute/attention.cu:158-167); softmax over j;
    o_i = sum_j p_ij v_j; query head h uses kv head h // (Hq/Hkv)
    (src/compute/attention_paged.cu:84-160); scale at src/graph/executor_forward.cu:566.
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    out = torch.empty_like(q)
    ii = torch.arange(T)[:, None]
    jj = torch.arange(T)[None, :]
    masked = jj > ii
    if window > 0:
        masked = masked | ((ii - jj) >= window)
    for h in range(Hq):
        s = (q[:, h, :] @ k[:, h // g, :].T) / math.sqrt(D)
        s = s.masked_fill(masked, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, h // g, :]
    return out


def swiglu_mlp(x, wg, wu, wd):
    """down( g/(1+exp(-g)) * u ), g = x Wg^T, u = x Wu^T
    (src/compute/activation.cu:67-87; src/graph/executor_forward.cu:933-951, 1124-1140)."""
    g = x @ wg.T
    u = x @ wu.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ wd.T


def attention_block(x, w, prefix, cfg, positions, window):
    """q/k/v projections without bias, per-head RMSNorm on q and k with the layer norms' eps,
    rotary encoding, attention, output projection (src/graph/executor_forward.cu:429-470,
    536-556, 565-604, 773-777)."""
    T = x.shape[0]
    Hq, Hkv, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).view(T, Hq, D)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).view(T, Hkv, D)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).view(T, Hkv, D)
    q = rmsnorm(q, w[prefix + "self_attn.q_norm.weight"], cfg["eps"])
    k = rmsnorm(k, w[prefix + "self_attn.k_norm.weight"], cfg["eps"])
    q = rope(q, positions, cfg["theta"])
    k = rope(k, positions, cfg["theta"])
    o = attention(q, k, v, window).reshape(T, Hq * D)
    return o @ w[prefix + "self_attn.o_proj.weight"].T


def forward(w, cfg, ids):
    """Logits [T, vocab] of one whole sequence (src/graph/executor_forward.cu:2701-3140):
    embedding; per layer h += attn(norm(h)), h += mlp(norm(h)); final norm; output head
    (the embedding table when tied)."""
    h = embedding(w["model.embed_tokens.weight"], ids)
    positions = list(range(len(ids)))
    for l in range(cfg["layers"]):
        p = f"model.layers.{l}."
        x = rmsnorm(h, w[p + "input_layernorm.weight"], cfg["eps"])
        h = h + attention_block(x, w, p, cfg, positions, cfg["windows"][l])
        x = rmsnorm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        h = h + swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
    x = rmsnorm(h, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(w, cfg, prompt, n_new):
    """Greedy decoding by re-running the whole sequence; ties go to the lowest index
    (src/compute/sampling.cu:29-45)."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(w, cfg, ids)[-1]
        tok = int((logits == logits.max()).nonzero()[0])  # the lowest index among equal maxima
        out.append(tok)
        ids.append(tok)
    return out


class PlainModel:
    """Convenience holder: a model folder read once."""

    def __init__(self, model_dir, dtype=torch.float32):
        self.cfg = read_config(model_dir)
        self.w = read_weights(model_dir, dtype)

    def logits(self, ids):
        return forward(self.w, self.cfg, ids)

    def generate(self, prompt, n_new):
        return greedy_generate(self.w, self.cfg, prompt, n_new)
