"""The plain implementation itself: properties each part must have, and pinned outputs."""
import json
import math
import os

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P
from plain import sampling_plain as S

HERE = os.path.dirname(os.path.abspath(__file__))


def test_pinned_outputs(model_folders):
    gold = json.load(open(os.path.join(HERE, "golden", "plain_tiny.json")))
    for name, g in gold.items():
        m = P.PlainModel(model_folders[name][0])
        lg = m.logits(g["ids"])
        got = torch.tensor([[float(lg[r, c]) for c in g["cols"]] for r in g["rows"]])
        assert torch.allclose(got, torch.tensor(g["logits"]), rtol=1e-4, atol=1e-5), name
        assert m.generate(g["ids"][:5], 6) == g["greedy"], name


def test_logits_are_causal(model_folders):
    m = P.PlainModel(model_folders["B"][0])
    ids = list(range(3, 33))
    a = m.logits(ids)
    b = m.logits(ids[:20] + [7] * 10)
    assert torch.allclose(a[:20], b[:20], atol=1e-6)
    assert not torch.allclose(a[20:], b[20:], atol=1e-3)


def test_float64_agrees_with_float32(model_folders):
    f = model_folders["C"][0]
    ids = list(range(1, 40))
    a, b = P.PlainModel(f).logits(ids), P.PlainModel(f, torch.float64).logits(ids)
    assert (a.double() - b).abs().max() < 1e-4


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0]])
    y = P.rmsnorm(x, torch.tensor([1.0, 2.0]), 0.0)
    assert torch.allclose(y, torch.tensor([[3.0, 8.0]]) / math.sqrt(12.5))
    assert P.rmsnorm(x, torch.ones(2), 1.0)[0, 0] < y[0, 0]     # eps matters


def test_rope_properties():
    x = torch.randn(5, 3, 8)
    assert torch.allclose(P.rope(x, [0] * 5, 1e4), x)            # position 0 is the identity
    r = P.rope(x, [0, 1, 2, 3, 4], 1e4)
    assert torch.allclose(r.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # pair (0, 4) turns by exactly pos radians (frequency 1), pair (3, 7) by pos * theta^(-3/4)
    v = torch.zeros(1, 1, 8)
    v[0, 0, 0] = 1.0
    out = P.rope(v, [2], 1e4)[0, 0]
    assert abs(out[0] - math.cos(2)) < 1e-6 and abs(out[4] - math.sin(2)) < 1e-6
    v = torch.zeros(1, 1, 8)
    v[0, 0, 3] = 1.0
    out = P.rope(v, [5], 1e4)[0, 0]
    a = 5 * 1e4 ** (-6 / 8)
    assert abs(out[3] - math.cos(a)) < 1e-6 and abs(out[7] - math.sin(a)) < 1e-6
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    s1 = (P.rope(q, [9], 1e4) * P.rope(k, [4], 1e4)).sum()
    s2 = (P.rope(q, [105], 1e4) * P.rope(k, [100], 1e4)).sum()
    assert abs(s1 - s2) < 1e-4


def test_attention_mask_groups_and_window():
    torch.manual_seed(0)
    T, Hq, Hkv, D = 12, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    o = P.attention(q, k, v)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])   # first token sees itself only
    # heads 0,1 read kv head 0; heads 2,3 read kv head 1
    v2 = v.clone()
    v2[:, 1] += 1.0
    o2 = P.attention(q, k, v2)
    assert torch.allclose(o2[:, :2], o[:, :2]) and torch.allclose(o2[:, 2:], o[:, 2:] + 1.0, atol=1e-5)
    # a window of at least T changes nothing; window 1 returns the token's own value
    assert torch.allclose(P.attention(q, k, v, window=T), o)
    assert torch.allclose(P.attention(q, k, v, window=1)[:, 0], v[:, 0])
    # window 3: token 7 sees 5, 6, 7 only
    ow = P.attention(q, k, v, window=3)
    s = (q[7, 0] @ k[5:8, 0].T) / math.sqrt(D)
    assert torch.allclose(ow[7, 0], torch.softmax(s, -1) @ v[5:8, 0], atol=1e-6)


def test_swiglu_formula():
    x = torch.tensor([[1.0, -2.0]])
    wg, wu, wd = torch.eye(2), 2 * torch.eye(2), torch.eye(2)
    y = P.swiglu_mlp(x, wg, wu, wd)
    exp = torch.tensor([[1 / (1 + math.exp(-1)) * 2.0, -2 / (1 + math.exp(2)) * -4.0]])
    assert torch.allclose(y, exp)


def test_sampling_twin():
    x = np.array([1.0, 3.0, 3.0, -1.0, 2.0])
    assert S.sample(x, 0.0, 0.3) == 1                                  # ties: lowest index
    assert S.sample(x, 1.0, 0.3, top_k=1) == 1
    keep, _ = S.kept_set(x, 1.0, top_k=2)
    assert keep.tolist() == [False, True, True, False, False]
    keep, _ = S.kept_set(x, 1.0, top_k=3)
    assert keep.tolist() == [False, True, True, False, True]
    keep, e = S.kept_set(x, 1.0, top_p=0.5)                            # two tied leaders are both kept
    assert keep.tolist() == [False, True, True, False, False]
    keep, _ = S.kept_set(x, 1.0, min_p=0.2)                            # exp(-1)=0.37 stays, exp(-2)=0.13 goes
    assert keep.tolist() == [False, True, True, False, True]
    p = S.penalize(x, [1, 1, 3], repetition=2.0, frequency=0.5, presence=0.25)
    assert np.allclose(p, [1.0, 3.0 / 2 - 1.0 - 0.25, 3.0, -2.0 - 0.5 - 0.25, 2.0])
    assert np.allclose(S.penalize(x, [1, 1, 3], frequency=1.0, last_n=1), [1, 3, 3, -2, 2])
    # the draw follows index order and the empirical frequencies follow softmax
    rng = np.random.default_rng(0)
    counts = np.bincount([S.sample(x, 1.0, u) for u in rng.random(20000)], minlength=5) / 20000
    assert np.allclose(counts, np.exp(x) / np.exp(x).sum(), atol=0.012)
    lo, hi, _ = S.draw_interval(x, 1.0, 2)
    assert S.sample(x, 1.0, (lo + hi) / 2) == 2
