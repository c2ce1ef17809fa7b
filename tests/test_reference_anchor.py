"""The plain implementation against outputs of kekzl/imp's own kernels.

tests/golden/reference_anchor.json holds what the reference's unmodified kernels gave on a B200 for
tiny inputs (made once by tests/golden/make_reference_anchor.py, which compiles them straight from
the reference's tree).  Every function of tests/plain/qwen3_plain.py that restates one of those
kernels is checked against it here, on the CPU, at the reference's own tolerances
(tests/test_layernorm.cu, tests/test_rope.cu: 1e-4 in float32; tests/test_attention.cu: 5e-2 in half;
the reference builds with --use_fast_math).  With IMP_REFERENCE_DIR set and a GPU, the file is made
again and must agree with the stored one.

Anchored on the reference's output this way: RMSNorm (eps inside the root, weight offset), the rotary
encoding (pairs i / i + D/2, angle pos * theta^(-2i/D), partial rotation), the per-head RMSNorm on q and
k BEFORE the rotation with one eps, the SwiGLU activation, the embedding gather, the greedy tie rule
(lowest index), causal grouped-query attention with its query-head to kv-head mapping and the window's
edge.  Anchored on reading only: the order of parts inside a layer, the tied output head.
"""
import json
import math
import os

import pytest
import torch

from plain import qwen3_plain as P

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ref():
    with open(os.path.join(HERE, "golden", "reference_anchor.json")) as f:
        return json.load(f)


def t(ref, name, *shape):
    return torch.tensor(ref[name], dtype=torch.float32).view(*shape)


def test_rmsnorm_matches_the_reference_kernel(ref):
    x, w = t(ref, "rmsnorm_x", 5, 48), t(ref, "rmsnorm_w", 48)
    assert torch.allclose(P.rmsnorm(x, w, 1e-5), t(ref, "rmsnorm_eps1e-5", 5, 48), rtol=1e-4, atol=1e-4)
    assert torch.allclose(P.rmsnorm(x, w, 0.5), t(ref, "rmsnorm_eps0.5", 5, 48), rtol=1e-4, atol=1e-4)
    # eps sits inside the root, beside the mean: outside it, or beside the sum, these numbers differ by far more
    wrong = x / (torch.sqrt((x * x).mean(-1, keepdim=True)) + 0.5) * w
    assert not torch.allclose(wrong, t(ref, "rmsnorm_eps0.5", 5, 48), rtol=1e-2, atol=1e-2)
    assert torch.allclose(P.rmsnorm(x, w + 1.0, 1e-6), t(ref, "rmsnorm_offset1", 5, 48), rtol=1e-4, atol=1e-4)


def test_rotary_encoding_matches_the_reference_kernel(ref):
    pos = ref["rope_positions"]
    q, k = t(ref, "rope_q", 6, 3, 16), t(ref, "rope_k", 6, 2, 16)
    # fast-math sin and cos lose accuracy with the angle (position 1000 here): 1e-4 at small angles, 2e-3 overall
    got_q, got_k = P.rope(q, pos, 10000.0), P.rope(k, pos, 10000.0)
    want_q, want_k = t(ref, "rope_q_out", 6, 3, 16), t(ref, "rope_k_out", 6, 2, 16)
    assert torch.allclose(got_q[:4], want_q[:4], atol=1e-4) and torch.allclose(got_k[:4], want_k[:4], atol=1e-4)
    assert torch.allclose(got_q, want_q, atol=2e-3) and torch.allclose(got_k, want_k, atol=2e-3)
    assert torch.equal(want_q[0], q[0]), "position 0 is the identity"
    # interleaved pairs (2i, 2i+1) would not give these numbers
    inter = q.clone().view(6, 3, 8, 2)
    assert not torch.allclose(P.rope(inter.transpose(-1, -2).reshape(6, 3, 16), pos, 10000.0), want_q, atol=1e-2)
    # Partial rotation (not used by this architecture; src/compute/rope.cu:84-101 with rope_dim = 8): the pairs are
    # (i, i + 4) within the first 8 components, but the reference keeps head_dim in the exponent of the angle,
    # theta^(-2i/16).  The engine's `rotary_dim` parameter follows the other convention, theta^(-2i/rotary_dim)
    # (tests/test_parts_gpu.py checks that one); what is pinned here is the reference's own formula.
    want8 = t(ref, "rope_q_out_dim8", 6, 3, 16)
    i = torch.arange(4, dtype=torch.float64)
    ang = torch.tensor(pos, dtype=torch.float64)[:, None] * (10000.0 ** (-2.0 * i / 16))[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    a, b = q[..., :4], q[..., 4:8]
    as_read = torch.cat([a * cos - b * sin, a * sin + b * cos, q[..., 8:]], -1)
    assert torch.allclose(as_read, want8, atol=2e-3)
    assert torch.equal(want8[..., 8:], q[..., 8:])


def test_qk_norm_comes_before_the_rotation_with_one_eps(ref):
    q, k = t(ref, "qknorm_q", 1, 4, 32), t(ref, "qknorm_k", 1, 2, 32)
    qw, kw = t(ref, "qknorm_qw", 32), t(ref, "qknorm_kw", 32)
    want_q, want_k = t(ref, "qknorm_q_out", 1, 4, 32), t(ref, "qknorm_k_out", 1, 2, 32)
    got_q = P.rope(P.rmsnorm(q, qw, 1e-3), [37], 1e6)
    got_k = P.rope(P.rmsnorm(k, kw, 1e-3), [37], 1e6)
    assert torch.allclose(got_q, want_q, atol=1e-2, rtol=1e-2) and torch.allclose(got_k, want_k, atol=1e-2, rtol=1e-2)   # half
    # the other order (rotate, then normalise with the weight) is a different function
    other = P.rmsnorm(P.rope(q, [37], 1e6), qw, 1e-3)
    assert not torch.allclose(other, want_q, atol=5e-2, rtol=5e-2)


def test_swiglu_embedding_and_greedy_match_the_reference_kernels(ref):
    g, u = t(ref, "swiglu_gate", 4, 24), t(ref, "swiglu_up", 4, 24)
    eye = torch.eye(24)
    # swiglu_mlp with identity matrices is the activation alone: g / (1 + exp(-g)) * u
    got = P.swiglu_mlp(torch.cat([g, u], -1), torch.eye(24, 48), torch.cat([torch.zeros(24, 24), eye], -1), eye)
    assert torch.allclose(got, t(ref, "swiglu_out", 4, 24), rtol=1e-4, atol=1e-4)
    table = t(ref, "embedding_table", 11, 8)
    assert torch.equal(P.embedding(table, ref["embedding_ids"]), t(ref, "embedding_out", 5, 8))
    logits = t(ref, "greedy_logits_503x2", 2, 503)
    for row, want in zip(logits, ref["greedy_picks"][:2]):
        assert int((row == row.max()).nonzero()[0]) == want        # the rule of greedy_generate
    assert ref["greedy_picks"] == [77, 502, 123], "ties go to the lowest index, in the two-stage kernel too"


def test_attention_matches_the_reference_kernel(ref):
    q, k, v = t(ref, "attention_q", 12, 4, 16), t(ref, "attention_k", 12, 2, 16), t(ref, "attention_v", 12, 2, 16)
    # the reference's launcher takes the scale as an argument (0.25 = 1/sqrt(16), what its caller passes:
    # src/graph/executor_forward.cu:566)
    assert 0.25 == 1 / math.sqrt(16)
    want = t(ref, "attention_out", 12, 4, 16)
    assert torch.allclose(P.attention(q, k, v), want, atol=5e-2), float((P.attention(q, k, v) - want).abs().max())
    assert float((P.attention(q, k, v) - want).abs().max()) < 5e-3      # in fact far inside the reference's own tolerance
    # query head h reads kv head h // 2: any other mapping is off by far more
    swapped = P.attention(q, k.flip(1), v.flip(1))
    assert float((swapped - want).abs().max()) > 0.1
    # a window of 5: position i sees i-4 .. i
    w5 = t(ref, "attention_out_window5", 12, 4, 16)
    assert float((P.attention(q, k, v, 5) - w5).abs().max()) < 5e-3
    assert float((P.attention(q, k, v, 4) - w5).abs().max()) > 1e-2 and float((P.attention(q, k, v, 6) - w5).abs().max()) > 1e-2


@pytest.mark.gpu
def test_the_stored_anchor_can_be_made_again(ref, tmp_path):
    """Only where the reference's tree is at hand (IMP_REFERENCE_DIR): compile its kernels, run them once more on
    the same tiny inputs, and compare with the stored file."""
    refdir = os.environ.get("IMP_REFERENCE_DIR")
    if not refdir or not os.path.isdir(os.path.join(refdir, "src", "compute")):
        pytest.skip("IMP_REFERENCE_DIR does not name the reference's source tree")
    import sys
    sys.path.insert(0, os.path.join(HERE, "golden"))
    from make_reference_anchor import build_and_run
    again = build_and_run(refdir, str(tmp_path))
    for key, want in ref.items():
        if isinstance(want, list):
            got = torch.tensor(again[key], dtype=torch.float64)
            assert torch.allclose(got, torch.tensor(want, dtype=torch.float64), atol=1e-6), key
