"""Trace replay against the plain implementation, in float32 and bfloat16: every request whole;
most of it at once and the last 32 tokens one by one; portions of changing size; and up to four
live requests mixed in shared steps with so few pages that pages are used again."""
import numpy as np
import pytest
import torch

from plain.qwen3_plain import PlainModel
from replay_helpers import collect, mixed, portions, round64, run_trace, tail_decode, whole

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (5, 9, 1, 70, 33, 47), "B": (1, 17, 33, 40, 96, 64), "C": (3, 50, 81, 26, 2, 65),
           "D": (200, 70, 3, 333, 129, 64)}


def make_requests(name, vocab):
    g = torch.Generator().manual_seed({"A": 0, "B": 1, "C": 2, "D": 3}[name])
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}


def tolerances(dtype, ref_scale):
    # float32: rounding of a few hundred fused multiply-adds.  bfloat16: 8 bits of mantissa on every
    # activation between kernels, a few layers deep: two percent of the largest logit.
    if dtype == "float32":
        return 1e-4, 1e-4
    return 0.02 * ref_scale, 0.02


@pytest.fixture(scope="module")
def expected(model_folders):
    out = {}
    for name, (folder, cd, _) in model_folders.items():
        m = PlainModel(folder)
        reqs = make_requests(name, cd["vocab_size"])
        out[name] = (reqs, {rid: m.logits(ids).numpy() for rid, ids in reqs.items()})
    return out


def check_rows(rows, reqs, ref, dtype):
    scale = max(float(np.abs(r).max()) for r in ref.values())
    atol, rtol = tolerances(dtype, scale)
    n = 0
    for rid, ids in reqs.items():
        for p in range(len(ids)):
            got = rows[(rid, p)]
            want = ref[rid][p]
            bad = np.abs(got - want) > atol + rtol * np.abs(want)
            assert not bad.any(), (f"request {rid} position {p}: max error {np.abs(got - want).max():.3g} "
                                   f"(allowed {atol:.3g} + {rtol:.3g}|x|) in {dtype}")
            n += 1
    assert n == sum(len(v) for v in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_all_ways_of_cutting(name, dtype, model_folders, expected, tmp_path):
    folder, cd, page = model_folders[name]
    V = cd["vocab_size"]
    reqs, ref = expected[name]
    longest = round64(max(len(v) for v in reqs.values()))

    results = {}
    cuts = [("whole", whole(reqs), longest), ("tail", tail_decode(reqs), longest), ("portions", portions(reqs), longest)]
    if name == "D":
        # portions long enough for the 128-token attention tiles, starting inside pages and tiles
        cuts.append(("wide_portions", portions(reqs, sizes=(70, 130, 2, 64, 100, 67)), longest))
    for label, steps, pool in cuts:
        out = run_trace(folder, dtype, steps, pool, str(tmp_path / label), V, page_size=page)
        rows = collect(steps, out)
        check_rows(rows, reqs, ref, dtype)
        results[label] = rows

    steps, peak = mixed(reqs)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"] if len(s["entries"]) > 1)
    assert peak < sum(round64(len(v)) for v in reqs.values()), "the pool must be too small to avoid reuse"
    out = run_trace(folder, dtype, steps, peak, str(tmp_path / "mixed"), V, page_size=page)
    rows = collect(steps, out)
    check_rows(rows, reqs, ref, dtype)
    results["mixed"] = rows

    if dtype == "float32":
        # The float32 kernels reduce every row in an order that depends on that row alone, so the
        # logits of a position are the same bits however the work was cut and batched.
        for label in [c[0] for c in cuts[1:]] + ["mixed"]:
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[label][key]), f"{label}: {key} differs from the whole run"
