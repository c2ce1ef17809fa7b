"""Generation through the entry point against the plain implementation: greedy tokens, long
decoding, the first tokens of a sequence, sampling that does not depend on the batch, preemption
that changes nothing, and CUDA-graph decode equal to launching kernel by kernel."""
import numpy as np
import pytest
import torch

from plain import sampling_plain as S
from plain.qwen3_plain import PlainModel

pytestmark = pytest.mark.gpu


def engine(folder, dtype, page, **kw):
    from imp_b200 import Engine, EngineConfig
    cfg = dict(compute_dtype=dtype, kv_block_size=page, max_batch_size=4, max_seq_len=512, kv_cache_tokens=2048,
               max_batch_tokens=64)
    cfg.update(kw)
    return Engine.from_folder(folder, EngineConfig(**cfg))


def prompts_for(vocab, lengths, seed=5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_plain(name, model_folders):
    from imp_b200 import GenerateParams
    folder, cd, page = model_folders[name]
    plain = PlainModel(folder)
    prompts = prompts_for(cd["vocab_size"], [1, 7, 30, 12])
    want = [plain.generate(p, 10) for p in prompts]
    eng = engine(folder, "float32", page, prefill_chunk_size=8)
    got = eng.generate(prompts, GenerateParams(max_tokens=10, temperature=0.0))
    assert got == want
    assert eng.free_pages() == eng.num_pages and not eng.has_work()
    # bfloat16 may flip a near-tie later on; its first tokens, from well separated logits, must agree
    eng16 = engine(folder, "bfloat16", page)
    got16 = eng16.generate(prompts, GenerateParams(max_tokens=10, temperature=0.0))
    for p, g, w in zip(prompts, got16, want):
        lg = plain.logits(p)[-1]
        top2 = torch.topk(lg, 2).values
        if float(top2[0] - top2[1]) > 0.05 * float(lg.abs().max()):
            assert g[0] == w[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype, model_folders):
    """300 tokens decoded one by one after a one-token prompt; logits of positions 0, 1, 2 and of the
    last positions against the whole-sequence computation."""
    from imp_b200 import StepEntry
    folder, cd, page = model_folders["B"]
    plain = PlainModel(folder)
    ids = prompts_for(cd["vocab_size"], [301], seed=9)[0]
    ref = plain.logits(ids)
    eng = engine(folder, dtype, page)
    rows = {}
    for i, t in enumerate(ids):
        lg = torch.from_numpy(eng.step_tokens([StepEntry("x", [t], [0])]))
        if i < 3 or i >= 290 or i in (23, 24, 25, 47, 48):     # the window of B is 24, its pages hold 16
            rows[i] = lg[0]
    eng.end("x")
    scale = float(ref.abs().max())
    atol, rtol = (1e-4, 1e-4) if dtype == "float32" else (0.02 * scale, 0.02)
    for i, row in rows.items():
        err = (row - ref[i]).abs()
        assert (err <= atol + rtol * ref[i].abs()).all(), f"position {i}: max error {err.max():.3g}"


def test_temperature_sampling_is_reproducible_and_independent_of_the_batch(model_folders):
    from imp_b200 import GenerateParams
    folder, cd, page = model_folders["B"]
    prompts = prompts_for(cd["vocab_size"], [17, 33, 40, 1], seed=1)
    gp = [GenerateParams(max_tokens=12, temperature=0.8, top_k=0, top_p=1.0, seed=1 + i) for i in range(4)]
    eng = engine(folder, "float32", page, prefill_chunk_size=8, max_batch_tokens=24)
    together = eng.generate(prompts, gp)
    alone = [eng.generate([p], g)[0] for p, g in zip(prompts, gp)]
    assert together == alone
    assert engine(folder, "float32", page).generate(prompts, gp) == together
    other = eng.generate([prompts[1]], GenerateParams(max_tokens=12, temperature=0.8, top_k=0, top_p=1.0, seed=99))[0]
    assert other != together[1]
    # the plain twin draws the same tokens from the plain logits with the same uniform numbers
    from imp_b200.sampling.sampler import uniform_for
    plain = PlainModel(folder)
    ids = list(prompts[1])
    for step in range(12):
        tok = S.sample(plain.logits(ids)[-1].double().numpy(), 0.8, uniform_for(2, step))
        assert tok == together[1][step], f"step {step}"
        ids.append(tok)


def test_filters_and_penalties_through_the_entry_point(model_folders):
    from imp_b200 import GenerateParams
    folder, cd, page = model_folders["A"]
    plain = PlainModel(folder)
    eng = engine(folder, "float32", page)
    p = prompts_for(cd["vocab_size"], [9], seed=3)[0]
    # top_k = 1 is greedy whatever the temperature
    assert eng.generate([p], GenerateParams(max_tokens=6, temperature=1.5, top_k=1))[0] == plain.generate(p, 6)
    # a strong repetition penalty: greedy with penalised logits, as the plain twin computes them
    out = eng.generate([p], GenerateParams(max_tokens=8, temperature=0.0, repetition_penalty=1.8,
                                           frequency_penalty=0.3, presence_penalty=0.2))[0]
    ids = list(p)
    for tok in out:
        x = S.penalize(plain.logits(ids)[-1].double().numpy(), ids, 1.8, 0.3, 0.2)
        assert tok == int(np.flatnonzero(x == x.max())[0])
        ids.append(tok)
    # top-k keeps every draw inside the k most likely tokens
    out = eng.generate([p], GenerateParams(max_tokens=12, temperature=2.0, top_k=3, top_p=1.0, seed=4))[0]
    ids = list(p)
    for tok in out:
        assert tok in torch.topk(plain.logits(ids)[-1], 3).indices.tolist()
        ids.append(tok)


def test_preemption_for_lack_of_pages_changes_no_token(model_folders):
    from imp_b200 import GenerateParams
    folder, cd, page = model_folders["A"]          # pages of 4 tokens
    prompts = prompts_for(cd["vocab_size"], [14, 15, 13], seed=6)
    gp = GenerateParams(max_tokens=20, temperature=0.0)
    roomy = engine(folder, "float32", page).generate(prompts, gp)
    tight = engine(folder, "float32", page, kv_cache_max_blocks=18, kv_cache_tokens=0)   # 72 tokens for 3 x 34
    got = tight.generate(prompts, gp)
    assert got == roomy
    assert tight.info()["scheduler"]["preemptions"] >= 1
    assert tight.free_pages() == 18
    # a request that can never fit is refused, not queued for ever
    with pytest.raises(MemoryError):
        tight.generate([list(range(60))], GenerateParams(max_tokens=40, temperature=0.0))


def test_cuda_graph_decode_equals_eager_decode(model_folders):
    from imp_b200 import GenerateParams
    folder, cd, page = model_folders["C"]
    prompts = prompts_for(cd["vocab_size"], [5, 21, 9], seed=8)
    gp = GenerateParams(max_tokens=16, temperature=0.0)
    a = engine(folder, "bfloat16", page, enable_cuda_graphs=True)
    b = engine(folder, "bfloat16", page, enable_cuda_graphs=False)
    assert a.generate(prompts, gp) == b.generate(prompts, gp)
    ia, ib = a.info(), b.info()
    assert ia["graph_captures"] >= 1 and ia["graph_replays"] > 10 and ib["graph_replays"] == 0


def test_entry_point_refuses_bad_input(model_folders):
    from imp_b200 import GenerateParams, StepEntry
    folder, cd, page = model_folders["A"]
    eng = engine(folder, "float32", page)
    with pytest.raises(ValueError, match="vocabulary"):
        eng.submit([1, 2, cd["vocab_size"]])
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step_tokens([StepEntry("a", [-1], [0])])
    with pytest.raises(ValueError, match="wanted row"):
        eng.step_tokens([StepEntry("a", [1, 2], [2])])
    with pytest.raises(ValueError, match="twice"):
        eng.step_tokens([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(TypeError):
        eng.generate([1, 2, 3], GenerateParams(max_tokens=2))
    assert eng.free_pages() == eng.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lookahead_changes_nothing(dtype, model_folders):
    """With `lookahead` the engine queues the next decode step before it has read the last one's tokens.
    Tokens, finish reasons and the cache's bookkeeping must be what they are without it: greedy and
    sampled requests, different lengths, an end-of-sequence token in the middle, a late arrival."""
    from imp_b200 import GenerateParams
    from imp_b200.engine.scheduler import FinishReason
    folder, cd, page = model_folders["B"]
    V = cd["vocab_size"]
    prompts = prompts_for(V, [3, 20, 9, 14], seed=21)
    params = [GenerateParams(max_tokens=25, temperature=0.0), GenerateParams(max_tokens=40, temperature=0.9, seed=5),
              GenerateParams(max_tokens=7, temperature=0.0), GenerateParams(max_tokens=33, temperature=0.7, top_k=20, seed=8)]
    runs = {}
    for la in (False, True):
        eng = engine(folder, dtype, page, lookahead=la)
        # make the greedy continuation of the first prompt end early: its 6th token becomes the end-of-sequence id
        probe = engine(folder, dtype, page, lookahead=False).generate([prompts[0]], params[0])[0]
        eng.eos_token_ids = (probe[5],)
        reqs = [eng.submit(p, q) for p, q in zip(prompts[:3], params[:3])]
        n_calls = 0
        while any(not r.done for r in reqs):
            outs = eng.step()
            n_calls += 1
            if n_calls == 6:                      # a request arrives while the others decode
                reqs.append(eng.submit(prompts[3], params[3]))
            for o in outs:
                assert o.token >= 0 or o.finished
        eng.drain()
        assert not eng.has_work() and eng.free_pages() == eng.num_pages
        eng.check_invariants()
        runs[la] = [(list(r.output), r.finish_reason) for r in reqs]
    if dtype == "float32":
        assert runs[True] == runs[False]
    else:
        # bfloat16 results depend on the batch's size through rounding (another kernel, another order of
        # additions), and a request that ends on its end-of-sequence token rides along for one step more
        # with the step ahead: a sampled token may then differ.  What must agree is what was decided.
        assert [(len(o), why) for o, why in runs[True]] == [(len(o), why) for o, why in runs[False]]
        assert [o[:3] for o, _ in runs[True]] == [o[:3] for o, _ in runs[False]]
    first = runs[True][0]
    assert first[1] == FinishReason.EOS and len(first[0]) <= 6
    assert runs[True][2][1] == FinishReason.LENGTH and len(runs[True][2][0]) == 7


def test_lookahead_overlaps_only_when_it_may(model_folders):
    """The step ahead is launched for plain decoding only: not while a prompt is still being read in
    portions, not for requests whose sampling needs their tokens on the host, not into a token that ends
    a request by its length."""
    from imp_b200 import GenerateParams
    folder, cd, page = model_folders["A"]
    eng = engine(folder, "bfloat16", page, prefill_chunk_size=8)
    r = eng.submit(prompts_for(cd["vocab_size"], [20])[0], GenerateParams(max_tokens=4, temperature=0.0))
    eng.step()
    assert not eng.info()["inflight"]                  # first portion of the prompt: nothing sampled yet
    eng.step(); eng.step()
    assert len(r.output) == 1 and eng.info()["inflight"]      # decoding: one step is under way
    eng.step()
    assert len(r.output) == 2 and eng.info()["inflight"]
    eng.step()
    assert len(r.output) == 3 and eng.info()["inflight"]      # the step under way brings the fourth, last token
    eng.step()
    assert r.done and len(r.output) == 4 and not eng.info()["inflight"] and not eng.has_work()   # nothing was launched beyond it
    pen = eng.submit([1, 2, 3], GenerateParams(max_tokens=5, temperature=0.0, repetition_penalty=1.3))
    while not pen.done:
        eng.step()
        assert not eng.info()["inflight"]              # the penalty reads the tokens on the host


def test_a_second_end_token_in_config_json_ends_generation(model_folders, tmp_path):
    """`eos_token_id` may be a list; every id of it ends a request.  The model folder is copied with a list whose
    SECOND entry is a token that a seeded run samples a few steps in: generation stops there, and runs on with ignore_eos."""
    import json
    import shutil

    from imp_b200 import GenerateParams
    from imp_b200.engine.scheduler import FinishReason
    folder, cd, page = model_folders["A"]
    prompt = prompts_for(cd["vocab_size"], [11], seed=33)[0]
    sampled = dict(max_tokens=12, temperature=1.0, seed=3)            # the same seed gives the same tokens every time
    free_run = engine(folder, "float32", page).generate([prompt], GenerateParams(**sampled))[0]
    at = next(i for i in range(2, 12) if free_run[i] not in free_run[:i])   # a token that has not appeared before it
    stop = free_run[at]
    never = next(t for t in range(cd["vocab_size"]) if t not in free_run)
    copy = tmp_path / "with_eos"
    shutil.copytree(folder, copy)
    config = json.load(open(copy / "config.json"))
    config["eos_token_id"] = [never, stop]
    json.dump(config, open(copy / "config.json", "w"))
    eng = engine(str(copy), "float32", page)
    assert eng.eos_token_ids == (never, stop)
    r = eng.submit(prompt, GenerateParams(**sampled))
    while not r.done:
        eng.step()
    assert list(r.output) == free_run[:at + 1] and r.finish_reason == FinishReason.EOS
    assert eng.generate([prompt], GenerateParams(ignore_eos=True, **sampled))[0] == free_run
