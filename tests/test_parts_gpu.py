"""Each part of the library alone against its plain counterpart, in float32 and bfloat16, at sizes that
differ from the engine tests' configurations.  Parts are built and run through the library's bench
(imp_bench_*: a stream, a workspace, a cache manager and the step function's batch builder, no model)."""
import pytest
import torch

from imp_b200.capi import ImpError
from imp_b200.cache.manager import PagedKVSpec
from imp_b200.parts.bench import PartBench
from imp_b200.parts.plan import PartSpec
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def close(got, want, dtype):
    got, want = got.float().cpu(), want.float().cpu()
    scale = max(float(want.abs().max()), 1e-3)
    atol, rtol = (2e-5 * scale, 2e-5) if dtype == torch.float32 else (0.02 * scale, 0.02)
    err = (got - want).abs()
    assert (err <= atol + rtol * want.abs()).all(), f"max error {err.max().item():.3g} (scale {scale:.3g})"


def place(t, dtype):
    return t.to(dtype).to(DEV)


def entries(lengths, prefix="s"):
    return [(f"{prefix}{i}", [1] * n, []) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    d, T = 72, 9
    bench = PartBench(NAME[dtype])
    w = 1 + 0.1 * rnd(d, seed=1)
    part = bench.build("norm", PartSpec("rmsnorm", {"size": d, "eps": 3e-5}), {"weight": place(w, dtype)})
    ctx = bench.prepare(entries([T]))
    h, br = rnd(T, d, seed=2, scale=2.0), rnd(T, d, seed=3).to(dtype)
    hd = h.clone().to(DEV)
    torch.cuda.synchronize()
    out = part.add_norm(hd, br.to(DEV), ctx=ctx)
    bench.sync()
    hs = h + br.float()
    assert torch.equal(hd.cpu(), hs)
    close(out, P.rmsnorm(hs, w.to(dtype).float(), 3e-5), dtype)
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    picked = part.add_norm(hd, None, rows, ctx=ctx)
    bench.sync()
    close(picked, P.rmsnorm(hs, w.to(dtype).float(), 3e-5)[[8, 2]], dtype)
    assert torch.equal(hd.cpu(), hs), "with rows the stream is left as it is"
    # a weight offset (norms that store w - 1)
    off = bench.build("norm", PartSpec("rmsnorm", {"size": d, "eps": 3e-5, "weight_offset": 1.0}), {"weight": place(w - 1, dtype)})
    got = off.add_norm(hd, None, ctx=ctx)
    bench.sync()
    close(got, P.rmsnorm(hs, (w - 1).to(dtype).float() + 1.0, 3e-5), dtype)


def test_rotary_part_is_shared_between_equal_specs_and_checks_its_sizes():
    bench = PartBench("float32")
    spec = PartSpec("rotary", {"head_dim": 48, "theta": 5e4, "max_positions": 100, "rotary_dim": 32})
    a, b = bench.build("position", spec), bench.build("position", spec)
    assert a.ptr == b.ptr                                          # equal specs share one table
    other = bench.build("position", PartSpec("rotary", {"head_dim": 48, "theta": 1e4, "max_positions": 100, "rotary_dim": 32}))
    assert other.ptr != a.ptr
    with pytest.raises(ImpError, match="rotary_dim"):
        bench.build("position", PartSpec("rotary", {"head_dim": 48, "theta": 1e4, "max_positions": 8, "rotary_dim": 50}))
    with pytest.raises(ImpError, match="unknown position kind"):
        bench.build("position", PartSpec("alibi", {}))


def attention_setup(dtype, window, qk_norm=True, Hq=6, Hkv=2, Dh=32, d=80, page_size=4, positions=1, rotary_dim=None):
    bench = PartBench(NAME[dtype], [PagedKVSpec(Hkv, Dh, window)] * positions, page_size=page_size)
    rot = {"head_dim": Dh, "theta": 1e4, "max_positions": 256}
    if rotary_dim:
        rot["rotary_dim"] = rotary_dim
    params = {"hidden_size": d, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": Dh, "window": window,
              "qk_norm": qk_norm, "qk_norm_eps": 1e-5, "position": {"kind": "rotary", "params": rot}}
    w = {"q_proj": rnd(Hq * Dh, d, seed=10, scale=0.2), "k_proj": rnd(Hkv * Dh, d, seed=11, scale=0.2),
         "v_proj": rnd(Hkv * Dh, d, seed=12, scale=0.2), "o_proj": rnd(d, Hq * Dh, seed=13, scale=0.2)}
    if qk_norm:
        w.update({"q_norm": 1 + 0.1 * rnd(Dh, seed=14), "k_norm": 1 + 0.1 * rnd(Dh, seed=15)})
    w = {k: v.to(dtype) for k, v in w.items()}
    part = bench.build("mixer", PartSpec("gqa_attention", params), {k: v.to(DEV) for k, v in w.items()})
    return bench, part, params, {k: v.float() for k, v in w.items()}


def plain_attention_part(x, w, Hq, Hkv, Dh, window, qk_norm=True, eps=1e-5, rotary_dim=None):
    T = x.shape[0]
    q = (x @ w["q_proj"].T).view(T, Hq, Dh)
    k = (x @ w["k_proj"].T).view(T, Hkv, Dh)
    v = (x @ w["v_proj"].T).view(T, Hkv, Dh)
    if qk_norm:
        q, k = P.rmsnorm(q, w["q_norm"], eps), P.rmsnorm(k, w["k_norm"], eps)
    pos = list(range(T))
    if rotary_dim:
        q = torch.cat([P.rope(q[..., :rotary_dim], pos, 1e4), q[..., rotary_dim:]], -1)
        k = torch.cat([P.rope(k[..., :rotary_dim], pos, 1e4), k[..., rotary_dim:]], -1)
    else:
        q, k = P.rope(q, pos, 1e4), P.rope(k, pos, 1e4)
    return P.attention(q, k, v, window).reshape(T, Hq * Dh) @ w["o_proj"].T


def run_mixer(bench, part, x, ctx, cache):
    torch.cuda.synchronize()
    out = part.forward(x.to(DEV), ctx, cache)
    bench.sync()
    return out.clone()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 7])
def test_attention_part_whole_then_in_portions(dtype, window):
    bench, part, params, w = attention_setup(dtype, window)
    Hq, Hkv, Dh, d = 6, 2, 32, 80
    lengths = [37, 5]
    xs = [rnd(n, d, seed=20 + i).to(dtype) for i, n in enumerate(lengths)]
    want = [plain_attention_part(x.float(), w, Hq, Hkv, Dh, window) for x in xs]
    # whole, both sequences in one batch
    ctx = bench.prepare(entries(lengths, "w"))
    out = run_mixer(bench, part, torch.cat(xs), ctx, bench.cache_view(0))
    bench.commit()
    close(out[:37], want[0], dtype)
    close(out[37:], want[1], dtype)
    # portions of 10, 2, 20, 1, 4 for the first sequence; the second rides along one token at a time
    done, outs, other = 0, [], 0
    for n in (10, 2, 20, 1, 4):
        es = [("p0", [1] * n, [])]
        parts = [xs[0][done:done + n]]
        if other < lengths[1]:
            es.append(("p1", [1], []))
            parts.append(xs[1][other:other + 1])
        ctx = bench.prepare(es)
        o = run_mixer(bench, part, torch.cat(parts), ctx, bench.cache_view(0))
        bench.commit()
        outs.append(o[:n])
        if other < lengths[1]:
            close(o[n:], want[1][other:other + 1], dtype)
            other += 1
        done += n
    close(torch.cat(outs), want[0], dtype)
    info = bench.cache_info()
    if window:
        assert any(p < 0 for p in info["paged"][0]["tables"]["2"]), "pages behind the window were given back"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_without_qk_norm_and_with_another_layers_cache(dtype):
    bench, part, params, w = attention_setup(dtype, 0, qk_norm=False, page_size=16)
    Hq, Hkv, Dh, d = 6, 2, 32, 80
    x = rnd(21, d, seed=30).to(dtype)
    ctx = bench.prepare(entries([21]))
    out = run_mixer(bench, part, x, ctx, bench.cache_view(0))
    close(out, plain_attention_part(x.float(), w, Hq, Hkv, Dh, 0, qk_norm=False), dtype)
    # a reader of that cache: its own queries over the keys and values the owner wrote
    w2 = {"q_proj": rnd(Hq * Dh, d, seed=70, scale=0.2), "k_proj": rnd(Hkv * Dh, d, seed=71, scale=0.2),
          "v_proj": rnd(Hkv * Dh, d, seed=72, scale=0.2), "o_proj": rnd(d, Hq * Dh, seed=73, scale=0.2)}
    w2 = {k: v.to(dtype) for k, v in w2.items()}
    reader = bench.build("mixer", PartSpec("gqa_attention", params), {k: v.to(DEV) for k, v in w2.items()})
    w2 = {k: v.float() for k, v in w2.items()}
    x2 = rnd(21, d, seed=31).to(dtype)
    out2 = run_mixer(bench, reader, x2, ctx, bench.cache_view(0, writes=False))
    T = 21
    q = P.rope((x2.float() @ w2["q_proj"].T).view(T, Hq, Dh), list(range(T)), 1e4)
    k = P.rope((x.float() @ w["k_proj"].T).view(T, Hkv, Dh), list(range(T)), 1e4)
    v = (x.float() @ w["v_proj"].T).view(T, Hkv, Dh)
    close(out2, P.attention(q, k, v).reshape(T, Hq * Dh) @ w2["o_proj"].T, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_with_partial_rotation(dtype):
    """rotary_dim < head_dim: the first rotary_dim components of every head are rotated, the rest pass."""
    bench, part, params, w = attention_setup(dtype, 0, Hq=4, Hkv=2, Dh=48, d=64, rotary_dim=32, page_size=8)
    x = rnd(19, 64, seed=33).to(dtype)
    ctx = bench.prepare(entries([19]))
    out = run_mixer(bench, part, x, ctx, bench.cache_view(0))
    close(out, plain_attention_part(x.float(), w, 4, 2, 48, 0, rotary_dim=32), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,F,T", [(80, 136, 5), (96, 100, 3), (64, 200, 40)])
def test_swiglu_part(dtype, d, F, T):
    bench = PartBench(NAME[dtype])
    w = {"gate_proj": rnd(F, d, seed=40, scale=0.2), "up_proj": rnd(F, d, seed=41, scale=0.2),
         "down_proj": rnd(d, F, seed=42, scale=0.2)}
    w = {k: v.to(dtype) for k, v in w.items()}
    part = bench.build("feed_forward", PartSpec("swiglu", {"hidden_size": d, "intermediate_size": F}),
                       {k: v.to(DEV) for k, v in w.items()})
    x = rnd(T, d, seed=43).to(dtype)
    ctx = bench.prepare(entries([T]))
    out = run_mixer(bench, part, x, ctx, None)
    close(out, P.swiglu_mlp(x.float(), w["gate_proj"].float(), w["up_proj"].float(), w["down_proj"].float()), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    V, d = 131, 72
    bench = PartBench(NAME[dtype])
    table = rnd(V, d, seed=50).to(dtype)
    emb = bench.build("embedding", PartSpec("token_embedding", {"vocab_size": V, "hidden_size": d}), {"weight": table.to(DEV)})
    ctx = bench.prepare([("e", [0, 130, 7, 7], [])])
    h = emb.embed(ctx)
    bench.sync()
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), table.float()[[0, 130, 7, 7]])
    scaled = bench.build("embedding", PartSpec("token_embedding", {"vocab_size": V, "hidden_size": d, "scale": 3.0}),
                         {"weight": table.to(DEV)})
    h3 = scaled.embed(ctx)
    bench.sync()
    assert torch.equal(h3.cpu(), table.float()[[0, 130, 7, 7]] * 3.0)
    head = bench.build("head", PartSpec("linear_head", {"vocab_size": V, "hidden_size": d}), {"weight": table.to(DEV)})   # tied
    for R in (3, 40):
        x = rnd(R, d, seed=51).to(dtype)
        torch.cuda.synchronize()
        lg = head.forward(x.to(DEV), ctx)
        bench.sync()
        assert lg.dtype == torch.float32
        close(lg, x.float() @ table.float().T, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_hands_the_second_sum_on(dtype):
    """h += attn(norm1(h)); pending = ffn(norm2(h)): the block's result equals the plain layer once the
    pending branch is added."""
    bench, attn, params, wa = attention_setup(dtype, 0, page_size=8)
    d, F, T = 80, 96, 12
    wf = {"gate_proj": rnd(F, d, seed=60, scale=0.2), "up_proj": rnd(F, d, seed=61, scale=0.2),
          "down_proj": rnd(d, F, seed=62, scale=0.2)}
    wf = {k: v.to(dtype) for k, v in wf.items()}
    n1w, n2w = (1 + 0.1 * rnd(d, seed=63)).to(dtype), (1 + 0.1 * rnd(d, seed=64)).to(dtype)
    ffn = bench.build("feed_forward", PartSpec("swiglu", {"hidden_size": d, "intermediate_size": F}),
                      {k: v.to(DEV) for k, v in wf.items()})
    n1 = bench.build("norm", PartSpec("rmsnorm", {"size": d, "eps": 1e-6}), {"weight": n1w.to(DEV)})
    n2 = bench.build("norm", PartSpec("rmsnorm", {"size": d, "eps": 1e-6}), {"weight": n2w.to(DEV)})
    block = bench.build_block("prenorm", {"mixer": attn, "feed_forward": ffn, "mixer_norm": n1, "ffn_norm": n2})
    with pytest.raises(ImpError, match="slot 'ffn_norm'"):
        bench.build_block("prenorm", {"mixer": attn, "feed_forward": ffn, "mixer_norm": n1})
    with pytest.raises(ImpError, match="norm"):
        bench.build_block("prenorm", {"mixer": attn, "feed_forward": ffn, "mixer_norm": n1, "ffn_norm": ffn})
    ctx = bench.prepare(entries([T]))
    h0 = rnd(T, d, seed=65)
    pend0 = rnd(T, d, seed=66).to(dtype)
    h = h0.clone().to(DEV)
    p0 = pend0.to(DEV)
    torch.cuda.synchronize()
    pending = block.block_forward(h, p0, ctx, bench.cache_view(0))
    bench.sync()
    hp = h0 + pend0.float()
    hp = hp + plain_attention_part(P.rmsnorm(hp, n1w.float(), 1e-6), wa, 6, 2, 32, 0)
    f = P.swiglu_mlp(P.rmsnorm(hp, n2w.float(), 1e-6), wf["gate_proj"].float(), wf["up_proj"].float(),
                     wf["down_proj"].float())
    close(h, hp, dtype)
    close(pending, f, dtype)
