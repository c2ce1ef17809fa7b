"""Each part alone against its plain counterpart, in float32 and bfloat16, at sizes that differ
from the engine tests' configurations."""
import math

import pytest
import torch

from gpu_helpers import DEV, dummy_entries, layer_cache, part_stepper, runtime
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


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


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from imp_b200.parts.builtin import RMSNorm
    rt = runtime(dtype)
    d, T = 72, 9
    w = 1 + 0.1 * rnd(d, seed=1)
    part = RMSNorm({"size": d, "eps": 3e-5}, {"weight": place(w, dtype)}, rt)
    h, br = rnd(T, d, seed=2, scale=2.0), rnd(T, d, seed=3).to(dtype)
    hd = h.clone().to(DEV)
    out = part.add_norm(hd, br.to(DEV))
    hs = h + br.float()
    assert torch.equal(hd.cpu(), hs)
    close(out, P.rmsnorm(hs, w.to(dtype).float(), 3e-5), dtype)
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    close(part.add_norm(hd, None, rows), P.rmsnorm(hs, w.to(dtype).float(), 3e-5)[[8, 2]], dtype)
    x = place(rnd(5, d, seed=4), dtype)
    close(part.norm_rows(x), P.rmsnorm(x.float().cpu(), w.to(dtype).float(), 3e-5), dtype)


def test_rotary_part_tables_and_sharing():
    from imp_b200.parts.builtin import build_part
    from imp_b200.parts.plan import PartSpec
    rt = runtime(torch.float32)
    spec = PartSpec("rotary", {"head_dim": 48, "theta": 5e4, "max_positions": 100, "rotary_dim": 32})
    a, b = build_part("position", spec, {}, rt), build_part("position", spec, {}, rt)
    assert a is b                                          # equal specs share one table
    cos, sin, rot = a.rotary_tables()
    assert rot == 32 and cos.shape == (100, 16)
    i = torch.arange(16, dtype=torch.float64)
    ang = 37 * 5e4 ** (-2 * i / 32)
    assert torch.allclose(cos[37].cpu().double(), ang.cos(), atol=1e-7)
    assert torch.allclose(sin[37].cpu().double(), ang.sin(), atol=1e-7)
    with pytest.raises(ValueError):
        build_part("position", PartSpec("rotary", {"head_dim": 48, "theta": 1e4, "max_positions": 8, "rotary_dim": 50}), {}, rt)


def attention_setup(dtype, window, qk_norm=True, Hq=6, Hkv=2, Dh=32, d=80):
    from imp_b200.parts.builtin import GQAAttention
    from imp_b200.parts.plan import PartSpec
    rt = runtime(dtype)
    params = {"hidden_size": d, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": Dh, "window": window,
              "qk_norm": qk_norm, "qk_norm_eps": 1e-5,
              "position": PartSpec("rotary", {"head_dim": Dh, "theta": 1e4, "max_positions": 256})}
    w = {"q_proj": rnd(Hq * Dh, d, seed=10, scale=0.2), "k_proj": rnd(Hkv * Dh, d, seed=11, scale=0.2),
         "v_proj": rnd(Hkv * Dh, d, seed=12, scale=0.2), "o_proj": rnd(d, Hq * Dh, seed=13, scale=0.2),
         "q_norm": 1 + 0.1 * rnd(Dh, seed=14), "k_norm": 1 + 0.1 * rnd(Dh, seed=15)}
    w = {k: v.to(dtype) for k, v in w.items()}
    part = GQAAttention(params, {k: v.to(DEV) for k, v in w.items()}, rt)
    return rt, part, params, {k: v.float() for k, v in w.items()}


def plain_attention_part(x, w, Hq, Hkv, Dh, window, qk_norm=True, eps=1e-5):
    T = x.shape[0]
    q = (x @ w["q_proj"].T).view(T, Hq, Dh)
    k = (x @ w["k_proj"].T).view(T, Hkv, Dh)
    v = (x @ w["v_proj"].T).view(T, Hkv, Dh)
    if qk_norm:
        q, k = P.rmsnorm(q, w["q_norm"], eps), P.rmsnorm(k, w["k_norm"], eps)
    pos = list(range(T))
    q, k = P.rope(q, pos, 1e4), P.rope(k, pos, 1e4)
    return P.attention(q, k, v, window).reshape(T, Hq * Dh) @ w["o_proj"].T


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 7])
def test_attention_part_whole_then_in_portions(dtype, window):
    from imp_b200.engine.step import StepEntry
    rt, part, params, w = attention_setup(dtype, window)
    Hq, Hkv, Dh, d = 6, 2, 32, 80
    lengths = [37, 5]
    xs = [rnd(n, d, seed=20 + i).to(dtype) for i, n in enumerate(lengths)]
    want = [plain_attention_part(x.float(), w, Hq, Hkv, Dh, window) for x in xs]
    stepper, cache = part_stepper([part.cache_spec(params)], rt, page_size=4)
    # whole, both sequences in one batch
    ctx = stepper.prepare(dummy_entries(lengths, "w"))
    out = part.forward(torch.cat(xs).to(DEV), ctx, layer_cache(cache, ctx))
    stepper.commit(ctx)
    close(out[:37], want[0], dtype)
    close(out[37:], want[1], dtype)
    # portions of 10, 2, 20, 1, 4 for the first sequence; the second rides along one token at a time
    done, outs, other = 0, [], 0
    for n in (10, 2, 20, 1, 4):
        entries = [StepEntry("p0", [1] * n, [])]
        parts = [xs[0][done:done + n]]
        if other < lengths[1]:
            entries.append(StepEntry("p1", [1], []))
            parts.append(xs[1][other:other + 1])
        ctx = stepper.prepare(entries)
        o = part.forward(torch.cat(parts).to(DEV), ctx, layer_cache(cache, ctx))
        stepper.commit(ctx)
        outs.append(o[:n])
        if other < lengths[1]:
            close(o[n:], want[1][other:other + 1], dtype)
            other += 1
        done += n
    close(torch.cat(outs), want[0], dtype)
    stepper.check_device_status()
    cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_without_qk_norm_and_with_another_layers_cache(dtype):
    rt, part, params, w = attention_setup(dtype, 0, qk_norm=False)
    Hq, Hkv, Dh, d = 6, 2, 32, 80
    x = rnd(21, d, seed=30).to(dtype)
    stepper, cache = part_stepper([part.cache_spec(params)], rt, page_size=16)
    ctx = stepper.prepare(dummy_entries([21]))
    out = part.forward(x.to(DEV), ctx, layer_cache(cache, ctx))
    close(out, plain_attention_part(x.float(), w, Hq, Hkv, Dh, 0, qk_norm=False), dtype)
    # a reader of that cache: its own queries over the keys and values the owner wrote
    rt2, reader, _, w2 = attention_setup(dtype, 0, qk_norm=False)
    x2 = rnd(21, d, seed=31).to(dtype)
    out2 = reader.forward(x2.to(DEV), ctx, layer_cache(cache, ctx, writes=False))
    T = 21
    q = P.rope((x2.float() @ w2["q_proj"].T).view(T, Hq, Dh), list(range(T)), 1e4)
    k = P.rope((x.float() @ w["k_proj"].T).view(T, Hkv, Dh), list(range(T)), 1e4)
    v = (x.float() @ w["v_proj"].T).view(T, Hkv, Dh)
    close(out2, P.attention(q, k, v).reshape(T, Hq * Dh) @ w2["o_proj"].T, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,F,T", [(80, 136, 5), (96, 100, 3), (64, 200, 40)])
def test_swiglu_part(dtype, d, F, T):
    from imp_b200.parts.builtin import SwiGLU
    rt = runtime(dtype)
    w = {"gate_proj": rnd(F, d, seed=40, scale=0.2), "up_proj": rnd(F, d, seed=41, scale=0.2),
         "down_proj": rnd(d, F, seed=42, scale=0.2)}
    w = {k: v.to(dtype) for k, v in w.items()}
    part = SwiGLU({"hidden_size": d, "intermediate_size": F}, {k: v.to(DEV) for k, v in w.items()}, rt)
    assert part.interleaved == (F % 8 == 0)
    x = rnd(T, d, seed=43).to(dtype)
    out = part.forward(x.to(DEV), None)
    close(out, P.swiglu_mlp(x.float(), w["gate_proj"].float(), w["up_proj"].float(), w["down_proj"].float()), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from imp_b200.parts.builtin import LinearHead, TokenEmbedding
    rt = runtime(dtype)
    V, d = 131, 72
    table = rnd(V, d, seed=50).to(dtype)
    emb = TokenEmbedding({"vocab_size": V, "hidden_size": d}, {"weight": table.to(DEV)}, rt)
    ids = torch.tensor([0, 130, 7, 7], dtype=torch.int32, device=DEV)
    h = emb.forward(ids, None)
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), table.float()[[0, 130, 7, 7]])
    head = LinearHead({"vocab_size": V, "hidden_size": d}, {"weight": table.to(DEV)}, rt)   # tied
    for R in (3, 40):
        x = rnd(R, d, seed=51).to(dtype)
        lg = head.forward(x.to(DEV))
        assert lg.dtype == torch.float32
        want = x.float() @ table.float().T
        if dtype == torch.float32:
            close(lg, want, dtype)
        else:
            close(lg, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_hands_the_second_sum_on(dtype):
    """h += attn(norm1(h)); pending = ffn(norm2(h)): the block's result equals the plain layer once the
    pending branch is added."""
    from imp_b200.parts.builtin import PreNormBlock, RMSNorm, SwiGLU
    rt, attn, params, wa = attention_setup(dtype, 0)
    d, F, T = 80, 96, 12
    wf = {"gate_proj": rnd(F, d, seed=60, scale=0.2), "up_proj": rnd(F, d, seed=61, scale=0.2),
          "down_proj": rnd(d, F, seed=62, scale=0.2)}
    wf = {k: v.to(dtype) for k, v in wf.items()}
    n1w, n2w = (1 + 0.1 * rnd(d, seed=63)).to(dtype), (1 + 0.1 * rnd(d, seed=64)).to(dtype)
    ffn = SwiGLU({"hidden_size": d, "intermediate_size": F}, {k: v.to(DEV) for k, v in wf.items()}, rt)
    n1 = RMSNorm({"size": d, "eps": 1e-6}, {"weight": n1w.to(DEV)}, rt)
    n2 = RMSNorm({"size": d, "eps": 1e-6}, {"weight": n2w.to(DEV)}, rt)
    block = PreNormBlock(attn, ffn, n1, n2, rt)
    stepper, cache = part_stepper([attn.cache_spec(params)], rt, page_size=8)
    ctx = stepper.prepare(dummy_entries([T]))
    h0 = rnd(T, d, seed=65)
    pend0 = rnd(T, d, seed=66).to(dtype)
    h, pending = block.forward(h0.clone().to(DEV), pend0.to(DEV), ctx, layer_cache(cache, ctx))
    hp = h0 + pend0.float()
    hp = hp + plain_attention_part(P.rmsnorm(hp, n1w.float(), 1e-6), wa, 6, 2, 32, 0)
    f = P.swiglu_mlp(P.rmsnorm(hp, n2w.float(), 1e-6), wf["gate_proj"].float(), wf["up_proj"].float(),
                     wf["down_proj"].float())
    close(h, hp, dtype)
    close(pending, f, dtype)
