#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen3-8B shape, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]

Prints ONE JSON line.  Everything goes through the engine's public entry point (imp_b200.Engine, a thin
layer over the C API): host token lists in, sampled token ids out, every step with its host-to-device
copy of the batch arrays from pinned memory and its device-to-host read of the tokens.

`value` is decoded tokens per second at the default batch (8) with every sequence's context ending at
the configured context length (4096): K decode steps after W warm-up steps, timed on the device with
CUDA events on the engine's stream.  `e2e` is the same workload, K further steps, timed by the wall clock
around the calls.  `prefill` is one 2,048-token prompt in one step (and in 512-token portions), from the
upload of the batch to the last row's logits on the host.  `protocol` holds the full decode run of the
benchmark configuration, 2,048 greedy steps from 2,048 cached tokens to 4,096, at batch 1, 8 and 64, with
the first and last 256 steps and the spread over 256-step windows; `points` repeats its overall figures.
`yardsticks` times cuBLASLt (torch.mm, what the reference's engine calls for its T>1 products,
src/compute/gemm.cu:303-445) at the four prefill shapes beside this library's kernel, and the whole
prefill with the products on the library arm.  Roofline fractions use MEASURED_PEAKS.json when the driver
wrote it, else the stated fallback.  Every decode step streams all weights (about 16 GB), far more than
the 126 MB L2, so no explicit L2 flush is needed between timed iterations ("inputs larger than L2").

Other runs, each printing its own JSON line:
    python bench.py --only decode [--batch B] [--context C] [--page P] [--layers N] [--no-graphs]
    python bench.py --only prefill [--tokens T] [--chunk C] [--layers N]
    python bench.py --only mixed [--batch B] [--chunk C] [--context X]     B sequences decoding beside a prompt's portions
    IMP_B200_NVCC_FLAGS=-DIMP_TIMELINE python bench.py --only timeline [--batch B] [--context C] [--workload 0.6b|14b]   (a table, not JSON)
    python bench.py --workload 0.6b [--dtype float32]     64 requests, prompts 16..1024, 256 greedy tokens, 512-token portions
    python bench.py --workload 14b                        8 prompts of 8,192 tokens in 2,048-token portions, 512 tokens at T=0.7
(`--context` may exceed the configured 4096: the cache and the position table grow with it.)
"""
import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-8B shape: the third configuration of the baseline record.
MODEL = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "torch_dtype": "bfloat16", "max_position_embeddings": 4096,
}
# The two other shapes of the baseline record, with their workloads (see run_workload).
MODEL_06B = dict(MODEL, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True, max_position_embeddings=8192)
MODEL_14B = dict(MODEL, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                 intermediate_size=17408, max_position_embeddings=16384)
CONTEXT = 4096
START = 2048
STAGGER = 128      # prompts of a batch finish their prefill a step apart: room for the early ones to run all 2,048 steps
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=FALLBACK_PEAKS["bf16_tflops"]), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.device, self.samples, self.proc = device, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(float(parts[0])))
                mx = max(mx, int(float(parts[1])))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, n_layers):
    d, hq, hkv, dh, f, v = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                            cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = (hq + 2 * hkv) * dh * d + d * hq * dh + 3 * f * d          # matrix elements
    norms = 2 * d + 2 * dh
    weight_bytes = 2 * (n_layers * (per_layer + norms) + v * d + d)         # every weight a decode step reads once
    kv_bytes_per_token = n_layers * 2 * hkv * dh * 2
    return per_layer, weight_bytes, kv_bytes_per_token


def prefill_flops(cfg, n_layers, T):
    per_layer, _, _ = model_numbers(cfg, n_layers)
    hq, dh = cfg["num_attention_heads"], cfg["head_dim"]
    linear = 2.0 * T * per_layer * n_layers + 2.0 * cfg["vocab_size"] * cfg["hidden_size"]
    attn = n_layers * hq * 4.0 * dh * (T * (T + 1) / 2.0)                    # QK^T and PV over the causal half
    return linear + attn


def spread(xs):
    return {"min": round(min(xs), 4), "median": round(statistics.median(xs), 4), "max": round(max(xs), 4)}


def random_prompt(rng, vocab, n):
    return [rng.randrange(vocab) for _ in range(n)]


def make_engine(cfgd, args, max_batch, max_ctx, budget=PREFILL_TOKENS, chunk=0, dtype="bfloat16", seed=0, pool_tokens=None):
    from imp_b200 import Engine, EngineConfig
    ecfg = EngineConfig(max_batch_size=max_batch, max_seq_len=max_ctx, kv_block_size=args.page or PAGE,
                        kv_cache_tokens=pool_tokens or (max_batch * max_ctx + 2 * budget), max_batch_tokens=budget,
                        prefill_chunk_size=chunk, compute_dtype=dtype, enable_cuda_graphs=not args.no_graphs)
    t0 = time.time()
    eng = Engine.from_random(cfgd, ecfg, seed=seed, std=0.02)
    return eng, time.time() - t0


def start_decoding(eng, rng, vocab, B, prompt_len, max_tokens):
    """Submit B prompts and step until every one has its first token (real prefill fills the cache)."""
    from imp_b200 import GenerateParams
    gp = GenerateParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    reqs = [eng.submit(random_prompt(rng, vocab, prompt_len), gp) for _ in range(B)]
    waiting = {r.rid for r in reqs}
    while waiting:
        for o in eng.step():
            waiting.discard(o.rid)
    return reqs


def stop(eng, reqs):
    for r in reqs:
        eng.cancel(r)
    eng.drain()
    for r in reqs:
        r.release()


def timed_steps(eng, n, B, wall=None):
    """n decode steps of B sequences between two CUDA events on the engine's stream: device milliseconds.  `wall`
    (a list) also gets the host's milliseconds around the same calls, tokens read on the host after every step."""
    t0 = time.perf_counter()
    eng.timer_start()
    for _ in range(n):
        outs = eng.step()
        assert len(outs) == B, f"{len(outs)} tokens from a step of {B} sequences: a request left the batch"
    ms = eng.timer_stop()
    if wall is not None:
        wall.append((time.perf_counter() - t0) * 1e3)
    return ms


def time_prefill(eng, rng, vocab, n_prompt, chunk, reps=7):
    """One prompt of n_prompt tokens, whole or in portions of `chunk`, to the last row's logits on the host."""
    from imp_b200 import StepEntry
    ms = []
    for i in range(1 + reps):      # one warm-up; the products run at the power cap and vary by a few per cent
        prompt = random_prompt(rng, vocab, n_prompt)
        step = chunk or n_prompt
        eng.timer_start()
        for a in range(0, n_prompt, step):
            part = prompt[a:a + step]
            eng.step_tokens([StepEntry("pf", part, [len(part) - 1] if a + step >= n_prompt else [])])
        t = eng.timer_stop()
        eng.end("pf")
        if i > 0:
            ms.append(t)
    return ms


def decode_protocol(eng, rng, cfgd, n_layers, B, peaks, window=256):
    """The benchmark configuration's decode run: B sequences with 2,048 cached tokens (real prefill) decode
    greedily to 4,096; device time per 256-step window."""
    _, weight_bytes, kv_per_tok = model_numbers(cfgd, n_layers)
    total = CONTEXT - START
    reqs = start_decoding(eng, rng, cfgd["vocab_size"], B, START, total + STAGGER)
    eng.step()                                       # the first decode step of a batch size runs eagerly, the second is captured
    eng.step()
    done, win_ms, wall_ms = 0, [], []       # the two steps above are not counted: the stagger leaves room for them
    while done + window <= total:
        win_ms.append(timed_steps(eng, window, B, wall_ms) / window)
        done += window
    stop(eng, reqs)

    def point(ms, ctx):
        gbs = (weight_bytes + B * ctx * kv_per_tok) / (ms * 1e-3) / 1e9
        return {"tok_s": round(B / ms * 1e3, 1), "ms": round(ms, 4), "context": int(ctx), "gbs": round(gbs, 1),
                "frac": round(gbs / peaks["hbm_gbs"], 4)}

    n = len(win_ms)
    all_ms = sum(win_ms) / n
    e2e_ms = sum(wall_ms) / (n * window)       # the same steps by the host's clock, through the entry point
    return {"batch": B, "steps": n * window, "first256": point(win_ms[0], START + 2 + window / 2),
            "last256": point(win_ms[-1], START + 2 + (n - 0.5) * window),
            "all": point(all_ms, START + 2 + n * window / 2), "ms_per_step_over_windows": spread(win_ms),
            "e2e": {"tok_s": round(B / e2e_ms * 1e3, 1), "ms": round(e2e_ms, 4), "over_device": round(e2e_ms / all_ms, 4)}}


def yardsticks(peaks, reps=20):
    """cuBLASLt (through torch.mm) at the four prefill products of the benchmark shape beside this library's own
    choice of kernel for the same product, each timed with CUDA events over `reps` launches on one stream."""
    import torch

    from imp_b200.ops import kernels as K
    d, f, T = MODEL["hidden_size"], MODEL["intermediate_size"], PREFILL_TOKENS
    qkv = (MODEL["num_attention_heads"] + 2 * MODEL["num_key_value_heads"]) * MODEL["head_dim"]
    shapes = {"qkv": (T, qkv, d), "o": (T, d, MODEL["num_attention_heads"] * MODEL["head_dim"]), "gate_up": (T, 2 * f, d),
              "down": (T, d, f)}
    out = {}
    g = torch.Generator(device="cuda").manual_seed(0)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    for name, (M, N, Kd) in shapes.items():
        a = torch.randn(M, Kd, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        w = (torch.randn(N, Kd, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        wt = w.t()
        lib_ms = timed(lambda: torch.mm(a, wt, out=c))
        own_ms = timed(lambda: K.linear(c, a, w))
        flops = 2.0 * M * N * Kd
        out[name] = {"shape": f"{M}x{N}x{Kd}", "cublaslt_ms": round(lib_ms, 4), "own_ms": round(own_ms, 4),
                     "cublaslt_tflops": round(flops / lib_ms / 1e9, 1), "own_tflops": round(flops / own_ms / 1e9, 1),
                     "own_over_cublaslt": round(lib_ms / own_ms, 3)}
    return out


def attention_yardsticks(reps=20):
    """The prefill attention of the benchmark shape (2,048 tokens, one sequence, paged cache) three ways: this
    library's tcgen05 kernel, its plain mma.sync kernel (the class of kernel the reference runs on this architecture:
    4-warp WMMA, src/compute/attention_dispatch.cu:27-57), and the library attention behind torch's
    scaled_dot_product_attention on the same dense q, k, v.  CUDA events over `reps` launches each."""
    import math

    import torch

    from imp_b200.ops import attention as A
    from imp_b200.ops import kernels as K
    T, Hq, Hkv, Dh, P = PREFILL_TOKENS, MODEL["num_attention_heads"], MODEL["num_key_value_heads"], MODEL["head_dim"], PAGE
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(T, Hq * Dh, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(T, Hkv, Dh, generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn(T, Hkv, Dh, generator=g, device=dev).to(torch.bfloat16)
    n_pages = T // P
    perm = torch.randperm(n_pages, generator=g, device=dev)
    kc = torch.zeros(n_pages, Hkv, P, Dh, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    pos = torch.arange(T, device=dev)
    kc[perm[pos // P], :, pos % P] = k
    vc[perm[pos // P], :, pos % P] = v
    bt = perm.to(torch.int32).view(1, n_pages).contiguous()
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    positions = pos.to(torch.int32)
    status = K.new_status(dev)
    scale = 1.0 / math.sqrt(Dh)

    def tiles(n):
        t0 = torch.arange(0, T, n, dtype=torch.int32, device=dev)
        return t0, torch.full_like(t0, n)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    out = torch.empty(T, Hq * Dh, dtype=torch.bfloat16, device=dev)
    t128, r128 = tiles(128)
    t32, r32 = tiles(32)
    res = {"shape": f"{T} tokens, {Hq}/{Hkv} heads x {Dh}, causal"}
    res["own_tcgen05_us"] = round(timed(lambda: A.prefill_attention_tc(out, q, Hq, Hkv, Dh, kc, vc, bt, seq, positions, t128, r128,
                                                                       scale, 0, status)), 1)
    res["own_mma_sync_us"] = round(timed(lambda: A.prefill_attention(out, q, Hq, Hkv, Dh, kc, vc, bt, seq, positions, t32, r32,
                                                                     scale, 0, status)), 1)
    K.check_status(status)
    try:
        qd = q.view(T, Hq, Dh).transpose(0, 1).unsqueeze(0).contiguous()
        kd = k.transpose(0, 1).unsqueeze(0).repeat_interleave(Hq // Hkv, dim=1).contiguous()
        vd = v.transpose(0, 1).unsqueeze(0).repeat_interleave(Hq // Hkv, dim=1).contiguous()
        sdpa = torch.nn.functional.scaled_dot_product_attention
        res["torch_sdpa_us"] = round(timed(lambda: sdpa(qd, kd, vd, is_causal=True, scale=scale)), 1)
    except Exception as e:
        res["torch_sdpa_us"] = None
        res["torch_sdpa_error"] = f"{type(e).__name__}: {e}"[:120]
    flops = 4.0 * Hq * Dh * T * (T + 1) / 2
    res["own_tcgen05_tflops"] = round(flops / res["own_tcgen05_us"] / 1e6, 1)
    return res


def library_arm_prefill(args):
    """The whole 2,048-token prefill with the products of more than 16 rows on cuBLASLt (IMP_B200_GEMM=cublas is
    read once per process, so this is a run of its own)."""
    env = dict(os.environ, IMP_B200_GEMM="cublas")
    cmd = [sys.executable, os.path.abspath(__file__), "--only", "prefill"] + (["--layers", str(args.layers)] if args.layers else [])
    try:
        p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        line = [l for l in p.stdout.splitlines() if l.startswith("{")][-1]
        d = json.loads(line)
        return {"ms": d["ms"], "launches": d.get("launches"), "fallback_calls": d.get("fallback_calls")}
    except Exception as e:   # the yardstick is extra: its absence must not take the line with it
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


TIMELINE_KERNELS = {2: "sum of K parts", 3: "decode attention", 4: "add+norm (cluster)", 5: "few-rows product (mma.sync)",
                    6: "add+norm (one CTA a row)", 7: "merge of key splits", 10: "few-rows product", 11: "few-rows product, K parts",
                    12: "few-rows gate/up + SwiGLU", 20: "many-rows product (pairs)", 21: "many-rows product (pairs), K parts",
                    22: "many-rows gate/up + SwiGLU (pairs)", 23: "many-rows q,k,v + norm + rotation (pairs)"}


def run_timeline(args):
    """One decode step as its kernels saw it: needs a build with IMP_B200_NVCC_FLAGS=-DIMP_TIMELINE, in which thread 0 of
    every CTA of the decode kernels records the global timer at its start, after its wait for the kernel before it, and
    at its end.  Prints, per kernel, the launches of one step with the mean time from the wait to the last CTA's end, the
    mean gap between the end of the launch before and the wait, how long before the wait the CTAs were resident (and
    fetching what does not depend on earlier kernels), and the spread of the CTAs' ends."""
    import ctypes
    import numpy as np
    import torch
    from imp_b200.ops import attention as A
    from imp_b200.ops import library as L
    if "-DIMP_TIMELINE" not in os.environ.get("IMP_B200_NVCC_FLAGS", ""):
        print("bench.py --only timeline needs IMP_B200_NVCC_FLAGS=-DIMP_TIMELINE (a diagnostic build of the library)")
        return 2
    cfgd = dict({"0.6b": MODEL_06B, "14b": MODEL_14B}.get(args.workload, MODEL))
    n_layers = args.layers or cfgd["num_hidden_layers"]
    cfgd["num_hidden_layers"] = n_layers
    B, ctx = args.batch, args.context or CONTEXT
    eng, _ = make_engine(cfgd, args, B, ctx)
    rng = random.Random(0)
    reqs = start_decoding(eng, rng, cfgd["vocab_size"], B, ctx - 4 * B - 16, 4 * B + 24)   # the early ones still run at the end
    for _ in range(8):
        eng.step()
    torch.cuda.synchronize()
    cap = 400000
    buf = torch.zeros(cap * 4, dtype=torch.int64, device="cuda")
    count = torch.zeros(1, dtype=torch.int32, device="cuda")
    for handle, name in ((L.load(), "imp_tl_set_gemm_tc"), (L.load(), "imp_tl_set_norm"), (L.load(), "imp_tl_set_gemm_stream"),
                         (A.variant(cfgd["head_dim"]), "imp_tl_set_attention_mma")):
        fn = getattr(handle, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p]
        assert fn(buf.data_ptr(), cap, count.data_ptr()) == 0, name
    eng.step()
    torch.cuda.synchronize()
    count.zero_()
    torch.cuda.synchronize()
    eng.step()
    torch.cuda.synchronize()
    n = min(int(count.item()), cap)
    rec = buf[: 4 * n].view(n, 4).cpu().numpy()
    stop(eng, reqs)
    kern = (rec[:, 0] >> 48) & 0xFFFF
    t0, t1, t2 = rec[:, 1], rec[:, 2], rec[:, 3]
    # a launch's CTAs all leave their wait after the launch before has ended: runs of one kernel in the order of the waits
    launches = []
    for i in np.argsort(t1, kind="stable"):
        if not launches or launches[-1][0] != int(kern[i]):
            launches.append((int(kern[i]), []))
        launches[-1][1].append(i)
    base = int(t0.min())
    rows, prev_end = [], None
    for k, idx in launches:
        idx = np.array(idx)
        wait, end = int(t1[idx].min()), int(t2[idx].max())
        rows.append({"kernel": TIMELINE_KERNELS.get(k, str(k)), "ctas": len(idx), "wait_us": (wait - base) / 1e3,
                     "busy_us": (end - wait) / 1e3, "gap_us": (wait - prev_end) / 1e3 if prev_end is not None else 0.0,
                     "early_us": (wait - int(t0[idx].min())) / 1e3, "end_spread_us": (end - int(t2[idx].min())) / 1e3})
        prev_end = end
    print(f"batch {B}, context {ctx}, {n_layers} layers: {n} CTAs in {len(rows)} launches of the marked kernels, "
          f"{(int(t2.max()) - base) / 1e3:.1f} us from the first start to the last end")
    mid = len(rows) // 2
    per_layer = max(1, len(rows) // n_layers)
    print("one layer from the middle of the step:")
    print(f"  {'kernel':<30} {'CTAs':>5} {'wait at':>9} {'wait->end':>9} {'gap before':>10} {'resident before wait':>20} {'spread of ends':>14}")
    for r in rows[mid:mid + per_layer]:
        print(f"  {r['kernel']:<30} {r['ctas']:5d} {r['wait_us']:9.2f} {r['busy_us']:9.2f} {r['gap_us']:10.2f} {r['early_us']:20.2f} {r['end_spread_us']:14.2f}")
    print("means over the step's launches (us):")
    names = []
    for r in rows:
        if r["kernel"] not in names:
            names.append(r["kernel"])
    for name in names:
        sel = [r for r in rows if r["kernel"] == name]
        mean = lambda key: sum(r[key] for r in sel) / len(sel)
        print(f"  {name:<30} x{len(sel):<4d} wait->end {mean('busy_us'):6.2f}  gap before {mean('gap_us'):6.2f}  "
              f"resident before wait {mean('early_us'):6.2f}  spread of ends {mean('end_spread_us'):5.2f}")
    return 0


def run_mixed(args):
    """Steps in which `--batch` sequences decode (contexts near `--context`) beside one portion of `--chunk` tokens of a
    long prompt: the decode-only step, the mixed step, and the portion the scheduler actually cut (it ends a step on a
    multiple of 256 rows).  One JSON line."""
    from imp_b200 import Engine, EngineConfig, GenerateParams
    B, C, ctx = args.batch, args.chunk or 512, args.context or 2048
    cfgd = dict(MODEL)
    cfgd["max_position_embeddings"] = 16384
    n_layers = args.layers or MODEL["num_hidden_layers"]
    cfgd["num_hidden_layers"] = n_layers
    ecfg = EngineConfig(max_batch_size=B + 1, max_seq_len=16384, kv_block_size=args.page or PAGE,
                        kv_cache_tokens=(B + 1) * (ctx + 600) + 16384, max_batch_tokens=B + C, prefill_chunk_size=C,
                        compute_dtype="bfloat16", enable_cuda_graphs=not args.no_graphs)
    eng = Engine.from_random(cfgd, ecfg, seed=0, std=0.02)
    rng = random.Random(0)
    V = cfgd["vocab_size"]
    reqs = start_decoding(eng, rng, V, B, ctx, 400)
    for _ in range(5):
        eng.step()
    eng.timer_start()
    for _ in range(10):
        eng.step()
    decode_ms = eng.timer_stop() / 10
    long_prompt = 14 * C
    eng.submit(random_prompt(rng, V, long_prompt), GenerateParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    eng.step()
    eng.step()
    n = 8
    before = eng.info()
    eng.timer_start()
    for _ in range(n):
        eng.step()
    mixed_ms = eng.timer_stop() / n
    info = eng.info()
    print(json.dumps({"only": "mixed", "layers": n_layers, "decoding": B, "context": ctx, "portion_asked": C,
                      "decode_only_ms": round(decode_ms, 3), "mixed_ms": round(mixed_ms, 3),
                      "launches_per_mixed_step": (info["launches"] - before["launches"]) / n,
                      "fallback_calls": info["fallback_calls"]}))
    return 0


def run_ours(args):
    peaks, peak_src = read_peaks()
    cfgd = dict(MODEL)
    n_layers = args.layers or MODEL["num_hidden_layers"]
    cfgd["num_hidden_layers"] = n_layers
    if args.only == "decode" and args.context > cfgd["max_position_embeddings"]:
        cfgd["max_position_embeddings"] = args.context
    B = args.batch
    rng = random.Random(0)
    _, weight_bytes, kv_per_tok = model_numbers(cfgd, n_layers)
    V = cfgd["vocab_size"]

    if args.only == "decode":
        ctx = max(args.context or CONTEXT, args.steps + args.warmup + 64)
        eng, _ = make_engine(cfgd, args, B, ctx)
        reqs = start_decoding(eng, rng, V, B, ctx - args.steps - args.warmup - 4 * B - 2, args.steps + args.warmup + 4 * B + 8)
        for _ in range(args.warmup):
            eng.step()
        before = eng.info()
        ms = timed_steps(eng, args.steps, B) / args.steps
        info = eng.info()
        print(json.dumps({"only": "decode", "batch": B, "layers": n_layers, "context": ctx, "ms_per_step": round(ms, 4),
                          "launches_per_step": (info["launches"] - before["launches"]) / args.steps,
                          "graph_replays": info["graph_replays"] - before["graph_replays"], "fallback_calls": info["fallback_calls"]}))
        stop(eng, reqs)
        return 0

    maxB = max(B, 64) if not args.only else 1
    # the position table and the longest sequence leave room for the stagger of a batch's prompts
    cfgd["max_position_embeddings"] = CONTEXT + STAGGER
    eng, setup_s = make_engine(cfgd, args, maxB, CONTEXT + STAGGER)

    # ---- prefill: one prompt of 2,048 tokens, whole and in 512-token portions ------------------------
    n_prompt = args.tokens if (args.only == "prefill" and 0 < args.tokens <= PREFILL_TOKENS) else PREFILL_TOKENS
    pf_ms = time_prefill(eng, rng, V, n_prompt, args.chunk if args.only == "prefill" else 0)
    pf = statistics.median(pf_ms)
    if args.only == "prefill":
        info = eng.info()
        print(json.dumps({"only": "prefill", "layers": n_layers, "tokens": n_prompt, "chunk": args.chunk, "ms": round(pf, 3),
                          "spread_ms": spread(pf_ms), "launches": info["launches"], "fallback_calls": info["fallback_calls"],
                          "gemm": os.environ.get("IMP_B200_GEMM", "tcgen05")}))
        return 0
    pf_flops = prefill_flops(cfgd, n_layers, PREFILL_TOKENS)
    pf512 = time_prefill(eng, rng, V, PREFILL_TOKENS, 512, reps=5)
    prefill = {"value": round(PREFILL_TOKENS / pf * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pf, 3),
               "frac": round(pf_flops / (pf * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
               "frac_of_sustained": round(pf_flops / (pf * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4),
               "spread_ms": spread(pf_ms),
               "in_512_portions": {"value": round(PREFILL_TOKENS / statistics.median(pf512) * 1e3, 1),
                                   "ms": round(statistics.median(pf512), 3), "spread_ms": spread(pf512)}}

    # ---- the headline: K decode steps at batch B with contexts ending at 4096, device-timed, then K more by the
    # ---- wall clock through the same calls (the end-to-end figure), clocks sampled throughout ----------------
    K_, W = args.steps, args.warmup
    slack = 4 * B            # prompts finish their prefill at different steps: the early ones decode a few tokens first
    plen = CONTEXT - 2 * (K_ + W) - slack - 2
    with ClockSampler(0) as clocks:
        reqs = start_decoding(eng, rng, V, B, plen, 2 * (K_ + W) + slack + 2)
        for _ in range(W):
            eng.step()
        before = eng.info()
        ms = timed_steps(eng, K_, B) / K_
        after = eng.info()
        for _ in range(W):
            eng.step()
        t0 = time.perf_counter()
        for _ in range(K_):
            outs = eng.step()
            assert len(outs) == B
        e2e_ms = (time.perf_counter() - t0) / K_ * 1e3
        h2d = eng.info()["h2d_bytes_last_step"]
        stop(eng, reqs)
    value = B / ms * 1e3
    mean_ctx = CONTEXT - (K_ + W) - K_ / 2.0 - slack / 2.0
    step_bytes = weight_bytes + B * mean_ctx * kv_per_tok
    achieved = step_bytes / (ms * 1e-3) / 1e9
    launches = after["launches"] - before["launches"]

    # ---- the configuration's own protocol: 2,048 -> 4,096 at batch 1, 8 and 64 ------------------------------
    protocol, points = {}, {}
    if not args.quick:
        for b in (1, 8, 64):
            r = decode_protocol(eng, rng, cfgd, n_layers, b, peaks)
            protocol[f"b{b}"] = r
            points[f"decode_b{b}"] = r["all"]["tok_s"]
            points[f"decode_b{b}_ms"] = r["all"]["ms"]
            points[f"decode_b{b}_frac"] = r["all"]["frac"]
    info = eng.info()
    eng.close()

    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B bf16, context 4096); prefill tok/s at 2,048 tokens",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": K_, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen3-8B-shaped", "layers": n_layers, "layers_of_config": MODEL["num_hidden_layers"],
                   "hidden": cfgd["hidden_size"], "q_heads": cfgd["num_attention_heads"],
                   "kv_heads": cfgd["num_key_value_heads"], "head_dim": cfgd["head_dim"],
                   "intermediate": cfgd["intermediate_size"], "vocab": cfgd["vocab_size"],
                   "global_batch": B, "seq_len": CONTEXT, "max_positions": CONTEXT + STAGGER, "page_size": args.page or PAGE,
                   "weights": "random N(0,0.02) seed 0",
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (16 GB of weights per step)",
                   "cache_fill": "real prefill", "api": "C API through the Python entry point", "peaks": peak_src},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "protocol": protocol,
        "e2e": {"value": round(B / e2e_ms * 1e3, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B + 4},
        "gpu_launches": launches,
        "fallback_calls": info["fallback_calls"],
        "clocks": clocks.summary(),
        "setup_s": round(setup_s, 1),
        "workspace_mb": round(info["workspace_bytes"] / 2 ** 20, 1),
    }
    if not args.quick:
        try:
            line["yardsticks"] = yardsticks(peaks)
            try:
                line["yardsticks"]["attention_prefill_2048"] = attention_yardsticks()
            except Exception as e:     # a yardstick is extra: its absence must not take the line with it
                line["yardsticks"]["attention_prefill_2048"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
            line["yardsticks"]["prefill_2048_on_cublaslt"] = library_arm_prefill(args)
            line["yardsticks"]["prefill_2048_own_ms"] = prefill["ms"]
        except Exception as e:
            line["yardsticks"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    from imp_b200 import capi
    line["library"] = os.path.basename(capi.loaded_library_path() or "")
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------- workloads
def run_workload(args):
    """The two other workloads of the baseline record, through Engine.submit / Engine.step.  Protocol of the
    reference's own bench loop (tools/imp-cli/main.cpp:142-215): synthetic ids, one discarded warm-up, wall clock."""
    from imp_b200 import GenerateParams
    peaks, peak_src = read_peaks()
    rng = random.Random(1)
    if args.workload == "0.6b":
        cfgd = dict(MODEL_06B)
        n_req, chunk, ctx, gen = 64, 512, 8192, 256
        lens = [rng.randint(16, 1024) for _ in range(n_req)]
        gp = GenerateParams(temperature=0.0, max_tokens=gen, ignore_eos=True)
        seed, budget, max_batch = 2, 2048, 64
    else:
        cfgd = dict(MODEL_14B)
        n_req, chunk, ctx, gen = 8, 2048, 16384, 512
        lens = [8192] * n_req
        gp = GenerateParams(temperature=0.7, top_k=40, top_p=0.9, seed=7, max_tokens=gen, ignore_eos=True)
        seed, budget, max_batch = 3, 2048 + 8, 8
    if args.layers:
        cfgd["num_hidden_layers"] = args.layers
    n_layers = cfgd["num_hidden_layers"]
    dtype = args.dtype
    if dtype == "float32":
        cfgd["torch_dtype"] = "float32"
    eng, setup_s = make_engine(cfgd, args, max_batch, ctx, budget=budget, chunk=chunk, dtype=dtype, seed=seed,
                               pool_tokens=sum(lens) + n_req * (gen + 2 * (args.page or PAGE)))
    V = cfgd["vocab_size"]
    warm = eng.generate([random_prompt(rng, V, 40)], GenerateParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert len(warm[0]) == 4
    prompts = [random_prompt(rng, V, n) for n in lens]
    reqs = [eng.submit(p, gp) for p in prompts]
    t0 = time.perf_counter()
    n_steps = decode_only_steps = 0
    decode_s = 0.0
    live = {r.rid for r in reqs}
    first_token_at = {}
    while live:
        all_decoding = len(first_token_at) == n_req      # every prompt has been read: this step only decodes
        t_s = time.perf_counter()
        outs = eng.step()
        dt = time.perf_counter() - t_s
        n_steps += 1
        if all_decoding:
            decode_only_steps += 1
            decode_s += dt
        for o in outs:
            first_token_at.setdefault(o.rid, time.perf_counter() - t0)
            if o.finished:
                live.discard(o.rid)
    eng.drain()
    total_s = time.perf_counter() - t0
    n_out = sum(len(r.output) for r in reqs)
    assert n_out == n_req * gen, f"{n_out} tokens generated, {n_req * gen} expected"
    info = eng.info()
    _, weight_bytes, kv_per_tok = model_numbers(cfgd, n_layers)
    elem = 2 if dtype == "bfloat16" else 4
    line = {"workload": args.workload, "dtype": dtype, "layers": n_layers, "requests": n_req, "prompt_tokens": sum(lens),
            "generated_tokens": n_out, "seconds": round(total_s, 3), "steps": n_steps,
            "generated_tok_s": round(n_out / total_s, 1), "total_tok_s": round((n_out + sum(lens)) / total_s, 1),
            "time_to_last_first_token_s": round(max(first_token_at.values()), 3),
            "prefill_tok_s": round(sum(lens) / max(first_token_at.values()), 1),
            "decode_only_steps": decode_only_steps,
            "decode_ms_per_step": round(decode_s / decode_only_steps * 1e3, 3) if decode_only_steps else None,
            "preemptions": info["scheduler"]["preemptions"], "fallback_calls": info["fallback_calls"],
            "graph_replays": info["graph_replays"], "setup_s": round(setup_s, 1), "peaks": peak_src}
    if decode_only_steps:
        mean_ctx = sum(lens) / n_req + gen / 2
        gbs = (weight_bytes * elem / 2 + n_req * mean_ctx * kv_per_tok * elem / 2) / (decode_s / decode_only_steps) / 1e9
        line["decode_roofline_frac"] = round(gbs / peaks["hbm_gbs"], 4)
    print(json.dumps(line))
    return 0


def run_reference(args):
    """The one offline install the contract describes is attempted once (it cannot succeed: the reference is a
    CMake C++/CUDA project without setup.py or pyproject.toml, it needs CUDA >= 13.1 where this image has 12.9,
    and its configure step fetches googletest, CUTLASS and two more projects from the network)."""
    why = "kekzl/imp is not pip-installable (no setup.py/pyproject.toml; CMake needs CUDA >= 13.1 and network fetches)"
    target = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(target) or not os.listdir(target):
        if os.path.isdir("/root/reference") and os.path.isdir("/opt/wheelhouse"):
            try:
                p = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--find-links",
                                    "/opt/wheelhouse", "--target", target, "/root/reference"], capture_output=True, text=True, timeout=300)
                tail = (p.stderr or p.stdout).strip().splitlines()
                why += f": pip install --target baseline/_ref exited {p.returncode}" + (f" ({tail[-1][:160]})" if tail else "")
            except Exception as e:
                why += f": pip install could not run ({type(e).__name__})"
        else:
            why += ": no reference tree or wheelhouse on this machine, nothing was attempted"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "timeline", "mixed"],
                    help="run one phase only and print its timing (for profiling small cases)")
    ap.add_argument("--workload", default="", choices=["", "0.6b", "14b"], help="one of the two other workloads of the baseline record")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="with --workload: the compute type")
    ap.add_argument("--quick", action="store_true", help="skip the 2,048-step protocol runs and the yardsticks")
    ap.add_argument("--context", type=int, default=0,
                    help="with --only decode: the contexts end here instead of at the configured length (may be longer)")
    ap.add_argument("--tokens", type=int, default=0, help="with --only prefill: tokens of the prompt (at most 2048)")
    ap.add_argument("--chunk", type=int, default=0, help="with --only prefill: portions of this many tokens (0 = whole)")
    ap.add_argument("--page", type=int, default=0, help="tokens per cache page (0 = the default of the engine's configuration)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode kernels one by one (for profilers)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.only == "timeline":
        return run_timeline(args)
    if args.only == "mixed":
        return run_mixed(args)
    if args.workload:
        return run_workload(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
