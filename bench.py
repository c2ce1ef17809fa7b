#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen3-8B shape, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at the default batch (8) with every
sequence's context ending at the configured context length (4096): K decode steps timed with CUDA
events after W warm-up steps, through the engine's step function (cache, kernels, CUDA graph) with
the batch arrays and the argmax on the device side of the clock.  `e2e` is the same workload through
the public entry point (`Engine.submit` / `Engine.step`): host token lists in, sampled token ids out,
every step with its host-to-device copy of the batch arrays from pinned memory and its
device-to-host read of the tokens.  `prefill` is one 2,048-token prompt in one step; `points` holds
decode at batch 1 and 64.  Roofline fractions use MEASURED_PEAKS.json when the driver wrote it,
else the stated fallback.  Every decode step streams all weights (about 16 GB), far more than the
126 MB L2, so no explicit L2 flush is needed between timed iterations ("inputs larger than L2").

For profiling and for other sizes one phase can be run alone; it prints its own short JSON line:
    python bench.py --only decode [--batch B] [--context C] [--page P] [--layers N] [--no-graphs]
    python bench.py --only prefill [--tokens T] [--layers N]
(`--context` may exceed the configured 4096: the cache and the position table grow with it.)
"""
import argparse
import json
import os
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
CONTEXT = 4096
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


def fill_cache(eng, rid, n_tokens):
    """Give request `rid` n_tokens of (random) keys and values without computing them."""
    eng.cache.add_request(rid)
    eng.cache.reserve(rid, n_tokens)
    eng.cache.commit(rid, n_tokens)


def time_decode(eng, B, ctx_end, steps, warmup, torch, K, StepEntry):
    """Device time of `steps` decode steps at batch B whose contexts end at ctx_end.  Returns (ms/step, launches/step)."""
    from imp_b200.ops import library
    start = ctx_end - steps - warmup
    rids = [f"d{B}_{i}" for i in range(B)]
    for r in rids:
        fill_cache(eng, r, start)
    tok = torch.zeros(B, dtype=torch.int32, device=eng.model.rt.device)
    host_tok = [1] * B

    def one():
        logits = eng.stepper.step([StepEntry(r, [t], [0]) for r, t in zip(rids, host_tok)])
        K.argmax(logits, tok)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    before = library.launch_calls
    graphs = len(eng.stepper._graphs)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    eng.stepper.check_device_status("decode bench")
    calls = (library.launch_calls - before) / steps
    for r in rids:
        eng.stepper.finish(r)
    return ms, calls


def count_forward_launches(eng, B, torch, StepEntry):
    """Launcher calls of one eager decode forward of B sequences (what one graph replay stands for)."""
    from imp_b200.ops import library
    rids = [f"c{i}" for i in range(B)]
    for r in rids:
        fill_cache(eng, r, 32)
    saved = eng.stepper.use_cuda_graphs
    eng.stepper.use_cuda_graphs = False
    before = library.launch_calls
    eng.stepper.step([StepEntry(r, [1], [0]) for r in rids])
    n = library.launch_calls - before
    eng.stepper.use_cuda_graphs = saved
    torch.cuda.synchronize()
    for r in rids:
        eng.stepper.finish(r)
    return n


def run_ours(args):
    import torch

    from imp_b200 import Engine, EngineConfig, GenerateParams, StepEntry, config_from_dict
    from imp_b200.ops import kernels as K
    from imp_b200.ops import library

    peaks, peak_src = read_peaks()
    cfgd = dict(MODEL)
    n_layers = args.layers or MODEL["num_hidden_layers"]
    cfgd["num_hidden_layers"] = n_layers
    if args.only == "decode" and args.context > cfgd["max_position_embeddings"]:
        cfgd["max_position_embeddings"] = args.context
    mc = config_from_dict(cfgd)
    torch.cuda.set_device(0)
    B = args.batch
    maxB = max(B, 64) if not args.only else B
    _, _, kv_per_tok = model_numbers(cfgd, n_layers)
    max_ctx = max(CONTEXT, args.context) if args.only == "decode" else CONTEXT
    ecfg = EngineConfig(max_batch_size=maxB, max_seq_len=max_ctx, kv_block_size=args.page or PAGE,
                        kv_cache_tokens=maxB * max_ctx + 4 * CONTEXT, max_batch_tokens=PREFILL_TOKENS,
                        compute_dtype="bfloat16", enable_cuda_graphs=not args.no_graphs)
    t0 = time.time()
    eng = Engine.from_random(mc, ecfg, seed=0, std=0.02)
    for g in eng.cache.paged:          # stand-in cache contents for sequences that are not really prefilled
        g.storage.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    setup_s = time.time() - t0
    _, weight_bytes, _ = model_numbers(cfgd, n_layers)

    gen = torch.Generator().manual_seed(0)
    if args.only == "decode":
        ctx = max(args.context or CONTEXT, args.steps + args.warmup + 1)
        ms, calls = time_decode(eng, B, ctx, args.steps, args.warmup, torch, K, StepEntry)
        print(json.dumps({"only": "decode", "batch": B, "layers": n_layers, "context": ctx, "ms_per_step": round(ms, 4),
                          "launcher_calls_per_step": calls}))
        return 0
    # ---- prefill: one prompt of 2,048 tokens in one step --------------------------------------------
    n_prompt = PREFILL_TOKENS
    if args.only == "prefill" and 0 < args.tokens <= PREFILL_TOKENS:
        n_prompt = args.tokens
    prompt = torch.randint(0, mc.vocab_size, (n_prompt,), generator=gen).tolist()
    pf_ms = []
    for i in range(1 + 7):      # one warm-up, seven timed: the products run at the power cap and vary by a few per cent
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.stepper.step([StepEntry("pf", prompt, [n_prompt - 1])])
        e1.record()
        torch.cuda.synchronize()
        eng.stepper.finish("pf")
        if i > 0:
            pf_ms.append(e0.elapsed_time(e1))
    eng.stepper.check_device_status("prefill bench")
    pf = statistics.median(pf_ms)
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": n_layers, "tokens": n_prompt, "ms": round(pf, 3)}))
        return 0
    pf_flops = prefill_flops(cfgd, n_layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / pf * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pf, 3),
               "frac": round(pf_flops / (pf * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}

    # ---- decode at the headline batch, device-timed, with clocks sampled ---------------------------------
    per_forward = count_forward_launches(eng, B, torch, StepEntry)
    with ClockSampler(0) as clocks:
        ms, calls = time_decode(eng, B, CONTEXT, args.steps, args.warmup, torch, K, StepEntry)
    value = B / ms * 1e3
    mean_ctx = CONTEXT - args.steps / 2.0
    step_bytes = weight_bytes + B * mean_ctx * kv_per_tok
    achieved = step_bytes / (ms * 1e-3) / 1e9
    # A graph replay stands for `per_forward` kernel launches of this library; the argmax adds one.
    launches = int(args.steps * (per_forward + 1)) if eng.stepper._graphs else int(calls * args.steps)

    # ---- other batch sizes -------------------------------------------------------------------------
    points = {}
    for b in (1, 64):
        steps_b = max(8, min(args.steps, 32))
        ms_b, _ = time_decode(eng, b, CONTEXT, steps_b, args.warmup, torch, K, StepEntry)
        points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)
        points[f"decode_b{b}_ms"] = round(ms_b, 3)

    # ---- end to end through the entry point: real prompts, host tokens in and out -----------------------
    e2e_steps, e2e_warm = args.steps, args.warmup
    # Prompts finish their prefill at different steps (they share the token budget), so the early ones
    # decode a few tokens before the timed region starts: leave room for that, so that all B requests
    # are still decoding at its end.
    slack = 4 * B
    plen = CONTEXT - e2e_steps - e2e_warm - 1 - slack
    gp = GenerateParams(temperature=0.0, max_tokens=e2e_steps + e2e_warm + 1 + slack, ignore_eos=True)
    reqs = [eng.submit(torch.randint(0, mc.vocab_size, (plen,), generator=gen).tolist(), gp) for _ in range(B)]
    while any(not r.output for r in reqs):
        eng.step()
    for _ in range(e2e_warm):
        eng.step()
    torch.cuda.synchronize()
    t_e2e = time.perf_counter()
    step_ms = []
    for _ in range(e2e_steps):
        t_s = time.perf_counter()
        eng.step()
        step_ms.append((time.perf_counter() - t_s) * 1e3)
    torch.cuda.synchronize()
    if os.environ.get("IMP_BENCH_DEBUG"):
        print("e2e step ms:", [round(x, 2) for x in step_ms], "graphs", sorted(eng.stepper._graphs),
              "running", len(eng.scheduler.running), file=sys.stderr)
    e2e_ms = (time.perf_counter() - t_e2e) / e2e_steps * 1e3
    assert all(not r.done and len(r.output) >= 1 + e2e_warm + e2e_steps for r in reqs), "a request left the batch"
    for r in reqs:
        eng.scheduler.cancel(r.rid)
    buf = eng.stepper.buffers
    h2d = 4 * (buf.small_words + len(buf.bt_off) * B * buf.max_pages)
    d2h = 4 * B + 4

    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B bf16, context 4096); prefill tok/s at 2,048 tokens",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen3-8B-shaped", "layers": n_layers, "layers_of_config": MODEL["num_hidden_layers"],
                   "hidden": cfgd["hidden_size"], "q_heads": cfgd["num_attention_heads"],
                   "kv_heads": cfgd["num_key_value_heads"], "head_dim": cfgd["head_dim"],
                   "intermediate": cfgd["intermediate_size"], "vocab": cfgd["vocab_size"],
                   "global_batch": B, "seq_len": CONTEXT, "page_size": args.page or PAGE, "weights": "random N(0,0.02) seed 0",
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (16 GB of weights per step)",
                   "cache_fill": "random pages for value/points, real prefill for e2e",
                   "peaks": peak_src},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "e2e": {"value": round(B / e2e_ms * 1e3, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "setup_s": round(setup_s, 1),
        "library": os.path.basename(library.loaded_library_path() or ""),
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    # The reference is a CMake C++/CUDA project (no setup.py or pyproject.toml; CUDA >= 13.1 and
    # network fetches at configure time), so the one offline install attempt fails before any build.
    print(json.dumps({"impl": "reference",
                      "unavailable": "kekzl/imp is not pip-installable (no setup.py/pyproject.toml; CMake needs "
                                     "CUDA >= 13.1 and network fetches): pip install --target baseline/_ref failed"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="", choices=["", "decode", "prefill"],
                    help="run one phase only and print its timing (for profiling small cases)")
    ap.add_argument("--context", type=int, default=0,
                    help="with --only decode: the contexts end here instead of at the configured length (may be longer)")
    ap.add_argument("--tokens", type=int, default=0, help="with --only prefill: tokens of the prompt (at most 2048)")
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
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
