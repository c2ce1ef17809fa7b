"""Command line in the manner of the reference's imp-cli (tools/imp-cli/args.cpp:65-187).

Option names and meanings are the reference's where it has them (--model,
--prompt, --max-tokens, --temperature, --top-p, --top-k, --seed, --min-p,
--repeat-penalty, --frequency-penalty, --presence-penalty, --typical-p,
--dry-multiplier, --dry-base, --dry-allowed-length, --dry-penalty-last-n,
--mirostat, --mirostat-tau, --mirostat-eta, --device,
--no-cuda-graphs, --prefill-chunk-size, --bench, --bench-pp, --bench-reps);
--random-weights, --weights-seed, --weights-std, --dtype, --kv-pages,
--page-size, --max-batch, --max-seq-len, --bench-batch are this engine's.
Without a tokenizer the prompt is a list of token ids ("5,17,3" or "5 17 3");
any other text is taken byte by byte.  Output is the generated token ids on
stdout and the reference's two timing lines (`pp ...`, `tg ...`) on stderr
(tools/imp-cli/main.cpp:212-215, 570-572).
"""
from __future__ import annotations

import argparse
import sys
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="imp-cli", description="Qwen3 dense decoder on one B200")
    p.add_argument("--model", required=True, help="model folder (config.json + model.safetensors; "
                                                  "config.json alone with --random-weights)")
    p.add_argument("--prompt", default=None, help="token ids (comma or space separated) or text taken as bytes")
    p.add_argument("--max-tokens", type=int, default=256, help="maximum tokens to generate (default: 256)")
    p.add_argument("--temperature", type=float, default=0.7, help="sampling temperature, 0 = greedy (default: 0.7)")
    p.add_argument("--top-p", type=float, default=0.9, help="top-p (nucleus) sampling (default: 0.9)")
    p.add_argument("--top-k", type=int, default=40, help="top-k sampling (default: 40)")
    p.add_argument("--seed", type=int, default=-1, help="random seed, -1 for random (default: -1)")
    p.add_argument("--min-p", type=float, default=0.0, help="min-p threshold (default: 0.0 = disabled)")
    p.add_argument("--repeat-penalty", type=float, default=1.0, help="repetition penalty (default: 1.0 = disabled)")
    p.add_argument("--frequency-penalty", type=float, default=0.0)
    p.add_argument("--presence-penalty", type=float, default=0.0)
    p.add_argument("--repeat-last-n", type=int, default=0, help="penalty window, 0 = all tokens")
    p.add_argument("--typical-p", type=float, default=1.0, help="locally typical sampling (default: 1.0 = disabled)")
    p.add_argument("--dry-multiplier", type=float, default=0.0, help="DRY n-gram penalty scale (default: 0.0 = disabled)")
    p.add_argument("--dry-base", type=float, default=1.75, help="DRY exponential base (default: 1.75)")
    p.add_argument("--dry-allowed-length", type=int, default=2,
                   help="DRY: n-grams at or below this not penalized (default: 2)")
    p.add_argument("--dry-penalty-last-n", type=int, default=0, help="DRY: how far back to scan (default: 0 = all)")
    p.add_argument("--mirostat", type=int, default=0, help="Mirostat sampling (0=off, 2=v2) (default: 0)")
    p.add_argument("--mirostat-tau", type=float, default=5.0, help="Mirostat target entropy (default: 5.0)")
    p.add_argument("--mirostat-eta", type=float, default=0.1, help="Mirostat learning rate (default: 0.1)")
    p.add_argument("--device", type=int, default=0, help="CUDA device id (default: 0)")
    p.add_argument("--no-cuda-graphs", action="store_true", help="disable CUDA graph capture for decode")
    p.add_argument("--prefill-chunk-size", type=int, default=0, help="max tokens per prefill portion (0 = no cut)")
    p.add_argument("--bench", action="store_true", help="synthetic benchmark mode")
    p.add_argument("--bench-pp", type=int, default=512, help="synthetic prompt token count (default: 512)")
    p.add_argument("--bench-reps", type=int, default=3, help="repetitions to average (default: 3)")
    p.add_argument("--bench-batch", type=int, default=1, help="requests decoded together in --bench (default: 1)")
    p.add_argument("--random-weights", action="store_true", help="fill the tensors from --weights-seed "
                                                                 "instead of reading model.safetensors")
    p.add_argument("--weights-seed", type=int, default=0)
    p.add_argument("--weights-std", type=float, default=0.02)
    p.add_argument("--dtype", choices=["bf16", "fp32", "bfloat16", "float32"], default="bf16")
    p.add_argument("--kv-pages", type=int, default=0, help="cache pages per group (0 = from memory)")
    p.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default: 16)")
    p.add_argument("--max-batch", type=int, default=32, help="requests decoded together (default: 32)")
    p.add_argument("--max-seq-len", type=int, default=4096, help="longest context of a request (default: 4096)")
    p.add_argument("--ignore-eos", action="store_true")
    return p


def parse_prompt(text: str, vocab_size: int) -> List[int]:
    parts = text.replace(",", " ").split()
    try:
        ids = [int(x) for x in parts]
    except ValueError:
        ids = list(text.encode("utf-8"))
    if not ids:
        raise SystemExit("error: empty prompt")
    for t in ids:
        if not 0 <= t < vocab_size:
            raise SystemExit(f"error: prompt token {t} is outside the vocabulary of {vocab_size}")
    return ids


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if not args.bench and args.prompt is None:
        print("error: --prompt is required (or --bench)", file=sys.stderr)
        return 1

    from .config.engine_config import EngineConfig
    from .config.registry import load_config
    from .engine.engine import Engine, GenerateParams

    dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype)
    need = (args.bench_pp + args.max_tokens + 1) if args.bench else 0
    ecfg = EngineConfig(device_id=args.device, max_batch_size=max(args.max_batch, args.bench_batch),
                        max_seq_len=max(args.max_seq_len, need), kv_cache_max_blocks=args.kv_pages,
                        kv_block_size=args.page_size, prefill_chunk_size=args.prefill_chunk_size,
                        max_batch_tokens=max(2048, args.max_batch, args.bench_batch), compute_dtype=dtype,
                        enable_cuda_graphs=not args.no_cuda_graphs)
    t0 = time.time()
    if args.random_weights:
        mc = load_config(args.model)
        eng = Engine.from_random(mc, ecfg, seed=args.weights_seed, std=args.weights_std)
    else:
        eng = Engine.from_folder(args.model, ecfg)
    cache = eng.info()["cache"]
    print(f"model ready in {time.time() - t0:.1f}s ({eng.model.architecture}, {dtype}, "
          f"{cache['num_pages']} cache pages of {cache['page_size']})", file=sys.stderr)
    V = eng.vocab_size

    if args.bench:
        return run_bench(eng, args, V)

    prompt = parse_prompt(args.prompt, V)
    gp = GenerateParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                        max_tokens=args.max_tokens, seed=args.seed, min_p=args.min_p,
                        repetition_penalty=args.repeat_penalty, frequency_penalty=args.frequency_penalty,
                        presence_penalty=args.presence_penalty, repeat_last_n=args.repeat_last_n,
                        typical_p=args.typical_p, dry_multiplier=args.dry_multiplier, dry_base=args.dry_base,
                        dry_allowed_length=args.dry_allowed_length, dry_penalty_last_n=args.dry_penalty_last_n,
                        mirostat=args.mirostat, mirostat_tau=args.mirostat_tau, mirostat_eta=args.mirostat_eta,
                        ignore_eos=args.ignore_eos)
    req = eng.submit(prompt, gp)
    if req.done:
        print(f"error: request refused: {req.status.name.lower()}", file=sys.stderr)
        return 1
    # a step returns when its tokens have reached the host, so the wall clock brackets the device's work
    t_start = time.perf_counter()
    t_first = None
    n_out, finished = 0, False
    while not finished:
        for out in eng.step():
            finished = finished or out.finished
            if out.token >= 0:
                if t_first is None:
                    t_first = time.perf_counter()
                n_out += 1
                sys.stdout.write(f"{out.token} ")
                sys.stdout.flush()
    eng.drain()
    t_end = time.perf_counter()
    sys.stdout.write("\n")
    pp_ms = ((t_first or t_end) - t_start) * 1e3
    tg_ms = (t_end - (t_first or t_end)) * 1e3
    print(f"pp {len(prompt):5d} tokens in {pp_ms:8.2f} ms  ({len(prompt) / max(pp_ms, 1e-9) * 1e3:7.2f} tok/s)",
          file=sys.stderr)
    print(f"tg {n_out:5d} tokens in {tg_ms:8.2f} ms  "
          f"({(n_out - 1) / max(tg_ms, 1e-9) * 1e3 if n_out > 1 else 0.0:7.2f} tok/s)", file=sys.stderr)
    return 0


def run_bench(eng, args, V: int) -> int:
    """The reference's --bench protocol (tools/imp-cli/main.cpp:142-215): ids i % vocab, one discarded
    warm-up cycle, timed prefills, timed greedy decode runs with EOS ignored; averages."""
    from .engine.engine import GenerateParams

    B, pp, tg, reps = args.bench_batch, args.bench_pp, args.max_tokens, args.bench_reps
    tokens = [i % V for i in range(pp)]
    gp = GenerateParams(temperature=0.0, max_tokens=tg + 1, ignore_eos=True)
    print(f"Benchmark: pp={pp}, tg={tg}, batch={B}, reps={reps}", file=sys.stderr)

    def prefill():
        reqs = [eng.submit(tokens, gp) for _ in range(B)]
        waiting = {r.rid for r in reqs}
        while waiting:
            for o in eng.step():
                waiting.discard(o.rid)
        return reqs

    def drain(reqs):
        live = {r.rid for r in reqs}
        while live:
            for o in eng.step():
                if o.finished:
                    live.discard(o.rid)
        eng.drain()
        for r in reqs:
            r.release()

    print("Warmup...", file=sys.stderr)
    drain(prefill())
    pp_ms = 0.0
    for _ in range(reps):
        t0 = time.perf_counter()
        reqs = prefill()
        pp_ms += (time.perf_counter() - t0) * 1e3
        for r in reqs:
            eng.cancel(r)
        eng.drain()
    tg_ms = 0.0
    for _ in range(reps):
        reqs = prefill()
        t0 = time.perf_counter()
        drain(reqs)
        tg_ms += (time.perf_counter() - t0) * 1e3
    pp_avg, tg_avg = pp_ms / reps, tg_ms / reps
    print(f"pp {pp * B:5d} tokens  avg {pp_avg:8.2f} ms  ({pp * B / pp_avg * 1e3:7.2f} tok/s)  [{reps} reps]",
          file=sys.stderr)
    print(f"tg {tg * B:5d} tokens  avg {tg_avg:8.2f} ms  ({tg * B / tg_avg * 1e3:7.2f} tok/s)  [{reps} reps]",
          file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
