"""Driving bin/trace_run from tests: send steps, wait for each `done`, read the logits files."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def round64(n):
    return (n + 63) // 64 * 64


def run_trace(model_dir, dtype, steps, max_tokens, out_dir, vocab, page_size=None, timeout=600):
    """Run the steps (dicts with step/entries/end) through bin/trace_run.

    Returns {step: float32 array [wanted, vocab]} for the steps that wanted logits.
    """
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            if line.strip() != f"done {st['step']}":
                proc.stdin.close()
                err = proc.stderr.read()
                raise AssertionError(f"trace_run answered {line!r} to step {st['step']}\n{err[-3000:]}")
        proc.stdin.close()
        rc = proc.wait(timeout=timeout)
        err = proc.stderr.read()
        assert rc == 0, f"trace_run exited with {rc}\n{err[-3000:]}"
    finally:
        if proc.poll() is None:
            proc.kill()
    out = {}
    for st in steps:
        n_want = sum(len(e.get("want", [])) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if n_want:
            a = np.fromfile(path, dtype="<f4")
            assert a.size == n_want * vocab, f"step {st['step']}: {a.size} floats for {n_want} rows of {vocab}"
            out[st["step"]] = a.reshape(n_want, vocab)
        else:
            assert not os.path.exists(path), f"step {st['step']} wanted nothing but wrote a file"
    return out


def collect(steps, outputs):
    """{(request id, position): logits row} from the steps and their outputs."""
    pos = {}
    rows = {}
    for st in steps:
        r = 0
        for e in st["entries"]:
            start = pos.get(e["id"], 0)
            for w in e.get("want", []):
                rows[(e["id"], start + w)] = outputs[st["step"]][r]
                r += 1
            pos[e["id"]] = start + len(e["tokens"])
        for rid in st.get("end", []):
            pos.pop(rid, None)
    return rows


# ------------------------------------------------------------------ schedules
def whole(requests):
    """Each request alone, its whole prompt in one step."""
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(requests.items())]


def tail_decode(requests, tail=32):
    """Most of the prompt in one step, then the last `tail` tokens one by one."""
    steps, n = [], 0
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        n += 1
        for i in range(head, len(ids)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [ids[i]], "want": [0]}],
                          "end": [rid] if i == len(ids) - 1 else []})
            n += 1
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(7, 2, 5, 3, 2, 11, 1, 4, 2, 16, 2, 3)):
    """Each request alone, cut into portions of changing size, down to two tokens (and one)."""
    steps, n = [], 0
    for r, (rid, ids) in enumerate(requests.items()):
        i, k = 0, r
        while i < len(ids):
            m = min(sizes[k % len(sizes)], len(ids) - i)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[i:i + m], "want": list(range(m))}],
                          "end": [rid] if i + m == len(ids) else []})
            i += m
            n += 1
    return steps


def mixed(requests, max_live=4, sizes=(5, 2, 9, 3, 2, 6, 13, 2)):
    """Up to `max_live` requests at a time: prompts in portions of changing size for the first
    two thirds of each request, then one token at a time, all in shared steps; a finished
    request's place (and pages) goes to the next one.  Returns (steps, peak of live tokens rounded
    up to 64 per request)."""
    waiting = list(requests.items())
    live = []     # [rid, ids, done, k]
    steps, n, peak, k = [], 0, 0, 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live.append([rid, ids, 0, k])
            k += 3
        entries, ended = [], []
        for item in live:
            rid, ids, done, kk = item
            if (n + kk) % 5 == 4 and len(live) > 1:
                continue                      # sits this step out and goes on later
            prompt_part = (2 * len(ids)) // 3
            if done < prompt_part:
                m = min(sizes[(kk + n) % len(sizes)], prompt_part - done)
            else:
                m = 1
            entries.append({"id": rid, "tokens": ids[done:done + m], "want": list(range(m))})
            item[2] = done + m
            if item[2] == len(ids):
                ended.append(rid)
        if not entries:
            n += 1
            continue
        peak = max(peak, sum(round64(item[2]) for item in live))
        steps.append({"step": n, "entries": entries, "end": ended})
        live = [it for it in live if it[0] not in ended]
        n += 1
    return steps, peak
