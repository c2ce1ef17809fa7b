"""Plain twin of the sampler: penalties, min-p, top-k, top-p and the draw, in float64 on the CPU.

Order and formulas from kekzl/imp (src/graph/executor.cu:43-115 for the order;
src/compute/sampling.cu:700-736 penalties, :767-810 min-p, :253-557 softmax of
logits/T, top-k, nucleus cut, renormalise, draw; :811-915 DRY; :917-1064
typical-p; :1067-1236 Mirostat v2).  Conventions of this engine
where the reference leaves room: ties at a cut are kept, and the draw walks the
kept tokens in index order.
"""
import math

import numpy as np


def penalize(logits, history, repetition=1.0, frequency=0.0, presence=0.0, last_n=0):
    x = np.array(logits, dtype=np.float64)
    h = list(history)[-last_n:] if last_n > 0 else list(history)
    counts = {}
    for t in h:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        v = x[t]
        if repetition != 1.0:
            v = v / repetition if v > 0 else v * repetition
        v -= frequency * c
        v -= presence
        x[t] = v
    return x


def kept_set(logits, temperature, top_k=0, top_p=1.0, min_p=0.0):
    """(kept mask, e) with e_i = exp(x_i/T - max/T) for kept-by-min-p tokens."""
    x = np.array(logits, dtype=np.float64)
    V = x.size
    keep = np.ones(V, dtype=bool)
    if min_p > 0:
        keep &= x >= x.max() + math.log(min_p)
    e = np.where(keep, np.exp((x - x.max()) / temperature), 0.0)
    z = e.sum()
    if 0 < top_k < V:
        kth = np.sort(x[keep])[::-1][min(top_k, keep.sum()) - 1]
        keep &= x >= kth
    if 0.0 < top_p < 1.0:
        order = np.argsort(-x, kind="stable")
        order = order[keep[order]]
        cum = np.cumsum(e[order])
        n = int(np.searchsorted(cum, top_p * z, side="left")) + 1
        n = min(n, order.size)
        cut = x[order[n - 1]]
        keep &= x >= cut
    return keep, e


def draw_interval(logits, temperature, token, **filters):
    """The interval [lo, hi) of uniform numbers that select `token` (index-order walk), and the kept mask."""
    keep, e = kept_set(logits, temperature, **filters)
    mass = np.where(keep, e, 0.0)
    total = mass.sum()
    cum = np.cumsum(mass)
    hi = cum[token] / total
    lo = (cum[token] - mass[token]) / total
    return lo, hi, keep


def sample(logits, temperature, u, **filters):
    if temperature <= 0 or filters.get("top_k", 0) == 1:
        x = np.asarray(logits)
        return int(np.flatnonzero(x == x.max())[0])
    keep, e = kept_set(logits, temperature, **filters)
    mass = np.where(keep, e, 0.0)
    cum = np.cumsum(mass)
    return int(np.searchsorted(cum, u * cum[-1], side="right"))


def dry(tokens, multiplier, base, allowed_length, last_n=0):
    """token -> penalty, by the reference's scan (src/compute/sampling.cu:826-880): for every
    position of the window, how many tokens before it equal the sequence's end, walking back."""
    n = len(tokens)
    if multiplier <= 0 or n < 2:
        return {}
    start = max(0, n - last_n) if last_n > 0 else 0
    longest = {}
    for pos in range(start, n):
        m, a, b = 0, pos - 1, n - 1
        while a >= start and b >= 0 and tokens[a] == tokens[b]:
            m, a, b = m + 1, a - 1, b - 1
        if m > allowed_length:
            longest[tokens[pos]] = max(longest.get(tokens[pos], 0), m)
    return {t: multiplier * base ** (m - allowed_length) for t, m in longest.items()}


def typical_keep(logits, typical_p, min_p=0.0):
    """Mask of the tokens locally typical filtering keeps (src/compute/sampling.cu:917-1064, with an
    exact cut instead of the reference's 256-bucket histogram): smallest |surprise - entropy| first,
    until the kept mass reaches typical_p; ties at the cut kept."""
    x = np.array(logits, dtype=np.float64)
    alive = np.isfinite(x)
    if min_p > 0:
        alive &= x >= x.max() + math.log(min_p)
    e = np.where(alive, np.exp(x - x.max()), 0.0)
    p = e / e.sum()
    with np.errstate(divide="ignore"):
        surprise = np.where(alive, -np.log2(np.where(p > 0, p, 1.0)), np.inf)
    H = float((p[alive] * surprise[alive]).sum())
    dev = np.abs(surprise - H)
    order = np.argsort(dev, kind="stable")
    order = order[alive[order]]
    cum = np.cumsum(p[order])
    n = min(int(np.searchsorted(cum, typical_p, side="left")) + 1, order.size)
    cut = dev[order[n - 1]]
    return alive & (dev <= cut), dev, cut


def mirostat_v2(logits, temperature, mu, u):
    """(token, surprise in bits) of one Mirostat v2 draw (src/compute/sampling.cu:1072-1200): keep
    surprise <= mu under softmax(logits / T) (everything if nothing passes), draw in index order."""
    x = np.array(logits, dtype=np.float64)
    T = temperature if temperature > 0 else 1.0
    e = np.exp((x - x.max()) / T)
    z = e.sum()
    threshold = x.max() + T * (math.log(z) - mu * math.log(2.0))
    keep = x >= threshold
    if not keep.any():
        keep[:] = True
    mass = np.where(keep, e, 0.0)
    cum = np.cumsum(mass)
    tok = int(np.searchsorted(cum, u * cum[-1], side="right"))
    return tok, -math.log2(max(e[tok] / z, 1e-30)), keep
