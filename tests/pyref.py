"""Second, independent restatement of internal/logits/sampler.go in numpy scalars.

Pure-Python loops: for small cases only.  It exists so that the C oracle is not checked
against itself; both follow the reference line by line (sampler.go:10-31, 98-296).
"""
import numpy as np

f32 = np.float32
f64 = np.float64


def fast_exp(x):
    x = f32(x)
    if x > f32(88.0):
        return f32(3.4028235e38)
    if x < f32(-88.0):
        return f32(0.0)
    ln2 = f32(0.693147180559945309417)
    ln2inv = f32(1.44269504088896340736)
    half = f32(0.5)
    if x < 0:
        k = int(f32(f32(x * ln2inv) - half))  # int() truncates toward zero like Go's int32()
    else:
        k = int(f32(f32(x * ln2inv) + half))
    r = f32(x - f32(f32(k) * ln2))
    r2 = f32(r * r)
    r3 = f32(r2 * r)
    r4 = f32(r2 * r2)
    poly = f32(f32(1.0) + r)
    poly = f32(poly + f32(r2 * f32(0.5)))
    poly = f32(poly + f32(r3 * f32(0.16666667)))
    poly = f32(poly + f32(r4 * f32(0.041666667)))
    poly = f32(poly + f32(f32(r4 * r) * f32(0.008333333)))
    scale = np.array([((k + 127) << 23) & 0xFFFFFFFF], dtype=np.uint32).view(np.float32)[0]
    return f32(poly * scale)


def sample(logits, recent, exclude, p):
    """logits: 1-D float32 array, patched in place.  p: mapping with the normalised
    parameters.  Returns (token, idx list, prob list, cut)."""
    V = len(logits)
    pen = f32(p["repeat_penalty"])
    if pen > f32(1.0) and len(recent) > 0:
        start = max(len(recent) - int(p["repeat_last_n"]), 0)
        seen, order = set(), []
        for t in recent[start:]:
            t = int(t)
            if 0 <= t < V and t not in seen:
                seen.add(t)
                order.append(t)
        for t in exclude:
            seen.discard(int(t))
        for t in order:
            if t not in seen:
                continue
            if logits[t] > 0:
                logits[t] = f32(logits[t] / pen)
            else:
                logits[t] = f32(logits[t] * pen)
    temp = f32(p["temperature"])
    top_p = f32(p["top_p"])
    if p["greedy"] or (int(p["top_k"]) == 1 and top_p >= 1 and temp == 1):
        best, bv = 0, logits[0]
        for i in range(1, V):
            if logits[i] > bv:
                best, bv = i, logits[i]
        return best, [], [], 0
    inv_temp = f32(f32(1.0) / temp)
    k = min(int(p["top_k"]), V)
    idx, val = [], []
    for i in range(V):
        v = f32(logits[i] * inv_temp)
        pos = len(val)
        while pos > 0 and val[pos - 1] < v:
            pos -= 1
        if pos >= k:
            continue
        idx.insert(pos, i)
        val.insert(pos, v)
        del idx[k:], val[k:]
    if not idx:
        return 0, [], [], 0
    maxv = max(val)
    prob = [f64(fast_exp(f32(v - maxv))) for v in val]
    s = f64(0.0)
    for e in prob:
        s = f64(s + e)
    if s == 0:
        return idx[0], idx, prob, 0
    inv = f64(1.0) / s
    prob = [f64(e * inv) for e in prob]
    min_p = f32(p["min_p"])
    if min_p > 0:
        thr = f64(prob[0] * f64(min_p))
        nidx, nprob, ns = [], [], f64(0.0)
        for i, e in zip(idx, prob):
            if e >= thr:
                nidx.append(i)
                nprob.append(e)
                ns = f64(ns + e)
        if len(nprob) < len(prob):
            idx, prob = nidx, nprob
            if ns > 0:
                sc = f64(1.0) / ns
                prob = [f64(e * sc) for e in prob]
    cut = len(prob)
    if top_p < 1:
        c = f64(0.0)
        for i, e in enumerate(prob):
            c = f64(c + e)
            if f32(c) >= top_p:
                cut = i + 1
                break
    r = f64(p["uniform"])
    c = f64(0.0)
    for i in range(cut):
        c = f64(c + prob[i])
        if r <= c:
            return idx[i], idx, prob, cut
    return idx[cut - 1], idx, prob, cut
