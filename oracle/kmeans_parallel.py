"""numpy restatement of the reference's k-means|| initialisation.

TEST INFRASTRUCTURE, not product code (see ``oracle/__init__.py``).

Scheme of ``kmeans_parallel`` + ``count_pts_per_centroid`` + ``kmeans_plus_plus``
(src/gpu/kmeans/kmeans_h2o4gpu.cu:331-563, 154-279; src/gpu/kmeans/kmeans_h2o4gpu.h:44-126):

1. one uniformly drawn row is the first candidate;
2. ``R = min(8, int(2 + ln k))`` rounds: cost(row) = squared distance to the nearest candidate
   so far, phi = sum of costs, a row becomes a candidate with probability
   ``min(1, 2 k cost / phi)`` (``prob_x > prob_threshold``, kmeans_h2o4gpu.cu:446-462);
3. more than k candidates: weight = rows nearest to each candidate, then k of them are drawn by
   D^2-weighted k-means++; otherwise all are kept.

Parity unpinned against the reference's own random stream: the reference draws from
``thrust::default_random_engine`` / ``std::mt19937`` with per-row ``discard`` and holds no test
or golden vector for this function, so its draws are not reproduced.  This restatement fixes
the random source instead: Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as
1, 2, 3", SC'11), key = seed, counter = (global row, round, stream), pinned in the tests by the
published known-answer vector of that generator.  The sums below are formed in the order the
CUDA kernels use, so the CUDA path is compared with this file draw for draw.
"""
import math

import numpy as np

STREAM_SAMPLE, STREAM_FIRST, STREAM_PLUSPLUS, STREAM_FILL = 7, 8, 9, 10
_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Philox4x32-10; counters are arrays (or scalars) of 32-bit words, key two Python ints."""
    c0, c1, c2, c3 = (np.atleast_1d(np.asarray(c, dtype=np.uint64)) & _MASK for c in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0 &= 0xFFFFFFFF
    k1 &= 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        n0 = (p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0)
        n1 = p1 & _MASK
        n2 = (p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1)
        n3 = p0 & _MASK
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def u01_53(a, b):
    """Uniform in the open interval (0, 1) from two 32-bit words: 52 random bits plus one half."""
    v = ((a >> np.uint64(6)) << np.uint64(26)) | (b >> np.uint64(6))
    return (v.astype(np.float64) + 0.5) * (1.0 / 4503599627370496.0)


def _warp_sum(a):
    """Butterfly sum over the last axis (32 lanes), as __shfl_xor with 16, 8, 4, 2, 1; lane 0."""
    idx = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        a = a + a[..., idx ^ o]
    return a[..., 0]


def row_cost(X, C):
    """Squared distance of every row to its nearest centre: argmin in float64, then the distance
    by direct differences with the lane-strided summation order of the CUDA kernel."""
    X64 = X.astype(np.float64)
    C64 = C.astype(np.float64)
    cn = (C64 * C64).sum(1)
    n, d = X.shape
    out = np.empty(n)
    lab = np.empty(n, dtype=np.int64)
    dp = -(-d // 32) * 32
    for s in range(0, n, 8192):
        xs = X64[s:s + 8192]
        sc = cn[None, :] - 2.0 * (xs @ C64.T)
        l = sc.argmin(1)
        lab[s:s + 8192] = l
        q = xs - C64[l]
        q = q * q
        qp = np.zeros((q.shape[0], dp))
        qp[:, :d] = q
        lanes = np.zeros((q.shape[0], 32))
        for j in range(dp // 32):            # lane t adds columns t, t + 32, ... in order
            lanes = lanes + qp[:, j * 32:(j + 1) * 32]
        out[s:s + 8192] = _warp_sum(lanes)
    return out, lab


def tree_sum(v):
    """Sum in the order of the two-stage CUDA reduction: 1024 blocks x 256 threads grid-stride,
    butterfly per warp, the eight warps in sequence; then one warp adds 32 block sums per lane in
    sequence and finishes with a butterfly."""
    n = v.shape[0]
    span = 1024 * 256
    reps = -(-n // span)
    p = np.zeros(reps * span)
    p[:n] = v
    p = p.reshape(reps, 1024, 256)
    acc = np.zeros((1024, 256))
    for j in range(reps):
        acc = acc + p[j]
    w = _warp_sum(acc.reshape(1024, 8, 32))
    blocks = np.zeros(1024)
    for j in range(8):
        blocks = blocks + w[:, j]
    lanes = np.zeros(32)
    blocks = blocks.reshape(32, 32)
    for j in range(32):
        lanes = lanes + blocks[:, j]
    return float(_warp_sum(lanes))


def _weighted_pick(wm, u, taken):
    """First index whose running sum exceeds u * total; sums in per-thread chunks of a 1024-thread
    block, then the chunks in sequence."""
    m = wm.shape[0]
    chunk = -(-m // 1024)
    local = np.zeros(1024)
    for t in range(1024):
        s = 0.0
        for i in range(t * chunk, min(m, (t + 1) * chunk)):
            s += float(wm[i])
        local[t] = s
    prefix = np.zeros(1025)
    acc = 0.0
    for t in range(1024):
        prefix[t] = acc
        acc += local[t]
    prefix[1024] = acc
    total = acc
    pick = -1
    if total > 0:
        target = u * total
        for t in range(1024):
            b, e = t * chunk, min(m, (t + 1) * chunk)
            if prefix[t + 1] > target and not (prefix[t] > target) and b < e:
                a = prefix[t]
                last_pos = -1
                for i in range(b, e):
                    if wm[i] > 0:
                        last_pos = i
                    a += float(wm[i])
                    if a > target:
                        pick = i
                        break
                if pick < 0:
                    pick = last_pos
                break
        if pick < 0:
            pos = np.flatnonzero(wm > 0)
            if pos.size:
                pick = int(pos[-1])
    if pick < 0:
        free = np.flatnonzero(~taken)
        pick = int(free[0]) if free.size else 0
    return pick


def weight_units(w):
    """Sample weights as the fixed-point integers of the CUDA path: wmax < 2^e,
    units = rint(w 2^(15-e)) 2^15 + rint(remainder 2^15); returns (units, weight of one unit)."""
    w = np.asarray(w, dtype=np.float64)
    _, e = math.frexp(float(w.max()))
    v = w * 2.0 ** (15 - e)
    p0 = np.rint(v)
    p1 = np.rint((v - p0) * 32768.0)
    return p0 * 32768.0 + p1, 2.0 ** -(30 - e)


def kmeans_parallel(X, k, seed, sample_weight=None):
    """Returns (centres k x d, global row index of every centre, rows of all candidates).  With sample
    weights a row's cost is weight x squared distance and a candidate's weight the sum of the weights
    of the rows nearest to it (the first candidate stays a uniform draw)."""
    n, d = X.shape
    w64 = None if sample_weight is None else np.asarray(sample_weight).astype(np.float64)
    k0, k1 = seed & 0xFFFFFFFF, 0
    r = philox4x32_10(0, 0, 0, STREAM_FIRST, k0, k1)
    first = ((int(r[0][0]) << 32) | int(r[1][0])) % n
    picked = [first]
    fresh = [first]
    cost = np.full(n, np.finfo(np.float64).max)
    rows = np.arange(n, dtype=np.uint64)
    rounds = min(8, int(2 + math.log(k)))
    for rnd in range(rounds):
        if fresh:
            c, _ = row_cost(X, X[np.asarray(fresh)])
            cost = np.minimum(cost, c)
        cw = cost if w64 is None else cost * w64
        phi = tree_sum(cw)
        fresh = []
        if not phi > 0:
            continue
        rr = philox4x32_10(rows & _MASK, rows >> np.uint64(32), rnd, STREAM_SAMPLE, k0, k1)
        u = u01_53(rr[0], rr[1])
        p = (2.0 * k * cw) / phi
        fresh = [int(i) for i in np.flatnonzero(p > u)]
        picked.extend(fresh)
    m = len(picked)
    if m <= k:
        out = list(picked)
        ctr = 0
        while len(out) < k:
            r = philox4x32_10(ctr, 0, 0, STREAM_FILL, k0, k1)
            ctr += 1
            row = ((int(r[0][0]) << 32) | int(r[1][0])) % n
            if row not in out:
                out.append(row)
        return X[np.asarray(out)].copy(), np.asarray(out), np.asarray(picked)
    cand = X[np.asarray(picked)]
    _, lab = row_cost(X, cand)
    if w64 is None:
        w = np.bincount(lab, minlength=m).astype(np.float64)
    else:
        units, unit = weight_units(np.asarray(sample_weight))
        w = np.bincount(lab, weights=units, minlength=m) * unit
    cand64 = cand.astype(np.float64)
    mind = np.full(m, np.finfo(np.float64).max)
    wm = w.copy()
    taken = np.zeros(m, dtype=bool)
    chosen = []
    for step in range(k):
        r = philox4x32_10(step, 0, 0, STREAM_PLUSPLUS, k0, k1)
        u = float(u01_53(r[0], r[1])[0])
        c = _weighted_pick(wm, u, taken)
        taken[c] = True
        chosen.append(c)
        s = np.zeros(m)
        for t in range(d):                   # one thread per candidate, columns in order
            q = cand64[:, t] - cand64[c, t]
            s = s + q * q
        mind = np.minimum(mind, s)
        wm = w * mind
    chosen = np.asarray(chosen)
    return cand[chosen].copy(), np.asarray(picked)[chosen], np.asarray(picked)


def potential(X, C):
    """Sum of squared distances to the nearest centre."""
    return float(row_cost(X, C)[0].sum())
