"""numpy restatement of the Lloyd solver on the reference's CPU path.

TEST INFRASTRUCTURE, not product code (see ``oracle/__init__.py``).

The reference's ``n_gpus=0`` path is scikit-learn's dense Lloyd solver
(src/interface_py/h2o4gpu/solvers/kmeans.py:738-750).  This file restates one
iteration of it so that tests can (a) walk the trajectory step by step
("teacher forcing": feed the oracle's centres of iteration t to one GPU step)
and (b) run it in float64 from float32 data, which sklearn's public API cannot
do without changing the data's dtype.  Behaviour restated, with the place each
rule comes from in scikit-learn's published algorithm:

* E-step: label = argmin_j (|c_j|^2 - 2 x.c_j), |x|^2 omitted, first minimum
  wins (``_k_means_lloyd.pyx`` chunked update; same tie rule as the GPU
  reference's ``make_new_labels``, src/gpu/kmeans/kmeans_labels.h:360-377).
* M-step: per-cluster sums and counts; empty clusters are relocated to the
  points farthest from their assigned centre, the donor cluster loses that
  point (``_relocate_empty_clusters_dense``); centres = sums / counts; a
  cluster that is still empty takes the centre of the largest cluster
  (``_average_centers``).
* Loop: T x (E, M), stop early when labels repeat ("strict convergence") or the
  squared shift <= tol, then one more E-step so labels match the returned
  centres (``_kmeans_single_lloyd``; the GPU reference does the same final
  pass, src/gpu/kmeans/kmeans_impl.h:217-231).
* fit() subtracts the column mean of X from X and init and adds it back.
* Sample weights (``fit(X, sample_weight=w)``): sums of w * x, counts of w, inertia of
  w * distance; the farthest points of the empty-cluster rule are chosen by the unweighted
  distance and move with their weight (``_relocate_empty_clusters_dense``).

The GPU reference's output conventions restated here: transform returns
|(|x|^2 + |c|^2 - 2 x.c)| (squared, no sqrt) as one column-major n x k block
(src/gpu/kmeans/kmeans_labels.cu:115-244, kmeans_labels.h:217-244;
src/interface_py/h2o4gpu/solvers/kmeans.py:420-421 reshapes order='F').
"""
import numpy as np

_CHUNK = 8192


def _as(X, dtype):
    return np.ascontiguousarray(X, dtype=dtype)


def scores(X, C):
    """|c|^2 - 2 x.c for every (row, centre); the quantity the E-step minimises."""
    cn = np.einsum("ij,ij->i", C, C)
    return cn[None, :] - 2.0 * (X @ C.T)


def assign(X, C, dtype=np.float64, return_gap=False):
    """E-step.  Returns int32 labels (and the best / second-best squared distances)."""
    C = _as(C, dtype)
    n = X.shape[0]
    k = C.shape[0]
    labels = np.empty(n, dtype=np.int32)
    best = np.empty(n, dtype=dtype)
    second = np.full(n, np.inf, dtype=dtype)
    for s in range(0, n, _CHUNK):
        Xc = _as(X[s:s + _CHUNK], dtype)
        S = scores(Xc, C)
        lab = np.argmin(S, axis=1)
        labels[s:s + _CHUNK] = lab
        if return_gap:
            xn = np.einsum("ij,ij->i", Xc, Xc)
            r = np.arange(Xc.shape[0])
            best[s:s + _CHUNK] = S[r, lab] + xn
            if k > 1:
                S[r, lab] = np.inf
                second[s:s + _CHUNK] = S.min(axis=1) + xn
    if return_gap:
        return labels, best, second
    return labels


def near_tie_mask(X, C, rel=1e-5, dtype=np.float64):
    """Rows whose two nearest-centre squared distances differ by < rel (relative)."""
    _, best, second = assign(X, C, dtype=dtype, return_gap=True)
    return (second - best) < rel * np.maximum(np.abs(second), np.finfo(dtype).tiny)


def sums_counts(X, labels, k, dtype=np.float64, sample_weight=None):
    """Un-normalised per-cluster sums (k x d) and integer counts (k); with sample weights the sums of
    w * x and the per-cluster sums of w (float)."""
    d = X.shape[1]
    sums = np.zeros((k, d), dtype=dtype)
    if sample_weight is None:
        counts = np.bincount(labels, minlength=k).astype(np.int64)
    else:
        counts = np.bincount(labels, weights=_as(sample_weight, dtype), minlength=k).astype(dtype)
    for s in range(0, X.shape[0], _CHUNK * 8):
        Xc = _as(X[s:s + _CHUNK * 8], dtype)
        if sample_weight is not None:
            Xc = Xc * _as(sample_weight[s:s + _CHUNK * 8], dtype)[:, None]
        lc = labels[s:s + _CHUNK * 8]
        order = np.argsort(lc, kind="stable")
        ls = lc[order]
        starts = np.flatnonzero(np.r_[True, ls[1:] != ls[:-1]])
        sums[ls[starts]] += np.add.reduceat(Xc[order], starts, axis=0)
    return sums, counts


def relocate_empty(X, labels, C_old, sums, counts, order="sklearn", dtype=np.float64, sample_weight=None):
    """Empty-cluster rule.  ``order='sklearn'`` picks the far points exactly as
    scikit-learn does (``np.argpartition`` tail, reversed: not a sorted order when
    two or more clusters are empty); ``order='descending'`` hands the farthest
    point to the lowest empty cluster id, the next farthest to the next, which
    is the engine's rule.  Returns the list of (cluster id, row) relocations."""
    empty = np.flatnonzero(counts == 0)
    moved = []
    if empty.size == 0:
        return moved
    Xd = _as(X, dtype)
    dist = ((Xd - _as(C_old, dtype)[labels]) ** 2).sum(axis=1)
    if dist.max() == 0:
        return moved
    ne = empty.size
    if order == "sklearn":
        far = np.argpartition(dist, -ne)[:-ne - 1:-1]
    else:
        # descending distance, ties -> lowest row index
        far = np.lexsort((np.arange(dist.size), -dist))[:ne]
    for cid, row in zip(empty, far):
        old = labels[row]
        w = 1 if sample_weight is None else dtype(sample_weight[row])
        sums[old] -= w * Xd[row]
        sums[cid] = w * Xd[row]
        counts[cid] = w
        counts[old] -= w
        moved.append((int(cid), int(row)))
    return moved


def average(sums, counts):
    """sums / counts; a still-empty cluster copies the largest cluster's row as
    it stands when its turn comes (already averaged if its index is lower)."""
    C = sums.copy()
    big = int(np.argmax(counts))
    for j in range(C.shape[0]):
        if counts[j] > 0:
            C[j] *= 1.0 / counts[j]
        else:
            C[j] = C[big]
    return C


def step(X, C, dtype=np.float64, order="sklearn", sample_weight=None):
    """One Lloyd iteration from centres C.  Returns (C_new, labels, counts, moved);
    counts are the ones after relocation."""
    k = C.shape[0]
    labels = assign(X, C, dtype=dtype)
    sums, counts = sums_counts(X, labels, k, dtype=dtype, sample_weight=sample_weight)
    moved = relocate_empty(X, labels, C, sums, counts, order=order, dtype=dtype, sample_weight=sample_weight)
    return average(sums, counts), labels, counts, moved


def fit(X, init, max_iter, tol=0.0, dtype=np.float64, center=True, order="sklearn",
        stop_on_repeat=True, keep_trajectory=False, sample_weight=None):
    """Whole fit.  Returns dict(centers, labels, n_iter, trajectory?)."""
    Xw = _as(X, dtype)
    C = _as(init, dtype).copy()
    if center:
        mean = Xw.mean(axis=0)
        Xw = Xw - mean
        C -= mean
    labels_old = np.full(Xw.shape[0], -1, dtype=np.int32)
    traj = []
    strict = False
    it = 0
    for it in range(max_iter):
        C_new, labels, _, moved = step(Xw, C, dtype=dtype, order=order, sample_weight=sample_weight)
        shift = float(((C_new - C) ** 2).sum())
        C = C_new
        if keep_trajectory:
            traj.append((C + mean if center else C.copy(), labels.copy(), moved))
        if stop_on_repeat and np.array_equal(labels, labels_old):
            strict = True
            break
        if shift <= tol:
            break
        labels_old = labels
    if not strict:
        labels = assign(Xw, C, dtype=dtype)
    if center:
        C = C + mean
    out = {"centers": C, "labels": labels, "n_iter": it + 1}
    if keep_trajectory:
        out["trajectory"] = traj
    return out


def inertia(X, C, labels, dtype=np.float64, sample_weight=None):
    Xd = _as(X, dtype)
    dist = ((Xd - _as(C, dtype)[labels]) ** 2).sum(axis=1)
    if sample_weight is not None:
        dist = dist * _as(sample_weight, dtype)
    return float(dist.sum())


def transform_sq_colmajor(X, C, dtype=np.float64):
    """The GPU reference's transform output: |xn + cn - 2 x.c| flattened column-major."""
    Xd, Cd = _as(X, dtype), _as(C, dtype)
    xn = np.einsum("ij,ij->i", Xd, Xd)
    D = np.abs(xn[:, None] + scores(Xd, Cd))
    return np.asfortranarray(D).ravel(order="F")


def transform_sq_exact(X, C, dtype=np.float64):
    """Squared distances by direct differences (no cancellation), n x k."""
    Xd, Cd = _as(X, dtype), _as(C, dtype)
    out = np.empty((Xd.shape[0], Cd.shape[0]), dtype=dtype)
    for j in range(Cd.shape[0]):
        out[:, j] = ((Xd - Cd[j]) ** 2).sum(axis=1)
    return out


def match_centers(A, B):
    """Greedy nearest matching of the rows of B onto the rows of A (used where
    relocated cluster ids may legitimately be permuted).  Returns perm with
    B[perm] aligned to A."""
    A = np.asarray(A, dtype=np.float64)
    B = np.asarray(B, dtype=np.float64)
    D = ((A[:, None, :] - B[None, :, :]) ** 2).sum(-1)
    perm = np.full(A.shape[0], -1)
    used = np.zeros(B.shape[0], bool)
    for i in np.argsort(D.min(axis=1)):
        row = np.where(used, np.inf, D[i])
        j = int(np.argmin(row))
        perm[i] = j
        used[j] = True
    return perm
