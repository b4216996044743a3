"""numpy statement of the parallel ("rank") formulation the CUDA traversal kernel uses.

The reference walks each partition with a sequential prioritized loop
(src/dci_cuda_kernel.cu:401-626).  The kernel instead enumerates every window
of every simple index, orders the windows of one composite index by
(priority, simple index, order inside the index) to get the outer iteration in
which each would be visited, and derives per point the iteration and lane of
its promotion.  This file states that computation on the host so that it can be
checked against the sequential oracle without a GPU.
"""
import numpy as np


def windows_of_index(keys, q, n, T):
    """All windows of one simple index in visiting order inside the index.

    Returns (start, priority) arrays.  Left windows start at s-T+1-j*T while the
    start is > -T, right windows at s+1+j*T while the start is < n+T-1
    (dci_cuda_kernel.cu:250-273).  Inside an index the visiting order is the
    merge of the two runs with "right first iff strictly nearer"; the single
    right window that exists when every key is < q compares as nearer than any
    left window (its signed difference is negative), so it comes first.
    """
    q = np.float32(q)
    s = int(np.searchsorted(keys, q, side="left")) - 1          # last key < q
    nl = -(-(s + 1) // T)
    nr = -(-(n + T - 2 - s) // T)
    lstart = s - T + 1 - T * np.arange(nl)
    rstart = s + 1 + T * np.arange(nr)
    lpri = np.abs(keys[np.maximum(lstart, 0)] - q).astype(np.float32)
    rpri = np.abs(keys[np.minimum(rstart, n - 1)] - q).astype(np.float32)
    special = (s == n - 1) and nr > 0
    if special:
        starts = np.concatenate([rstart, lstart])
        pri = np.concatenate([rpri, lpri])
    else:
        starts = np.concatenate([lstart, rstart])
        pri = np.concatenate([lpri, rpri])
    return starts, pri


def partition_candidates(skeys, sids, lo, n, L, S, T, qproj, knn, outer, max_cand):
    """Candidate mask (indexed by id - lo) and (stop, lane0_total) of one work item."""
    BIG = np.iinfo(np.int64).max
    K = np.full(n, BIG, np.int64)
    lane = np.full(n, -1, np.int64)
    for m in range(L):
        starts, pris, hs = [], [], []
        for h in range(S):
            i = m * S + h
            st, pr = windows_of_index(skeys[i, lo:lo + n], qproj[i], n, T)
            starts.append(st); pris.append(pr); hs.append(np.full(len(st), h))
        starts, pris, hs = map(np.concatenate, (starts, pris, hs))
        # window ids are laid out in (h, order inside index) order, so a stable
        # sort by priority alone gives the visiting order of the composite
        order = np.argsort(pris, kind="stable")
        rank = np.empty(len(order), np.int64)
        rank[order] = np.arange(len(order))
        promo = np.full(n, -1, np.int64)
        plane = np.full(n, -1, np.int64)
        for w in range(len(starts)):
            i = m * S + hs[w]
            a, b = max(starts[w], 0), min(starts[w] + T, n)
            if b <= a:
                continue
            pts = sids[i, lo + a:lo + b] - lo
            val = rank[w]
            upd = val > promo[pts]
            promo[pts[upd]] = val
            plane[pts[upd]] = (np.arange(a, b) - starts[w])[upd]
        better = promo < K                      # ties keep the lower composite
        K[better] = promo[better]
        lane[better] = plane[better]
    limit = n * S * T
    l0 = np.sort(K[lane == 0])
    stop = limit - 1
    if len(l0) >= knn:
        a = l0[knn - 1]
        b = max(a, outer * S - 1)
        c = max(a, l0[max_cand - 1]) if (max_cand > knn and len(l0) >= max_cand) else \
            (a if max_cand <= knn else BIG)
        stop = min(b, c, limit - 1)
    return K <= stop, int(stop), int((K[lane == 0] <= stop).sum())
