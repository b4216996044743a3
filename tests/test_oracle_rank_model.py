"""The parallel rank formulation must reproduce the sequential oracle exactly:
same promoted set, same stop iteration, same lane-0 count, on random cases that
include duplicate keys, queries outside the key range, n < T, T = 1, S = 1."""
import numpy as np
import pytest

from oracle import oracle
from tests.rank_model import partition_candidates


def _case(rng, trial):
    n = int(rng.integers(1, 300)); d = 12
    L = int(rng.integers(1, 4)); S = int(rng.integers(1, 6)); T = int(rng.integers(1, 13))
    P = int(rng.integers(1, 5))
    knn = int(rng.integers(1, 8)); max_cand = knn * int(rng.integers(0, 11)); outer = int(rng.integers(1, 60))
    N = n * P - int(rng.integers(0, min(n, 3)))
    N = max(N, 1)
    data = rng.standard_normal((N, d)).astype(np.float32)
    if trial % 5 == 0:
        data = np.round(data)                      # many equal keys
    proj = rng.standard_normal((L * S, d)).astype(np.float32)
    proj /= np.linalg.norm(proj, axis=1, keepdims=True)
    q = (rng.standard_normal((3, d)) * (1 if trial % 3 else 6)).astype(np.float32)
    return dict(N=N, d=d, L=L, S=S, T=T, P=P, knn=min(knn, N), max_cand=max_cand, outer=outer,
                data=data, proj=proj, q=q)


@pytest.mark.parametrize("seed", range(4))
def test_rank_model_matches_sequential_oracle(seed):
    rng = np.random.default_rng(100 + seed)
    for trial in range(60):
        c = _case(rng, trial)
        o = oracle.OracleDCI(c["d"], c["L"], c["S"], c["P"], c["T"], c["proj"])
        o.add(c["data"])
        ids, dists, stats, mask = o.query(c["q"], c["knn"], c["outer"], c["max_cand"],
                                          want_stats=True, want_mask=True)
        qproj = oracle.project(c["proj"], c["q"])
        ppb = -(-c["N"] // c["P"])
        for qi in range(c["q"].shape[0]):
            for b in range(c["P"]):
                lo = b * ppb
                n = min(ppb, c["N"] - lo)
                if n <= 0:
                    assert stats[qi, b, 3] == 0
                    continue
                cand, stop, lane0 = partition_candidates(o.skeys, o.sids, lo, n, c["L"], c["S"], c["T"],
                                                         qproj[:, qi], c["knn"], c["outer"], c["max_cand"])
                ref = mask[qi, lo:lo + n].astype(bool)
                assert np.array_equal(cand, ref), (seed, trial, qi, b, {k: c[k] for k in ("N", "L", "S", "T", "P", "knn", "max_cand", "outer")})
                assert lane0 == stats[qi, b, 4]
                if not stats[qi, b, 5] and stats[qi, b, 0] < n * c["S"] * c["T"]:
                    assert stop == stats[qi, b, 0]


def test_bruteforce_and_exhaustive_configuration():
    """With the example's shape (20-point partitions, quota 100 per lane) lane 0
    can never fill its quota, so every point is promoted and the result is exact
    k-NN (dci_cuda_kernel.cu:598-607)."""
    rng = np.random.default_rng(0)
    z = (rng.standard_normal((2100, 50)) @ rng.standard_normal((50, 100))).astype(np.float32)
    data, q = z[:2000], z[2000:2040]
    proj = rng.standard_normal((14, 100)).astype(np.float32)
    proj /= np.linalg.norm(proj, axis=1, keepdims=True)
    o = oracle.OracleDCI(100, 2, 7, 100, 10, proj)
    o.add(data)
    ids, dists, stats = o.query(q, 10, 5000, want_stats=True)
    bi, bd = oracle.bruteforce(data, q, 10)
    assert np.array_equal(ids, bi) and np.array_equal(dists, bd)
    assert (stats[:, :, 3] == 20).all() and (stats[:, :, 5] == 1).all()
