"""Randomised parity: random index geometries, neighbour counts, iteration caps and candidate quotas
(tiny partitions, duplicate rows, rounded keys, far queries included) -- neighbour ids and distance
bits must equal the sequential restatement's on every case."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _case(seed, c):
    rng = np.random.default_rng(seed * 100000 + c)
    kind = c % 6
    N = int(rng.integers(1, 200)) if kind == 0 else int(rng.integers(200, 20000))
    d = int(rng.choice([3, 8, 16, 24, 37, 64, 100, 128]))
    L = int(rng.integers(1, 4)); S = int(rng.integers(1, 9)); T = int(rng.choice([1, 2, 3, 7, 10, 16, 20]))
    P = int(rng.choice([1, 2, 3, 7, 20, 100]))
    k = int(rng.integers(1, min(N, 60) + 1))
    outer = int(rng.choice([1, 5, 50, 5000])); mc = int(rng.choice([0, 1, k, 3 * k, 10 * k, 1000000]))
    lat = int(rng.integers(1, d + 1))
    A = rng.standard_normal((lat, d)).astype(np.float32)
    data = (rng.standard_normal((N, lat)).astype(np.float32) @ A).astype(np.float32)
    query = (rng.standard_normal((12, lat)).astype(np.float32) @ A).astype(np.float32)
    if kind == 1:
        data, query = np.round(data), np.round(query * 2) / 2
    if kind == 2:
        query *= 5
    if kind == 3:
        data[N // 2:] = data[:N - N // 2]          # duplicate points: equal distances, ties by id
    proj = rng.standard_normal((L * S, d)).astype(np.float32)
    proj /= np.linalg.norm(proj, axis=1, keepdims=True)
    return dict(N=N, d=d, L=L, S=S, T=T, P=P, k=k, outer=outer, mc=mc, kind=kind), data, query, proj


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_configurations_match_the_oracle(seed):
    from dciknn_cuda_b200 import DCI
    for c in range(40):
        p, data, query, proj = _case(seed, c)
        g = DCI(p["d"], p["L"], p["S"], p["P"], p["T"], proj=torch.from_numpy(proj))
        g.add(torch.from_numpy(data).cuda())
        ids, dists = g.query(torch.from_numpy(query).cuda(), p["k"], p["outer"], max_num_candidates=p["mc"],
                             return_int_ids=True)
        o = oracle.OracleDCI(p["d"], p["L"], p["S"], p["P"], p["T"], proj)
        o.add(data)
        oi, od = o.query(query, p["k"], p["outer"], p["mc"])
        assert np.array_equal(ids.cpu().numpy(), oi), (c, p)
        assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32)), (c, p)
        # the same with all work items on two CTAs: every CTA then takes many (query, partition) pairs in
        # turn, so whatever it keeps in shared memory from one pair must not leak into the next
        g.set_max_ctas(2)
        ids, dists = g.query(torch.from_numpy(query).cuda(), p["k"], p["outer"], max_num_candidates=p["mc"],
                             return_int_ids=True)
        assert np.array_equal(ids.cpu().numpy(), oi), ("two CTAs", c, p)
        assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32)), ("two CTAs", c, p)
        g.free()


def test_small_partitions_warp_kernel_and_cta_kernel_agree_with_the_oracle():
    """Partitions of at most 32 points with at most 32 windows per composite index are answered by a
    kernel that gives one warp to every (query, partition) pair; with the per-phase cycle counters on,
    the same handle runs the CTA kernel.  Both must return the oracle's neighbours, distance bits and
    (for up to two composite indices) per-pair counters."""
    from dciknn_cuda_b200 import DCI
    rng = np.random.default_rng(2)
    ran = 0
    for t in range(90):
        N = int(rng.integers(1, 600)); P = int(rng.integers(max(1, N // 32), N + 2)); d = int(rng.choice([3, 8, 16, 37, 100]))
        L = int(rng.integers(1, 4)); S = int(rng.integers(1, 9)); T = int(rng.choice([1, 2, 3, 7, 10, 16]))
        k = int(rng.integers(1, min(N, 40) + 1)); outer = int(rng.choice([1, 5, 5000])); mc = int(rng.choice([0, 1, k, 10 * k, 10 ** 6]))
        data = rng.standard_normal((N, d)).astype(np.float32)
        query = rng.standard_normal((9, d)).astype(np.float32)
        if t % 3 == 0:
            data, query = np.round(data), np.round(query * 2) / 2        # equal keys and equal distances
        proj = rng.standard_normal((L * S, d)).astype(np.float32)
        proj /= np.linalg.norm(proj, axis=1, keepdims=True)
        ppb = -(-N // P)
        if ppb > 32 or S * (-(-ppb // T) + 2) > 32:
            continue
        ran += 1
        o = oracle.OracleDCI(d, L, S, P, T, proj)
        o.add(data)
        oi, od, ost = o.query(query, k, outer, mc, want_stats=True)
        g = DCI(d, L, S, P, T, proj=torch.from_numpy(proj))
        g.add(torch.from_numpy(data).cuda())
        q = torch.from_numpy(query).cuda()
        for mode in ("warp", "warp+counters", "cta"):
            g.enable_work_stats(mode == "warp+counters" and L <= 2, phases=mode == "cta")
            ids, dists = g.query(q, k, outer, max_num_candidates=mc, return_int_ids=True)
            assert np.array_equal(ids.cpu().numpy(), oi), (mode, t)
            assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32)), (mode, t)
            if mode == "warp+counters" and L <= 2:
                gs = g.get_work_stats(9).numpy()
                for col in (1, 2, 3, 4, 5):
                    assert np.array_equal(gs[:, :, col], ost[:, :, col]), (mode, t, col)
        g.free()
    assert ran >= 30


@pytest.mark.parametrize("n", [17960, 17984, 18000, 18004, 18005, 18006, 18020, 18100])
def test_partition_sizes_around_the_shared_memory_limit_of_the_build(n):
    """The index build sorts a segment in shared memory when it fits and in a global slab when it
    does not; partition sizes on both sides of that limit must build the same index."""
    from dciknn_cuda_b200 import DCI
    rng = np.random.default_rng(n)
    data = rng.standard_normal((n, 4)).astype(np.float32)
    proj = rng.standard_normal((2, 4)).astype(np.float32)
    proj /= np.linalg.norm(proj, axis=1, keepdims=True)
    g = DCI(4, 1, 2, 1, 10, proj=torch.from_numpy(proj))
    g.add(torch.from_numpy(data).cuda())
    keys, ids = g.get_index()
    okeys, oids = oracle.build(oracle.project(proj, data), 1)
    assert np.array_equal(np.asarray(ids), oids)
    assert np.array_equal(np.asarray(keys).view(np.uint32), okeys.view(np.uint32))
    g.free()
