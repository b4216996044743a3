"""GPU parity: every stage of the CUDA path against the CPU oracle, through the
public classes (which call the C ABI).  Integer results (index ids, neighbour
ids, traversal counters) must be identical; keys and distances are fp32 with a
fixed summation order on both sides, so they must be bit-identical too."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


def _dci(c, **kw):
    from dciknn_cuda_b200 import DCI
    return DCI(c["data"].shape[1], c["L"], c["S"], c["P"], c["T"], 0, proj=torch.from_numpy(c["proj"]), **kw)


def _run_both(c, stats=True, max_ctas=0):
    dev = torch.device("cuda", 0)
    data = torch.from_numpy(c["data"]).to(dev)
    query = torch.from_numpy(c["query"]).to(dev)
    g = _dci(c)
    g.set_max_ctas(max_ctas)
    g.add(data)
    if stats:
        g.enable_work_stats(True)
    mc = c.get("max_cand")
    ids, dists = g.query(query, c["k"], c["outer"], max_num_candidates=mc, return_int_ids=True)
    torch.cuda.synchronize()
    o = oracle.OracleDCI(c["data"].shape[1], c["L"], c["S"], c["P"], c["T"], c["proj"])
    o.add(c["data"])
    oi, od, ostats = o.query(c["query"], c["k"], c["outer"], mc, want_stats=True)
    gstats = g.get_work_stats(query.shape[0]).numpy() if stats else None
    return g, o, ids.cpu().numpy(), dists.cpu().numpy(), oi, od, gstats, ostats


def _limits(c):
    """n * S * T per partition: the reference's loop bound (dci_cuda_kernel.cu:458)."""
    N, P = c["data"].shape[0], c["P"]
    ppb = -(-N // P)
    n = np.clip(N - ppb * np.arange(P), 0, ppb)
    return n * c["S"] * c["T"]


def _assert_same(ids, dists, oi, od, gstats, ostats, name="", limits=None):
    assert np.array_equal(ids, oi), "%s: neighbour ids differ in %d of %d rows" % (
        name, int((ids != oi).any(1).sum()), ids.shape[0])
    assert np.array_equal(dists.view(np.uint32), od.view(np.uint32)), "%s: distances not bit-identical" % name
    if gstats is not None:
        for col, what in ((1, "windows"), (2, "entries"), (3, "promoted"), (4, "lane-0 promotions"), (5, "exhausted")):
            assert np.array_equal(gstats[:, :, col], ostats[:, :, col]), "%s: %s differ" % (name, what)
        live = ostats[:, :, 5] == 0
        if limits is not None:      # a loop that ran into its bound reports the bound itself
            live &= ostats[:, :, 0] < limits[None, :]
        assert np.array_equal(gstats[:, :, 0][live], ostats[:, :, 0][live]), "%s: stop iteration differs" % name


def test_directions_unit_norm_and_seeded():
    from dciknn_cuda_b200 import DCI
    a = DCI(100, 2, 7, seed=123).get_proj()
    b = DCI(100, 2, 7, seed=123).get_proj()
    c = DCI(100, 2, 7, seed=124).get_proj()
    assert a.shape == (14, 100)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert torch.allclose(a.norm(dim=1), torch.ones(14), atol=1e-6)
    big = DCI(4096, 4, 16, seed=5).get_proj() * (4096 ** 0.5)      # entries ~ N(0, 1)
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01
    assert abs(float((big ** 4).mean()) - 3.0) < 0.1              # Gaussian kurtosis
    corr = (big[0] * big[1]).mean()
    assert abs(float(corr)) < 0.08


@pytest.mark.parametrize("n,dim,L,S", [(1000, 100, 2, 7), (777, 37, 3, 12), (5000, 128, 2, 10), (300, 960, 3, 12), (64, 8, 1, 1),
                                       # at least 1024 rows of a multiple of 4 coordinates: rows streamed by TMA copies
                                       (3001, 100, 2, 6), (1500, 36, 1, 8), (2049, 960, 3, 12), (1025, 8, 1, 1),
                                       (70000, 96, 2, 10), (4100, 256, 2, 15), (4096, 44, 4, 10),
                                       (2000, 130, 2, 5), (3000, 128, 6, 7)])      # dim % 4 != 0, more than 40 directions
def test_projection_bit_exact(n, dim, L, S):
    from dciknn_cuda_b200 import DCI
    rng = np.random.default_rng(n)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    proj = cases.unit_rows(rng, L * S, dim)
    want = oracle.project(proj, x)
    xd = torch.from_numpy(x).cuda()
    for mode in ("exact", "exact_plain"):
        g = DCI(dim, L, S, proj=torch.from_numpy(proj))
        g.set_projection(mode)
        got = g.project(xd).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), mode
        if mode == "exact":       # an unaligned view of the same rows takes the other kernel
            pad = torch.empty(n * dim + 1, device="cuda")
            pad[1:] = xd.reshape(-1)
            got = g.project(pad[1:].view(n, dim)).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("N,P", [(2000, 100), (103, 10), (13, 40), (10000, 1), (30000, 2), (70000, 1), (140000, 2)])
def test_index_build_matches_oracle(N, P):
    """Covers the shared-memory sort (u16 and u32 payloads) and the global-scratch sort."""
    from dciknn_cuda_b200 import DCI
    rng = np.random.default_rng(N + P)
    dim, L, S = 16, 2, 3
    data = rng.standard_normal((N, dim)).astype(np.float32)
    if N == 2000:
        data = np.round(data * 2) / 2        # duplicate keys: ties must be ordered by id
    proj = cases.unit_rows(rng, L * S, dim)
    g = DCI(dim, L, S, P, 10, proj=torch.from_numpy(proj))
    g.add(torch.from_numpy(data).cuda())
    keys, ids = g.get_index()
    okeys, oids = oracle.build(oracle.project(proj, data), P)
    assert np.array_equal(ids.numpy(), oids)
    assert np.array_equal(keys.numpy().view(np.uint32), okeys.view(np.uint32))


@pytest.mark.parametrize("max_ctas", [0, 1])
@pytest.mark.parametrize("row", cases.EDGE_CASES, ids=[r[0] for r in cases.EDGE_CASES])
def test_query_edge_cases(row, max_ctas):
    """max_ctas = 1: one CTA takes every (query, partition) pair in turn, so nothing it keeps in shared
    memory from one pair may leak into the next."""
    c = cases.edge_case(row)
    _, _, ids, dists, oi, od, gs, os_ = _run_both(c, max_ctas=max_ctas)
    _assert_same(ids, dists, oi, od, gs, os_, c["name"], _limits(c))


def test_example_configuration_is_exact_knn():
    """configs[0]: exhaustive under the reference's stop rule, so the result is exact k-NN."""
    c = cases.example_config()
    c["max_cand"] = None
    _, _, ids, dists, oi, od, gs, os_ = _run_both(c)
    _assert_same(ids, dists, oi, od, gs, os_, "example")
    bi, bd = oracle.bruteforce(c["data"], c["query"], c["k"])
    assert np.array_equal(ids, bi) and np.array_equal(dists.view(np.uint32), bd.view(np.uint32))


@pytest.mark.parametrize("max_ctas", [0, 3])
def test_c2_shaped_partitions(max_ctas):
    """configs[1] cut down to 4 partitions of 10 000 points (shared-memory path, u16 ranks)."""
    c = cases.c2_shaped()
    c["max_cand"] = None
    _, _, ids, dists, oi, od, gs, os_ = _run_both(c, max_ctas=max_ctas)
    _assert_same(ids, dists, oi, od, gs, os_, "c2-shaped")
    assert (os_[:, :, 5] == 0).all()          # the quota stops every partition before it runs out


@pytest.mark.parametrize("shape", ["high_dim", "mixture", "large_k"])
def test_shapes_of_the_other_benchmark_configurations(shape):
    """Cut-down cases with the geometry and data distribution of the other configurations: dim 960 with
    36 simple indices and a quota of 10 000; the 256-centre mixture in dim 96; k = 100 with S = 15 and
    20 000 outer iterations.  Counters included."""
    c = {"high_dim": lambda: cases.high_dim_shaped(n=6000, nq=12, P=3),
         "mixture": lambda: cases.mixture_shaped(n=30000, nq=24, P=3),
         "large_k": lambda: cases.large_k_shaped(n=4800, nq=8, P=4)}[shape]()
    for max_ctas in (0, 2):
        _, _, ids, dists, oi, od, gs, os_ = _run_both(c, max_ctas=max_ctas)
        _assert_same(ids, dists, oi, od, gs, os_, shape, _limits(c))


def test_large_partition_global_scratch_path():
    """One partition of 30 000 points does not fit shared memory: global-scratch variant."""
    rng = np.random.default_rng(3)
    c = dict(data=cases.latent_linear(rng, 30000, 16, 32, 0.01), query=cases.latent_linear(rng, 6, 16, 32, 0.01),
             L=2, S=4, P=1, T=10, k=10, outer=5000, max_cand=None, proj=cases.unit_rows(rng, 8, 32))
    for max_ctas in (0, 1):
        _, _, ids, dists, oi, od, gs, os_ = _run_both(c, max_ctas=max_ctas)
        _assert_same(ids, dists, oi, od, gs, os_, "global-scratch")


@pytest.mark.parametrize("n", [65526, 65530])
def test_partition_sizes_around_the_16_bit_position_limit(n):
    """Positions are kept in 16 bits while ppb + T <= 65536 (a position plus the offset of the window
    grid must fit): 65 526 points with T = 10 are the largest such partition, 65 530 take 32 bits."""
    rng = np.random.default_rng(n)
    c = dict(data=cases.latent_linear(rng, n, 8, 16, 0.01), query=cases.latent_linear(rng, 4, 8, 16, 0.01),
             L=2, S=3, P=1, T=10, k=10, outer=5000, max_cand=None, proj=cases.unit_rows(rng, 6, 16))
    _, _, ids, dists, oi, od, gs, os_ = _run_both(c)
    _assert_same(ids, dists, oi, od, gs, os_, "position limit")


def test_wide_rank_path():
    """More than 65 535 windows per composite index: 32-bit ranks."""
    rng = np.random.default_rng(4)
    c = dict(data=cases.latent_linear(rng, 20000, 8, 16, 0.01), query=cases.latent_linear(rng, 4, 8, 16, 0.01),
             L=1, S=4, P=1, T=1, k=5, outer=5000, max_cand=None, proj=cases.unit_rows(rng, 4, 16))
    for max_ctas in (0, 1):
        _, _, ids, dists, oi, od, gs, os_ = _run_both(c, max_ctas=max_ctas)
        _assert_same(ids, dists, oi, od, gs, os_, "wide-rank")


def test_default_k_returns_every_point():
    """num_neighbours = -1 means k = N (reference core.py:84-85): every point of every
    partition is promoted (lane 0 cannot reach k) and the result is the full sorted list."""
    rng = np.random.default_rng(8)
    c = dict(data=cases.latent_linear(rng, 3000, 8, 16, 0.01), query=cases.latent_linear(rng, 5, 8, 16, 0.01),
             L=2, S=3, P=3, T=10, k=3000, outer=5000, max_cand=None, proj=cases.unit_rows(rng, 6, 16))
    g = _dci(c)
    g.add(torch.from_numpy(c["data"]).cuda())
    ids, dists = g.query(torch.from_numpy(c["query"]).cuda(), return_int_ids=True)      # default k
    bi, bd = oracle.bruteforce(c["data"], c["query"], 3000)
    assert np.array_equal(ids.cpu().numpy(), bi)
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), bd.view(np.uint32))


def test_large_k_uses_global_selection_buffers():
    rng = np.random.default_rng(9)
    c = dict(data=cases.latent_linear(rng, 20000, 8, 16, 0.01), query=cases.latent_linear(rng, 3, 8, 16, 0.01),
             L=2, S=3, P=2, T=10, k=15000, outer=5000, max_cand=None, proj=cases.unit_rows(rng, 6, 16))
    _, _, ids, dists, oi, od, gs, os_ = _run_both(c)
    _assert_same(ids, dists, oi, od, gs, os_, "large-k")


@pytest.mark.parametrize("n,dim,L,S,P,nq,k", [(6000, 64, 2, 4, 2, 11, 10), (4000, 960, 3, 12, 2, 6, 10),
                                              (5000, 24, 2, 3, 2, 19, 100), (30000, 40, 2, 10, 3, 5, 10)])
def test_exhaustive_partitions_take_the_query_group_path(n, dim, L, S, P, nq, k):
    """A quota no partition can meet makes every work item exhaustive; the library then answers
    queries in groups whose distance pass loads each row once for the group.  Results must not change."""
    rng = np.random.default_rng(n + dim)
    c = dict(data=cases.latent_linear(rng, n, 8, dim, 0.01), query=cases.latent_linear(rng, nq, 8, dim, 0.01),
             L=L, S=S, P=P, T=10, k=k, outer=5000, max_cand=1000000, proj=cases.unit_rows(rng, L * S, dim))
    g, _, ids, dists, oi, od, gs, os_ = _run_both(c)
    _assert_same(ids, dists, oi, od, gs, os_, "query-groups")
    g.enable_work_stats(False, phases=True)
    g.query(torch.from_numpy(c["query"]).cuda(), c["k"], c["outer"], max_num_candidates=c["max_cand"])
    assert g.get_phase_cycles()["queries_per_pass"] > 1


def test_query_host_buffers_match_device_buffers():
    c = cases.example_config(n=1000, nq=40)
    g = _dci(c)
    g.add(torch.from_numpy(c["data"]).cuda())
    ids, dists = g.query(torch.from_numpy(c["query"]).cuda(), 10, return_int_ids=True)
    hi, hd = g.query_host(torch.from_numpy(c["query"]), 10)
    assert torch.equal(ids.cpu(), hi) and torch.equal(dists.cpu(), hd)


def test_query_batches_and_repeat_calls_agree():
    c = cases.example_config(n=1500, nq=64)
    g = _dci(c)
    g.add(torch.from_numpy(c["data"]).cuda())
    q = torch.from_numpy(c["query"]).cuda()
    a = g.query(q, 10)
    b = g.query(q, 10)
    one = g.query(q[5], 10)
    assert a[0].dtype == torch.float32 and a[0].shape == (64, 10)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert torch.equal(one[0][0], a[0][5]) and torch.equal(one[1][0], a[1][5])
    assert g.launch_count() > 0


def test_mdci_two_shards_on_one_device_matches_oracle():
    """MDCI's sharding and merge (reference core.py:121-157) with both shards on GPU 0."""
    from dciknn_cuda_b200 import MDCI
    rng = np.random.default_rng(11)
    data = cases.latent_linear(rng, 3001, 20, 48)
    query = cases.latent_linear(rng, 33, 20, 48)
    projs = [cases.unit_rows(rng, 10, 48) for _ in range(3)]
    m = MDCI(48, 2, 5, 20, 10, devices=[0, 0, 0], projs=[torch.from_numpy(p) for p in projs])
    m.add(torch.from_numpy(data))
    ids, dists = m.query(torch.from_numpy(query).cuda(), 10, return_int_ids=True)
    o = oracle.OracleMDCI(48, 2, 5, 20, 10, projs)
    o.add(data)
    oi, od = o.query(query, 10)
    assert np.array_equal(ids.cpu().numpy(), oi)
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32))
    f_ids, _ = m.query(torch.from_numpy(query).cuda(), 10)
    assert f_ids.dtype == torch.float32 and torch.equal(f_ids.long(), ids)


def test_packed_lists_and_their_merge_equal_the_two_tensor_path():
    """dci_b200_query_packed + dci_b200_merge_shards_packed (what MDCI ships between GPUs) against
    dci_b200_query + dci_b200_merge_shards, including a shard shorter than k."""
    from dciknn_cuda_b200 import DCI
    from dciknn_cuda_b200.core import merge_shards, merge_shards_packed
    rng = np.random.default_rng(12)
    query = torch.from_numpy(cases.latent_linear(rng, 21, 10, 32)).cuda()
    sizes, k = (2500, 1800, 4), 7
    packed, ids, dists = [], [], []
    for n in sizes:
        g = DCI(32, 2, 4, 6, 10, 0, seed=100 + n)
        g.add(torch.from_numpy(cases.latent_linear(rng, n, 10, 32)).cuda())
        p = g.query_packed(query, k)
        assert p.shape == (21, k) and p.dtype == torch.int64
        a = torch.full((21, k), -1, dtype=torch.int32, device="cuda")
        d = torch.full((21, k), float("inf"), device="cuda")
        ai, di = g.query(query, min(k, n), return_int_ids=True)
        a[:, :ai.shape[1]], d[:, :di.shape[1]] = ai, di
        assert torch.equal(p >> 32, torch.where(a >= 0, d.view(torch.int32).long(), torch.full_like(p, -1)))
        assert torch.equal(p & 0xFFFFFFFF, torch.where(a >= 0, a.long(), torch.full_like(p, 0xFFFFFFFF)))
        packed.append(p); ids.append(a); dists.append(d)
    offsets = [0, 2501, 5002]
    want = merge_shards(torch.stack(ids).contiguous(), torch.stack(dists).contiguous(), offsets, k)
    got = merge_shards_packed(torch.stack(packed).contiguous(), offsets, k)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1].view(torch.int32), want[1].view(torch.int32))


def test_mdci_with_an_empty_trailing_shard():
    """9 points on 4 shards: the reference's rule leaves the last shard without rows."""
    from dciknn_cuda_b200 import MDCI
    rng = np.random.default_rng(13)
    data = cases.latent_linear(rng, 9, 4, 8)
    query = cases.latent_linear(rng, 5, 4, 8)
    m = MDCI(8, 1, 2, 2, 3, devices=[0, 0, 0, 0], seeds=[1, 2, 3, 4])
    m.add(torch.from_numpy(data))
    assert [g.num_points for g in m.dcis] == [3, 3, 3, 0]
    ids, dists = m.query(torch.from_numpy(query).cuda(), 9, max_num_candidates=1000, return_int_ids=True)
    bi, bd = oracle.bruteforce(data, query, 9)          # every point is retrieved: exact k-NN of all 9
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), bd.view(np.uint32))
    assert np.array_equal(np.sort(ids.cpu().numpy(), 1), np.sort(bi, 1))
