"""Properties that do not depend on the size of the oracle, checked at the
benchmark's full size (configs[1]: 1M points x 128, P=100, T=10, L=2, S=10):
rows sorted, ids valid and distinct, distances equal to a recomputation in the
reference's summation order, answers independent of how queries are batched,
host-buffer entry point identical, recall against exact brute force, and -- with
a quota that cannot be met -- exact k-NN."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def full():
    import bench
    cfg = dict(bench.CFG)
    data_h, query_h = bench.make_data(1, cfg["n_points"], 2000, cfg)
    from dciknn_cuda_b200 import DCI
    g = DCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], 0, seed=7)
    data = data_h.cuda()
    g.add(data)
    return cfg, g, data_h, query_h, data


def test_full_size_properties(full):
    cfg, g, data_h, query_h, data = full
    q = query_h.cuda()
    ids, dists = g.query(q, cfg["k"], cfg["outer"], return_int_ids=True)
    ids_c, dists_c = ids.cpu().numpy(), dists.cpu().numpy()
    assert (ids_c >= 0).all() and (ids_c < cfg["n_points"]).all()
    assert (np.diff(dists_c, axis=1) >= 0).all()
    assert all(len(set(r)) == cfg["k"] for r in ids_c[:500])
    # distances are those of the returned points, bit for bit (sequential fma order)
    sub = slice(0, 300)
    pts = data_h.numpy()[ids_c[sub].reshape(-1)]
    qq = np.repeat(query_h.numpy()[sub], cfg["k"], axis=0)
    re = np.array([oracle.bruteforce(pts[i:i + 1], qq[i:i + 1], 1)[1][0, 0] for i in range(0, pts.shape[0], 37)], np.float32)
    assert np.array_equal(re.view(np.uint32), dists_c[sub].reshape(-1)[::37].view(np.uint32))
    # batching does not change a query's answer
    a, d = g.query(q[100:164], cfg["k"], cfg["outer"], return_int_ids=True)
    assert torch.equal(a, ids[100:164]) and torch.equal(d, dists[100:164])
    hi, hd = g.query_host(query_h[:256], cfg["k"], cfg["outer"])
    assert torch.equal(hi, ids[:256].cpu()) and torch.equal(hd, dists[:256].cpu())
    # recall against exact brute force (ground truth with torch on the GPU)
    truth = torch.cdist(q[:200], data).topk(cfg["k"], largest=False).indices
    hit = (ids[:200].long().unsqueeze(2) == truth.unsqueeze(1)).any(2).float().mean().item()
    assert hit >= 0.9, hit


def test_full_size_answers_equal_the_oracle_bit_for_bit(full):
    """The sequential restatement of the reference, run on the index the GPU built (1M points, 100
    partitions of 10 000, 10 020 windows per composite index), must return the GPU's neighbours and
    distance bits for the same queries."""
    cfg, g, data_h, query_h, data = full
    nq = 256
    ids, dists = g.query(query_h[:nq].cuda(), cfg["k"], cfg["outer"], return_int_ids=True)
    keys, sids = g.get_index()
    qproj = oracle.project(g.get_proj().numpy(), query_h[:nq].numpy())
    oi, od = oracle.query_index(keys.numpy(), sids.numpy(), cfg["L"], cfg["S"], cfg["P"], cfg["T"], data_h.numpy(),
                                qproj, query_h[:nq].numpy(), cfg["k"], cfg["outer"], 10 * cfg["k"])
    assert np.array_equal(ids.cpu().numpy(), oi)
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32))


def test_full_size_exhaustive_quota_gives_exact_knn(full):
    cfg, g, data_h, query_h, data = full
    q = query_h[:64].cuda()
    ids, dists = g.query(q, cfg["k"], cfg["outer"], max_num_candidates=10 ** 7, return_int_ids=True)
    d2 = torch.cdist(q, data)
    cand = d2.topk(4 * cfg["k"], largest=False).indices.cpu().numpy()       # exact distances decide among these
    want_ids = np.empty((64, cfg["k"]), np.int32)
    want_d = np.empty((64, cfg["k"]), np.float32)
    dn, qn = data_h.numpy(), query_h.numpy()
    for i in range(64):
        bi, bd = oracle.bruteforce(dn[cand[i]], qn[i:i + 1], cfg["k"])
        want_ids[i], want_d[i] = cand[i][bi[0]], bd[0]
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), want_d.view(np.uint32))
    assert (ids.cpu().numpy() == want_ids).mean() > 0.999      # id order can differ only at exact distance ties


def test_full_size_tensor_core_projection_moves_few_results(full):
    """Keys from the tcgen05 3xTF32 projection differ from the exact ones in their last bits, which can
    move a point across a window boundary.  Measured on all 10 000 benchmark queries: 99.77 % of the
    result rows identical, recall unchanged.  That is below the 99.9 % the parity bar asks for, which is
    why the exact projection is the default; this test pins the measured level on 2 000 queries."""
    cfg, g, data_h, query_h, data = full
    from dciknn_cuda_b200 import DCI
    q = query_h.cuda()
    want, _ = g.query(q, cfg["k"], cfg["outer"], return_int_ids=True)
    t = DCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], 0, proj=g.get_proj())
    t.set_projection("tf32x3")
    t.add(data)
    got, _ = t.query(q, cfg["k"], cfg["outer"], return_int_ids=True)
    same = (got == want).all(1).float().mean().item()
    assert same >= 0.99, same
    truth = torch.cdist(q[:500], data).topk(cfg["k"], largest=False).indices
    rec = [(x[:500].long().unsqueeze(2) == truth.unsqueeze(1)).any(2).float().mean().item() for x in (want, got)]
    assert abs(rec[0] - rec[1]) < 0.005, rec
    t.free()
