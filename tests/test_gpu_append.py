"""Incremental add: append() must leave exactly the index a fresh add() of all rows builds."""
import numpy as np
import pytest
import torch

import cases
from dciknn_cuda_b200 import DCI
from oracle import oracle

pytestmark = pytest.mark.gpu


def _fresh(dim, L, S, P, T, proj, rows):
    d = DCI(dim, L, S, P, T, proj=torch.from_numpy(proj))
    d.add(torch.from_numpy(rows).cuda())
    return d


@pytest.mark.parametrize("n0,adds,P,T", [(3000, (1, 999, 2500), 7, 10), (500, (70000,), 1, 10), (2000, (13,), 100, 3)])
def test_append_equals_fresh_add_of_the_concatenation(n0, adds, P, T):
    rng = np.random.default_rng(77)
    dim, L, S = 24, 2, 5
    total = n0 + sum(adds)
    rows = cases.latent_linear(rng, total, 6, dim, 0.01)
    query = cases.latent_linear(rng, 33, 6, dim, 0.01)
    proj = cases.unit_rows(rng, L * S, dim)
    d = _fresh(dim, L, S, P, T, proj, rows[:n0])
    n = n0
    for a in adds:
        d.append(torch.from_numpy(rows[n:n + a]).cuda())
        n += a
        assert d.num_points == n
        f = _fresh(dim, L, S, P, T, proj, rows[:n])
        kd, idd = d.get_index()
        kf, idf = f.get_index()
        assert np.array_equal(np.asarray(idd), np.asarray(idf))
        assert np.array_equal(np.asarray(kd).view(np.uint32), np.asarray(kf).view(np.uint32))
        f.free()
    q = torch.from_numpy(query).cuda()
    ids, dists = d.query(q, 10, return_int_ids=True)
    o = oracle.OracleDCI(dim, L, S, P, T, proj)
    o.add(rows)
    oi, od = o.query(query, 10)
    assert np.array_equal(ids.cpu().numpy(), oi)
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32))
    d.free()


def test_append_argument_and_state_errors():
    d = DCI(8, 1, 3, 4, 10, seed=3)
    x = torch.randn(100, 8, device="cuda")
    with pytest.raises(RuntimeError):
        d.append(x)                               # nothing indexed yet
    d.add(x)
    with pytest.raises(ValueError):
        d.append(torch.randn(5, 9, device="cuda"))
    with pytest.raises(TypeError):
        d.append(torch.randn(5, 8))
    d.append(torch.empty(0, 8, device="cuda"))    # no-op
    assert d.num_points == 100
    d.append(torch.randn(5, 8, device="cuda"))
    assert d.num_points == 105
    d.clear()
    assert d.num_points == 0
    d.add(x)                                      # usable again after clear
    assert d.num_points == 100
    d.free()
