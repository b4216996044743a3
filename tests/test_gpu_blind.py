"""Blind querying on the device against the sequential restatement: same ids in the same
order, same promotion iterations, no distance computed."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


def _both(c):
    from dciknn_cuda_b200 import DCI
    g = DCI(c["data"].shape[1], c["L"], c["S"], c["P"], c["T"], 0, proj=torch.from_numpy(c["proj"]))
    g.add(torch.from_numpy(c["data"]).cuda())
    ids, iters = g.query(torch.from_numpy(c["query"]).cuda(), c["k"], c["outer"], blind=True,
                         max_num_candidates=c.get("max_cand"), return_int_ids=True)
    o = oracle.OracleDCI(c["data"].shape[1], c["L"], c["S"], c["P"], c["T"], c["proj"])
    o.add(c["data"])
    oi, ow = o.query_blind(c["query"], c["k"], c["outer"], c.get("max_cand"))
    return g, ids.cpu().numpy(), iters.cpu().numpy(), oi, ow


@pytest.mark.parametrize("row", [r for r in cases.EDGE_CASES if min(r[8], r[9]) > 0], ids=lambda r: r[0])
def test_blind_edge_cases_match_the_oracle(row):
    c = cases.edge_case(row)
    g, ids, iters, oi, ow = _both(c)
    assert ids.dtype == np.int32 and ids.shape == oi.shape
    assert np.array_equal(ids, oi)
    assert np.array_equal(iters.astype(np.int64), ow)
    g.free()


def test_blind_example_and_large_partition_configurations():
    for c in (cases.example_config(nq=40), cases.c2_shaped(n=30000, nq=24)):
        g, ids, iters, oi, ow = _both(c)
        assert np.array_equal(ids, oi) and np.array_equal(iters.astype(np.int64), ow)
        # the regular query afterwards is unaffected by the blind one
        q = torch.from_numpy(c["query"]).cuda()
        a, d = g.query(q, c["k"], c["outer"], return_int_ids=True)
        o = oracle.OracleDCI(c["data"].shape[1], c["L"], c["S"], c["P"], c["T"], c["proj"])
        o.add(c["data"])
        ei, ed = o.query(c["query"], c["k"], c["outer"])
        assert np.array_equal(a.cpu().numpy(), ei)
        assert np.array_equal(d.cpu().numpy().view(np.uint32), ed.view(np.uint32))
        g.free()


def test_blind_default_return_types_and_width():
    from dciknn_cuda_b200 import DCI
    g = DCI(16, 2, 3, 4, 10, seed=4)
    x = torch.randn(400, 16, device="cuda")
    g.add(x)
    ids, iters = g.query(x[:5], 3, 7, blind=True)                 # width = min(7, 10 * 3)
    assert ids.dtype == torch.float32 and iters.dtype == torch.int32 and ids.shape == iters.shape == (5, 7)
    with pytest.raises(ValueError):
        g.query(x[:5], 3, 7, blind=True, max_num_candidates=0)
    g.free()
