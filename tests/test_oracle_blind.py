"""Blind traversal of the sequential restatement: the listed ids are promoted points, in
ascending (promotion iteration, id), and agree with the regular query's promoted set."""
import numpy as np
import pytest

from oracle import oracle
from tests import cases


@pytest.mark.parametrize("row", [r for r in cases.EDGE_CASES if min(r[8], r[9]) > 0], ids=lambda r: r[0])
def test_blind_list_is_the_promoted_set_in_retrieval_order(row):
    c = cases.edge_case(row)
    o = oracle.OracleDCI(c["data"].shape[1], c["L"], c["S"], c["P"], c["T"], c["proj"])
    o.add(c["data"])
    ids, when = o.query_blind(c["query"], c["k"], c["outer"], c["max_cand"])
    _, _, stats, mask = o.query(c["query"], c["k"], c["outer"], c["max_cand"], want_stats=True, want_mask=True)
    width = min(c["outer"], c["max_cand"])
    assert ids.shape == when.shape == (c["query"].shape[0], width)
    ppb = -(-c["data"].shape[0] // c["P"])
    for q in range(ids.shape[0]):
        live = ids[q] >= 0
        nlive = int(live.sum())
        assert live[:nlive].all() and (when[q][~live] == -1).all()          # unused slots at the end
        assert nlive == min(width, int(mask[q].sum()))
        assert mask[q][ids[q][live]].all() and len(set(ids[q][live])) == nlive
        order = list(zip(when[q][live], ids[q][live]))
        assert order == sorted(order)
        # a point is promoted no later than its partition's loop ended
        assert (when[q][live] <= stats[q, ids[q][live] // ppb, 0]).all()
        if nlive < int(mask[q].sum()):                                       # truncated: nothing left out is earlier
            assert nlive == width
