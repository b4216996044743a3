"""Shard merge for result lists longer than the selection buffers (k > 1024)."""
import numpy as np
import pytest
import torch

import cases
from dciknn_cuda_b200 import DCI, merge_shards, shard_bounds
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k", [1025, 1500, 2600])
def test_merge_of_long_shard_lists_matches_the_sequential_mdci(k):
    rng = np.random.default_rng(123)
    D, dim, L, S, P, T = 3, 16, 2, 4, 2, 10
    data = cases.latent_linear(rng, 7000, 6, dim, 0.01)
    query = cases.latent_linear(rng, 9, 6, dim, 0.01)
    projs = [cases.unit_rows(rng, L * S, dim) for _ in range(D)]
    dpd, bounds = shard_bounds(data.shape[0], D)
    q = torch.from_numpy(query).cuda()
    ids, dists, keep = [], [], []
    for s, (lo, hi) in enumerate(bounds):
        d = DCI(dim, L, S, P, T, proj=torch.from_numpy(projs[s]))
        d.add(torch.from_numpy(data[lo:hi]).cuda())
        # a shard holds fewer than k points: its list ends with empty slots
        i, dd = d.query(q, min(k, hi - lo), return_int_ids=True)
        pad_i = torch.full((len(query), k), -1, dtype=torch.int32, device="cuda")
        pad_d = torch.full((len(query), k), float("inf"), dtype=torch.float32, device="cuda")
        pad_i[:, :i.shape[1]] = i
        pad_d[:, :i.shape[1]] = dd
        ids.append(pad_i); dists.append(pad_d); keep.append(d)
    gi, gd = merge_shards(torch.stack(ids).contiguous(), torch.stack(dists).contiguous(),
                          [s * dpd for s in range(D)], k)
    # the reference's merge (dciknn_cuda/core.py:146-157) on the sequential restatement's lists
    ei, ed = [], []
    for s, (lo, hi) in enumerate(bounds):
        o = oracle.OracleDCI(dim, L, S, P, T, projs[s])
        o.add(data[lo:hi])
        a, dd = o.query(query, min(k, hi - lo))
        a = a.astype(np.int64)
        a[a >= 0] += dpd * s
        pi = np.full((len(query), k), -1, dtype=np.int64)
        pd = np.full((len(query), k), np.inf, dtype=np.float32)
        pi[:, :a.shape[1]] = a
        pd[:, :a.shape[1]] = dd
        ei.append(pi); ed.append(pd)
    ei, ed = np.concatenate(ei, 1), np.concatenate(ed, 1)
    order = np.argsort(ed, axis=1, kind="stable")[:, :k]
    oi, od = np.take_along_axis(ei, order, 1), np.take_along_axis(ed, order, 1)
    assert np.array_equal(gi.cpu().numpy(), oi)
    assert np.array_equal(gd.cpu().numpy().view(np.uint32), od.view(np.uint32))
    for d in keep:
        d.free()
