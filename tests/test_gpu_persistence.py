"""Saving and reloading an index (not offered by the reference), and installing
the reference's own sorted index from the golden vectors."""
import glob
import os

import numpy as np
import pytest
import torch

from tests import cases

pytestmark = pytest.mark.gpu


def test_save_load_roundtrip(tmp_path):
    from dciknn_cuda_b200 import DCI
    c = cases.c2_shaped(n=20000, nq=40, P=2)
    data, q = torch.from_numpy(c["data"]).cuda(), torch.from_numpy(c["query"]).cuda()
    g = DCI(128, c["L"], c["S"], c["P"], c["T"], 0, seed=11)
    g.add(data)
    want = g.query(q, 10, return_int_ids=True)
    path = os.path.join(str(tmp_path), "index.npz")
    g.save(path)
    g.free()
    h = DCI.load(path, data)
    got = h.query(q, 10, return_int_ids=True)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    with pytest.raises(RuntimeError):
        h.set_index(data, *h.get_index())


def test_invalid_index_is_rejected():
    from dciknn_cuda_b200 import DCI
    rng = np.random.default_rng(0)
    data = torch.from_numpy(rng.standard_normal((500, 16)).astype(np.float32)).cuda()
    g = DCI(16, 2, 3, 5, 10, seed=3)
    g.add(data)
    keys, ids = g.get_index()
    g.clear()
    bad = keys.clone()
    bad[0, 10], bad[0, 11] = keys[0, 11] + 1.0, keys[0, 10] - 1.0      # not ascending any more
    with pytest.raises(ValueError):
        g.set_index(data, bad, ids)
    # a point named twice (and so another one never): ids stay inside the partition and keys stay
    # ascending, yet the segment is not a permutation and the point left out would have no position
    dup = ids.clone()
    dup[1, 7] = dup[1, 8]
    with pytest.raises(ValueError, match="twice"):
        g.set_index(data, keys, dup)
    assert g.num_points == 0
    with pytest.raises(RuntimeError):       # nothing is launched on a rejected index
        g.query(data[:2], 3)
    g.set_index(data, keys, ids)
    assert g.num_points == 500


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz"))),
                         ids=lambda p: os.path.basename(p)[:-4])
def test_traversal_on_the_references_own_index(path):
    """With the reference's sorted index installed (keys from its cuBLAS projection) the CUDA
    traversal returns the race-fixed reference's neighbours."""
    from dciknn_cuda_b200 import DCI
    z = np.load(path)
    L, S, P, T, k, outer, mc = [int(x) for x in z["params"]]
    data = torch.from_numpy(z["data"]).cuda()
    g = DCI(z["data"].shape[1], L, S, P, T, 0, proj=torch.from_numpy(z["proj"]))
    g.set_index(data, z["ref_keys"], z["ref_ids"])
    ids, dists = g.query(torch.from_numpy(z["query"]).cuda(), k, outer, max_num_candidates=mc, return_int_ids=True)
    assert (ids.cpu().numpy() == z["fixed_ids"]).all(1).mean() >= 0.999
    assert np.allclose(dists.cpu().numpy(), z["fixed_dists"], rtol=1e-6, atol=0)
