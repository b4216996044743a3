"""The CUDA library against the golden vectors of the reference's CUDA build:
with the reference's directions injected, the neighbour ids must equal the
race-fixed reference's for every query and distances agree to 1e-5 relative
(they are in fact bit-identical on these cases)."""
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
FILES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f)[:-4] for f in FILES])
def test_matches_race_fixed_reference(path):
    from dciknn_cuda_b200 import DCI
    z = np.load(path)
    L, S, P, T, k, outer, mc = [int(x) for x in z["params"]]
    g = DCI(z["data"].shape[1], L, S, P, T, 0, proj=torch.from_numpy(z["proj"]))
    g.add(torch.from_numpy(z["data"]).cuda())
    ids, dists = g.query(torch.from_numpy(z["query"]).cuda(), k, outer, max_num_candidates=mc, return_int_ids=True)
    ids, dists = ids.cpu().numpy(), dists.cpu().numpy()
    match = (ids == z["fixed_ids"]).all(1).mean()
    assert match >= 0.999, "id lists match the reference on %.2f%% of queries" % (100 * match)
    assert np.allclose(dists, z["fixed_dists"], rtol=1e-5, atol=0)
    assert (dists <= z["asis_dists"] * (1 + 1e-5)).all()      # dominance over the racy build
    _, gi = g.get_index()
    assert np.array_equal(gi.numpy(), z["ref_ids"])
