"""The optional tensor-core projection (tcgen05.mma, 3xTF32) against the exact
fp32 projection: keys agree to about 1e-6 of |x| (the directions are unit
vectors), far tighter than plain tf32 (1e-3), and a query answered with
tensor-core keys returns the same neighbours for nearly every query."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["tf32x3", "tf32x3_plain", "tf32x3_tile"])
@pytest.mark.parametrize("n,dim,L,S", [(1000, 128, 2, 10), (777, 100, 2, 7), (300, 37, 3, 12), (5000, 960, 3, 12), (129, 8, 1, 1), (40000, 64, 2, 10)])
def test_tensor_core_keys_match_exact_keys(n, dim, L, S, mode):
    from dciknn_cuda_b200 import DCI
    rng = np.random.default_rng(n + dim)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    proj = cases.unit_rows(rng, L * S, dim)
    g = DCI(dim, L, S, proj=torch.from_numpy(proj))
    g.set_projection(mode)
    got = g.project(torch.from_numpy(x).cuda()).cpu().numpy()
    want = oracle.project(proj, x)
    scale = np.linalg.norm(x, axis=1)[None, :]
    err = np.abs(got - want) / scale
    assert err.max() < 4e-6, err.max()
    ref64 = proj.astype(np.float64) @ x.astype(np.float64).T
    assert (np.abs(got - ref64) / scale).max() < 4e-6


def test_query_with_tensor_core_keys():
    from dciknn_cuda_b200 import DCI
    c = cases.c2_shaped(n=40000, nq=200, P=4)
    data, query = torch.from_numpy(c["data"]).cuda(), torch.from_numpy(c["query"]).cuda()
    res = {}
    for mode in ("exact", "tf32x3"):
        g = DCI(128, c["L"], c["S"], c["P"], c["T"], 0, proj=torch.from_numpy(c["proj"]))
        g.set_projection(mode)
        g.add(data)
        with pytest.raises(RuntimeError):
            g.set_projection("exact")
        res[mode] = g.query(query, 10, return_int_ids=True)
    same = (res["exact"][0] == res["tf32x3"][0]).all(1).float().mean().item()
    assert same >= 0.98, same        # 0.9977 of 10 000 queries at the benchmark's full size (tests/test_gpu_fullsize.py)
