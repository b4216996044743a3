"""The PyTorch-extension shim (dciknn_cuda_b200/_dci_b200.so): the seven entry points of the
reference's extension module (src/dci_cuda.cpp:175-183), driven with the calling sequence of the
reference's Python layer (dciknn_cuda/core.py:32-39, 69-75, 78-92, 143-157)."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


def _mod():
    from dciknn_cuda_b200.build import build_torch_shim
    build_torch_shim()
    from dciknn_cuda_b200 import _dci_b200
    return _dci_b200


def test_reference_call_sequence_matches_the_oracle():
    m = _mod()
    c = cases.example_config(n=2000, nq=64)
    dim, L, S, bs, ts, k = 100, c["L"], c["S"], c["P"], c["T"], c["k"]
    inst = m._dci_new(dim, L, S, 0)                                    # core.py:36
    m._dci_set_proj(inst, torch.from_numpy(c["proj"]))
    data = torch.from_numpy(c["data"]).cuda()
    m._dci_add(inst, dim, data.shape[0], data.flatten(), bs, ts)       # core.py:73
    q = torch.from_numpy(c["query"]).cuda()
    res = m._dci_query(inst, dim, q.shape[0], q.flatten(), k, False, 5000, 10 * k, bs, ts)   # core.py:88-89
    assert res.dtype == torch.float32 and res.shape == (2 * 64 * k,) and res.is_cuda
    half = res.shape[0] // 2                                            # core.py:90-92
    ids, dists = res[:half].reshape(64, -1), res[half:].reshape(64, -1)
    o = oracle.OracleDCI(dim, L, S, bs, ts, c["proj"])
    o.add(c["data"])
    oi, od = o.query(c["query"], k, 5000)
    assert np.array_equal(ids.cpu().numpy().astype(np.int32), oi)
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32))
    with pytest.raises(RuntimeError):
        m._dci_add(inst, dim, data.shape[0], data.flatten(), bs, ts)   # a second add is refused
    m._dci_clear(inst)
    m._dci_add(inst, dim, data.shape[0], data.flatten(), bs, ts)       # ... and allowed after clear
    m._dci_reset(inst)                                                  # new directions, empty index
    assert not torch.equal(m._dci_get_proj(inst, L * S, dim), torch.from_numpy(c["proj"]))
    with pytest.raises(RuntimeError):
        m._dci_query(inst, dim, 1, q[:1].flatten(), k, False, 5000, 10 * k, bs, ts)
    m._dci_free(inst)
    m._dci_free(inst)                                                   # harmless
    with pytest.raises(RuntimeError):
        m._dci_clear(inst)


def test_multi_query_fans_out_like_the_reference():
    """_dci_multi_query with two instances (both on device 0 here), then the reference's merge
    (core.py:146-157) with torch, against the sequential restatement of MDCI."""
    m = _mod()
    rng = np.random.default_rng(3)
    data = cases.latent_linear(rng, 2001, 16, 32)
    query = cases.latent_linear(rng, 20, 16, 32)
    projs = [cases.unit_rows(rng, 6, 32) for _ in range(2)]
    dpd = 2001 // 2 + 1
    insts, keep = [], []
    for i in range(2):
        inst = m._dci_new(32, 2, 3, 0)
        m._dci_set_proj(inst, torch.from_numpy(projs[i]))
        shard = torch.from_numpy(data[i * dpd:(i + 1) * dpd]).cuda()
        m._dci_add(inst, 32, shard.shape[0], shard.flatten(), 7, 5)
        insts.append(inst); keep.append(shard)
    q = torch.from_numpy(query).cuda()
    res = m._dci_multi_query(insts, 32, 20, [q.flatten(), q.flatten()], 6, False, 200, 30, 7, 5)
    ids, dists = [], []
    for i, r in enumerate(res):
        half = r.shape[0] // 2
        ids.append(r[:half].reshape(20, -1) + dpd * i)
        dists.append(r[half:].reshape(20, -1))
    ids, dists = torch.cat(ids, 1), torch.cat(dists, 1)
    order = torch.sort(dists, dim=1, stable=True).indices[:, :6]
    o = oracle.OracleMDCI(32, 2, 3, 7, 5, projs)
    o.add(data)
    oi, od = o.query(query, 6, 200, 30)
    assert np.array_equal(ids.gather(1, order).cpu().numpy().astype(np.int64), oi)
    assert np.array_equal(dists.gather(1, order).cpu().numpy().view(np.uint32), od.view(np.uint32))
