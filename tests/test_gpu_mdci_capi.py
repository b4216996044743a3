"""The sharded engine through the C ABI alone (dci_b200_mdci_*): what a C or C++ host calls in place
of the reference's MDCI class and _dci_multi_query (dciknn_cuda/core.py:110-157,
src/dci_cuda.cpp:120-134).  Checked against the sequential restatement of MDCI."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


def _run(devices, n_points, k, nq=33, dim=48, L=2, S=5, P=20, T=10, seed=11):
    from dciknn_cuda_b200 import _capi
    lib = _capi.lib()
    D = len(devices)
    rng = np.random.default_rng(seed)
    data = cases.latent_linear(rng, n_points, 20, dim)
    query = cases.latent_linear(rng, nq, 20, dim)
    projs = [cases.unit_rows(rng, L * S, dim) for _ in range(D)]
    m = C.c_void_p()
    devs = (C.c_int * D)(*devices)
    _capi.check(lib.dci_b200_mdci_create(C.byref(m), dim, L, S, devs, D, None))
    try:
        assert lib.dci_b200_mdci_num_devices(m) == D
        for i in range(D):
            _capi.check(lib.dci_b200_set_proj(C.c_void_p(lib.dci_b200_mdci_shard(m, i)),
                                              projs[i].ctypes.data_as(C.c_void_p)))
        _capi.check(lib.dci_b200_mdci_add(m, data.ctypes.data_as(C.c_void_p), n_points, P, T))
        assert lib.dci_b200_mdci_data_per_device(m) == n_points // D + 1
        assert lib.dci_b200_mdci_add(m, data.ctypes.data_as(C.c_void_p), n_points, P, T) == _capi.ERR_STATE
        ids = np.empty((nq, k), np.int64)
        dists = np.empty((nq, k), np.float32)
        for _ in range(2):      # the second call reuses every buffer
            ids[:] = -5
            _capi.check(lib.dci_b200_mdci_query_host(m, query.ctypes.data_as(C.c_void_p), nq, k, 5000, 10 * k,
                                                     ids.ctypes.data_as(C.c_void_p), dists.ctypes.data_as(C.c_void_p)))
        # device buffers on devices[0], caller's stream
        dev0 = torch.device("cuda", devices[0])
        with torch.cuda.device(dev0):
            q = torch.from_numpy(query).to(dev0)
            d_ids = torch.empty((nq, k), dtype=torch.int64, device=dev0)
            d_dists = torch.empty((nq, k), dtype=torch.float32, device=dev0)
            st = torch.cuda.Stream(dev0)
            st.wait_stream(torch.cuda.current_stream(dev0))
            _capi.check(lib.dci_b200_mdci_query(m, C.c_void_p(q.data_ptr()), nq, k, 5000, 10 * k,
                                                C.c_void_p(d_ids.data_ptr()), C.c_void_p(d_dists.data_ptr()),
                                                C.c_void_p(st.cuda_stream)))
            st.synchronize()
        assert np.array_equal(d_ids.cpu().numpy(), ids) and np.array_equal(d_dists.cpu().numpy(), dists)
        assert lib.dci_b200_mdci_query_host(m, query.ctypes.data_as(C.c_void_p), nq, 0, 5000, 10,
                                            ids.ctypes.data_as(C.c_void_p), dists.ctypes.data_as(C.c_void_p)) == _capi.ERR_ARG
        _capi.check(lib.dci_b200_mdci_clear(m))
        _capi.check(lib.dci_b200_mdci_add(m, data.ctypes.data_as(C.c_void_p), n_points, P, T))   # add / query / clear cycles
    finally:
        lib.dci_b200_mdci_destroy(m)
    return data, query, projs, ids, dists


def test_three_shards_on_one_device_match_the_sequential_mdci():
    data, query, projs, ids, dists = _run([0, 0, 0], 3001, 10)
    o = oracle.OracleMDCI(48, 2, 5, 20, 10, projs)
    o.add(data)
    oi, od = o.query(query, 10)
    assert np.array_equal(ids, oi)
    assert np.array_equal(dists.view(np.uint32), od.view(np.uint32))


def test_short_and_empty_shards():
    """9 points on 4 shards (3 + 3 + 3 + 0) with k = 9: every shard answers with the 3 points it has."""
    data, query, projs, ids, dists = _run([0, 0, 0, 0], 9, 9, nq=5, dim=8, L=1, S=2, P=2, T=3, seed=13)
    bi, bd = oracle.bruteforce(data, query, 9)
    assert np.array_equal(dists.view(np.uint32), bd.view(np.uint32))
    assert np.array_equal(np.sort(ids, 1), np.sort(bi.astype(np.int64), 1))


def test_two_devices_match_the_sequential_mdci():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    data, query, projs, ids, dists = _run([0, 1], 20001, 10, nq=50, dim=64)
    o = oracle.OracleMDCI(64, 2, 5, 20, 10, projs)
    o.add(data)
    oi, od = o.query(query, 10)
    assert np.array_equal(ids, oi)
    assert np.array_equal(dists.view(np.uint32), od.view(np.uint32))
