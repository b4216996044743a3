"""ctypes front end of oracle/dci_oracle.c (TEST INFRASTRUCTURE ONLY).

`OracleDCI` mirrors the reference's DCI class (dciknn_cuda/core.py:25-107) on
numpy arrays, with projection directions injected by the caller, and
`OracleMDCI` mirrors MDCI's sharding and merge (core.py:110-157).
"""
import ctypes as C
import os

import numpy as np

from .build import ORACLE_SO, build_oracle

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        _lib = C.CDLL(ORACLE_SO)
        fp, ip, ll = C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_longlong
        _lib.dci_oracle_project.argtypes = [fp, fp, ll, C.c_int, C.c_int, fp]
        _lib.dci_oracle_build.argtypes = [fp, C.c_int, C.c_int, C.c_int, fp, ip]
        _lib.dci_oracle_query.argtypes = [fp, ip, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                          fp, C.c_int, fp, fp, C.c_int, C.c_int, ll, C.c_int,
                                          ip, fp, C.POINTER(ll), C.POINTER(C.c_ubyte)]
        _lib.dci_oracle_query_blind.argtypes = [fp, ip, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                fp, C.c_int, C.c_int, ll, C.c_int, C.c_int, ip, C.POINTER(ll)]
        _lib.dci_oracle_bruteforce.argtypes = [fp, C.c_int, C.c_int, fp, C.c_int, C.c_int, ip, fp]
        _lib.dci_oracle_num_threads.restype = C.c_int
        _lib.dci_oracle_set_num_threads.argtypes = [C.c_int]
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def project(proj, x):
    """keys[i][p] = <proj[i], x[p]> with the oracle's fixed fp32 order."""
    proj, x = _f32(proj), _f32(x)
    out = np.empty((proj.shape[0], x.shape[0]), np.float32)
    rc = lib().dci_oracle_project(_p(proj, C.c_float), _p(x, C.c_float), x.shape[0], x.shape[1],
                                  proj.shape[0], _p(out, C.c_float))
    assert rc == 0
    return out


def build(keys_unsorted, P):
    keys_unsorted = _f32(keys_unsorted)
    I, N = keys_unsorted.shape
    skeys = np.empty((I, N), np.float32)
    sids = np.empty((I, N), np.int32)
    rc = lib().dci_oracle_build(_p(keys_unsorted, C.c_float), N, I, P, _p(skeys, C.c_float),
                                _p(sids, C.c_int))
    assert rc == 0
    return skeys, sids


def query_index(skeys, sids, L, S, P, T, data, qproj, query, k, outer, max_cand,
                want_stats=False, want_mask=False):
    """Run the traversal on an already built index with given projected queries
    (qproj is [I][nq])."""
    skeys, data, qproj, query = _f32(skeys), _f32(data), _f32(qproj), _f32(query)
    sids = np.ascontiguousarray(sids, dtype=np.int32)
    N, dim = data.shape
    nq = query.shape[0]
    assert skeys.shape == (L * S, N) and qproj.shape == (L * S, nq)
    ids = np.empty((nq, k), np.int32)
    dists = np.empty((nq, k), np.float32)
    stats = np.zeros((nq, P, 6), np.int64) if want_stats else None
    mask = np.zeros((nq, N), np.uint8) if want_mask else None
    rc = lib().dci_oracle_query(_p(skeys, C.c_float), _p(sids, C.c_int), N, L, S, P, T,
                                _p(data, C.c_float), dim, _p(qproj, C.c_float),
                                _p(query, C.c_float), nq, k, int(outer), int(max_cand),
                                _p(ids, C.c_int), _p(dists, C.c_float),
                                _p(stats, C.c_longlong) if want_stats else None,
                                _p(mask, C.c_ubyte) if want_mask else None)
    assert rc == 0
    out = [ids, dists]
    if want_stats:
        out.append(stats)
    if want_mask:
        out.append(mask)
    return tuple(out)


def query_index_blind(skeys, sids, L, S, P, T, qproj, k, outer, max_cand, width):
    """Blind traversal (no distances): ([nq, width] ids in retrieval order, [nq, width] iteration
    of promotion); unused slots hold -1."""
    skeys, qproj = _f32(skeys), _f32(qproj)
    sids = np.ascontiguousarray(sids, dtype=np.int32)
    N, nq = skeys.shape[1], qproj.shape[1]
    ids = np.empty((nq, width), np.int32)
    when = np.empty((nq, width), np.int64)
    rc = lib().dci_oracle_query_blind(_p(skeys, C.c_float), _p(sids, C.c_int), N, L, S, P, T,
                                      _p(qproj, C.c_float), nq, k, int(outer), int(max_cand), int(width),
                                      _p(ids, C.c_int), _p(when, C.c_longlong))
    assert rc == 0
    return ids, when


def bruteforce(data, query, k):
    data, query = _f32(data), _f32(query)
    ids = np.empty((query.shape[0], k), np.int32)
    dists = np.empty((query.shape[0], k), np.float32)
    rc = lib().dci_oracle_bruteforce(_p(data, C.c_float), data.shape[0], data.shape[1],
                                     _p(query, C.c_float), query.shape[0], k,
                                     _p(ids, C.c_int), _p(dists, C.c_float))
    assert rc == 0
    return ids, dists


class OracleDCI:
    """numpy mirror of dciknn_cuda.DCI (core.py:25-107) with injected directions."""

    def __init__(self, dim, num_comp_indices=2, num_simp_indices=7, bs=100, ts=10, proj=None):
        self.dim, self.L, self.S, self.P, self.T = dim, num_comp_indices, num_simp_indices, bs, ts
        self.proj = None if proj is None else _f32(proj).reshape(self.L * self.S, dim)
        self.num_points = 0

    def add(self, data):
        if self.num_points > 0:
            raise RuntimeError("DCI class does not support insertion of more than one tensor.")
        self.data = _f32(data)
        self.num_points = self.data.shape[0]
        self.skeys, self.sids = build(project(self.proj, self.data), self.P)

    def query(self, query, num_neighbours=-1, num_outer_iterations=5000, max_num_candidates=None,
              want_stats=False, want_mask=False):
        query = _f32(query).reshape(-1, self.dim)
        k = self.num_points if num_neighbours < 0 else num_neighbours
        mc = 10 * k if max_num_candidates is None else max_num_candidates   # core.py:87
        qproj = project(self.proj, query)
        return query_index(self.skeys, self.sids, self.L, self.S, self.P, self.T, self.data,
                           qproj, query, k, num_outer_iterations, mc, want_stats, want_mask)

    def query_blind(self, query, num_neighbours=-1, num_outer_iterations=5000, max_num_candidates=None):
        """Promoted point ids in retrieval order and their promotion iterations, each
        [nq, min(max_num_candidates, num_outer_iterations)] (dci_cuda_kernel.cu:775-776, :784-785)."""
        query = _f32(query).reshape(-1, self.dim)
        k = self.num_points if num_neighbours < 0 else num_neighbours
        mc = 10 * k if max_num_candidates is None else max_num_candidates
        width = min(mc, num_outer_iterations)
        return query_index_blind(self.skeys, self.sids, self.L, self.S, self.P, self.T,
                                 project(self.proj, query), k, num_outer_iterations, mc, width)


class OracleMDCI:
    """numpy mirror of dciknn_cuda.MDCI (core.py:110-157): shard i holds rows
    [i*dpd, (i+1)*dpd), dpd = N // D + 1; every shard answers every query; the
    merged list is the k smallest of the concatenated per-shard lists, stable in
    shard order."""

    def __init__(self, dim, num_comp_indices=2, num_simp_indices=7, bs=100, ts=10, projs=()):
        self.shards = [OracleDCI(dim, num_comp_indices, num_simp_indices, bs, ts, p) for p in projs]
        self.data_per_device = 0

    def add(self, data):
        D = len(self.shards)
        self.data_per_device = data.shape[0] // D + 1
        for i, s in enumerate(self.shards):
            s.add(data[i * self.data_per_device:(i + 1) * self.data_per_device])

    def query(self, query, num_neighbours, num_outer_iterations=5000, max_num_candidates=None):
        ids, dists = [], []
        for i, s in enumerate(self.shards):
            a, d = s.query(query, num_neighbours, num_outer_iterations, max_num_candidates)
            a = a.astype(np.int64)
            a[a >= 0] += self.data_per_device * i
            ids.append(a)
            dists.append(d)
        ids, dists = np.concatenate(ids, 1), np.concatenate(dists, 1)
        order = np.argsort(dists, axis=1, kind="stable")[:, :num_neighbours]
        return np.take_along_axis(ids, order, 1), np.take_along_axis(dists, order, 1)
