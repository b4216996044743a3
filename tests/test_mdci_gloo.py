"""MDCI in one-process-per-GPU mode, exercised on CPU with two `gloo` ranks.

The rank-local engine and the merge are injected (the CUDA library cannot run
here), so what is checked is the host logic of dciknn_cuda_b200.MDCI: shard
bounds (reference core.py:122-125), the id stride between ranks (core.py:149),
the all-gather layout [D, nq, k] and that every rank ends with the merged lists
the reference's MDCI would produce (core.py:153-157)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _OracleEngine:
    """Rank-local stand-in with the DCI methods MDCI uses, backed by the CPU oracle."""

    def __init__(self, dim, L, S, P, T, proj):
        from oracle import oracle
        self.o = oracle.OracleDCI(dim, L, S, P, T, proj)

    def add(self, shard):
        self.o.add(shard.numpy())

    def query(self, q, k, outer, max_num_candidates=None, return_int_ids=True):
        ids, dists = self.o.query(q.numpy(), k, outer, max_num_candidates)
        return torch.from_numpy(ids), torch.from_numpy(dists)


class _PackedOracleEngine(_OracleEngine):
    """The same stand-in with DCI.query_packed: one int64 key (distance bits << 32 | id) per slot."""

    def query_packed(self, q, k, outer, max_num_candidates=None):
        nq = q.shape[0]
        out = np.full((nq, k), -1, np.int64)
        n = self.o.num_points
        if n > 0:
            ids, dists = self.o.query(q.numpy(), min(k, n), outer, max_num_candidates)
            key = (dists.view(np.uint32).astype(np.uint64) << np.uint64(32)) | ids.astype(np.uint32).astype(np.uint64)
            key[ids < 0] = np.uint64(0xFFFFFFFFFFFFFFFF)
            out[:, :ids.shape[1]] = key.view(np.int64)
        return torch.from_numpy(out)


def _host_merge_packed(packed, offsets, k):
    key = packed.numpy().view(np.uint64)
    empty = key == np.uint64(0xFFFFFFFFFFFFFFFF)
    ids = (key & np.uint64(0xFFFFFFFF)).astype(np.int64)
    dists = (key >> np.uint64(32)).astype(np.uint32).view(np.float32).copy()
    ids[empty] = -1
    dists[empty] = np.inf
    return _host_merge(torch.from_numpy(ids), torch.from_numpy(dists), offsets, k)


def _host_merge(ids, dists, offsets, k):
    ids = ids.numpy().astype(np.int64)
    for s, off in enumerate(offsets):
        ids[s][ids[s] >= 0] += off
    D, nq, _ = ids.shape
    ids = ids.transpose(1, 0, 2).reshape(nq, D * k)
    d = dists.numpy().transpose(1, 0, 2).reshape(nq, D * k)
    order = np.argsort(d, axis=1, kind="stable")[:, :k]
    return torch.from_numpy(np.take_along_axis(ids, order, 1)), torch.from_numpy(np.take_along_axis(d, order, 1))


def _worker(rank, world, port, out_dir, packed=False, n_points=1001):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dciknn_cuda_b200.core import MDCI, shard_bounds
    from tests import cases
    rng = np.random.default_rng(5)
    data = cases.latent_linear(rng, n_points, 12, 24)
    query = cases.latent_linear(rng, 17, 12, 24)
    projs = [cases.unit_rows(rng, 6, 24) for _ in range(world)]
    eng = (_PackedOracleEngine if packed else _OracleEngine)(24, 2, 3, 7, 5, projs[rank])
    m = MDCI(24, 2, 3, 7, 5, process_group=dist.group.WORLD, _local_engine=eng, _merge=_host_merge,
             _merge_packed=_host_merge_packed)
    m.add(torch.from_numpy(data))
    dpd, bounds = shard_bounds(n_points, world)
    assert m.data_per_device == dpd == n_points // world + 1 and eng.o.num_points == bounds[rank][1] - bounds[rank][0]
    ids, dists = m.query(torch.from_numpy(query), 6, 200, max_num_candidates=30, return_int_ids=True)
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), ids=ids.numpy(), dists=dists.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("packed", [False, True])
def test_two_gloo_ranks_match_reference_mdci_semantics(tmp_path, packed):
    """packed: the ranks exchange one tensor of 64-bit (distance, id) keys instead of two tensors."""
    from oracle import oracle
    from tests import cases
    world, port = 2, 29500 + (os.getpid() + 7 * packed) % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path), packed), nprocs=world, join=True)
    rng = np.random.default_rng(5)
    data = cases.latent_linear(rng, 1001, 12, 24)
    query = cases.latent_linear(rng, 17, 12, 24)
    projs = [cases.unit_rows(rng, 6, 24) for _ in range(world)]
    o = oracle.OracleMDCI(24, 2, 3, 7, 5, projs)
    o.add(data)
    oi, od = o.query(query, 6, 200, 30)
    for r in range(world):
        z = np.load(os.path.join(str(tmp_path), "rank%d.npz" % r))
        assert np.array_equal(z["ids"], oi) and np.array_equal(z["dists"], od)


def test_trailing_empty_shard_contributes_nothing(tmp_path):
    """6 points on 4 ranks: the reference's rule gives shards of 2, 2, 2 and 0 rows; the empty rank
    still takes part in the gather and the merged lists are those of the three real shards."""
    from oracle import oracle
    from tests import cases
    world, port = 4, 31500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path), True, 6), nprocs=world, join=True)
    rng = np.random.default_rng(5)
    data = cases.latent_linear(rng, 6, 12, 24)
    query = cases.latent_linear(rng, 17, 12, 24)
    projs = [cases.unit_rows(rng, 6, 24) for _ in range(world)]
    want_i, want_d = [], []
    for r in range(3):
        o = oracle.OracleDCI(24, 2, 3, 7, 5, projs[r])
        o.add(data[2 * r:2 * r + 2])
        a, d = o.query(query, 2, 200, 30)
        want_i.append(a.astype(np.int64) + 2 * r)
        want_d.append(d)
    want_i, want_d = np.concatenate(want_i, 1), np.concatenate(want_d, 1)
    order = np.argsort(want_d, axis=1, kind="stable")
    want_i, want_d = np.take_along_axis(want_i, order, 1), np.take_along_axis(want_d, order, 1)
    for r in range(world):
        z = np.load(os.path.join(str(tmp_path), "rank%d.npz" % r))
        assert np.array_equal(z["ids"], want_i) and np.array_equal(z["dists"], want_d)


def test_shard_bounds_follow_the_reference_rule():
    from dciknn_cuda_b200.core import shard_bounds
    assert shard_bounds(10, 3) == (4, [(0, 4), (4, 8), (8, 10)])
    assert shard_bounds(8, 8) == (2, [(0, 2), (2, 4), (4, 6), (6, 8), (8, 8), (8, 8), (8, 8), (8, 8)])
    dpd, b = shard_bounds(10_000_000, 8)
    assert dpd == 1_250_001 and b[-1] == (8_750_007, 10_000_000)
