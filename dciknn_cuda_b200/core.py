"""DCI / MDCI: the reference's Python operator surface on the B200-native engine.

Mirrors dciknn_cuda/core.py of the reference (DCI: lines 25-107, MDCI: lines
110-169): same constructor arguments, same methods (add, query, clear, reset,
free), same argument checks and exception types, same return convention (a
pair of [num_queries, k] float32 CUDA tensors: neighbour ids, then Euclidean
distances, rows ascending by distance).  Everything below this file is the C
ABI of include/dci_b200.h; torch only supplies device memory and streams.

Extras, all keyword-only and defaulting to the reference's behaviour:
  seed / proj           choose or inject the projection directions (the reference
                        draws them from the process-global rand(), util_kernel.cu:124-127)
  max_num_candidates    the reference hard-codes 10 * num_neighbours (core.py:87, :141)
  MDCI(process_group=)  one process per GPU over torch.distributed instead of one
                        process driving every device
"""
import ctypes as C
import itertools
import os

import torch

from . import _capi

_seed_counter = itertools.count(1)


def _default_seed():
    # a fresh stream of directions per instance, like the reference, where every
    # _dci_new advances rand(); deterministic per process unless DCI_B200_SEED moves it
    base = int(os.environ.get("DCI_B200_SEED", "0"))
    z = (base * 0x9E3779B97F4A7C15 + next(_seed_counter) * 0xBF58476D1CE4E5B9 + 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def _device_index(device):
    if isinstance(device, torch.device):
        if device.type != "cuda":
            raise TypeError("device must be a cuda device")
        return torch.cuda.current_device() if device.index is None else device.index
    if isinstance(device, str):
        return _device_index(torch.device(device))
    return int(device)


def _stream_ptr(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


class DCI(object):
    """Prioritized DCI on one GPU (reference: dciknn_cuda/core.py:25-107)."""

    def __init__(self, dim, num_comp_indices=2, num_simp_indices=7, bs=100, ts=10, device=0, *,
                 seed=None, proj=None):
        if not torch.cuda.is_available():
            raise RuntimeError("DCI CUDA version requires GPU access, please check CUDA driver.")
        self._dim = dim
        self._num_comp_indices = num_comp_indices
        self._num_simp_indices = num_simp_indices
        self._block_size = bs
        self._thread_size = ts
        self._device = _device_index(device)
        self._array = None
        self._store = None
        self.num_points = 0
        self._handle = C.c_void_p()
        lib = _capi.lib()
        _capi.check(lib.dci_b200_create(C.byref(self._handle), dim, num_comp_indices, num_simp_indices,
                                        self._device, _default_seed() if seed is None else int(seed)))
        if proj is not None:
            self.set_proj(proj)

    # -- properties of the reference class (core.py:41-51)
    @property
    def dim(self):
        return self._dim

    @property
    def num_comp_indices(self):
        return self._num_comp_indices

    @property
    def num_simp_indices(self):
        return self._num_simp_indices

    @property
    def device(self):
        return torch.device("cuda", self._device)

    def _ensure_positive_integer(self, x):
        if not isinstance(x, int):
            raise TypeError("number must be an integer")
        elif x <= 0:
            raise ValueError("number must be positive")

    def _check_data(self, arr):
        # same checks, order and exception types as core.py:59-67
        if arr.shape[1] != self.dim:
            raise ValueError("mismatch between tensor dimension (%d) and the declared dimension of this DCI instance (%d)" % (arr.shape[1], self.dim))
        if arr.dtype != torch.float:
            raise TypeError("tensor must consist of single-precision floats")
        if not arr.is_contiguous():
            raise ValueError("the memory layout of tensor must be in row-major (C-order)")
        if not arr.is_cuda:
            raise TypeError("tensor must be a cuda tensor")
        if arr.device.index != self._device:
            raise ValueError("tensor lives on %s but this DCI instance was created on cuda:%d" % (arr.device, self._device))

    def _live(self):
        if not self._handle:
            raise RuntimeError("this DCI instance has been freed")
        return self._handle

    # -- directions (no counterpart in the reference's Python API)
    def get_proj(self):
        """The L*S unit directions as a [L*S, dim] float32 CPU tensor (row h + m*S)."""
        out = torch.empty(self._num_comp_indices * self._num_simp_indices, self._dim, dtype=torch.float32)
        _capi.check(_capi.lib().dci_b200_get_proj(self._live(), C.c_void_p(out.data_ptr())))
        return out

    def set_proj(self, proj):
        proj = torch.as_tensor(proj, dtype=torch.float32).cpu().contiguous()
        if tuple(proj.shape) != (self._num_comp_indices * self._num_simp_indices, self._dim):
            raise ValueError("proj must have shape [num_comp_indices * num_simp_indices, dim]")
        rc = _capi.lib().dci_b200_set_proj(self._live(), C.c_void_p(proj.data_ptr()))
        if rc == _capi.ERR_STATE:
            raise RuntimeError(_capi.lib().dci_b200_last_error().decode())
        _capi.check(rc)

    # -- reference methods
    def add(self, data):
        if self.num_points > 0:
            raise RuntimeError("DCI class does not support insertion of more than one tensor. Must combine all tensors into one tensor before inserting")
        self._check_data(data)
        if data.shape[0] == 0:
            raise ValueError("cannot add an empty tensor")
        with torch.cuda.device(self._device):
            _capi.check(_capi.lib().dci_b200_add(self._live(), C.c_void_p(data.data_ptr()), data.shape[0],
                                                self._block_size, self._thread_size, _stream_ptr(self._device)))
        self.num_points = data.shape[0]
        self._array = data          # the index borrows the tensor's memory
        self._store = None

    def append(self, data):
        """Adds more rows to a non-empty index (the reference has no such call: its add refuses a
        second tensor, dciknn_cuda/core.py:70-71).  The result equals clear() followed by add() of the
        concatenation of everything added so far, but only the new rows are projected.  The index
        keeps its own copy of the rows from the first append on (capacity grows geometrically), since
        the rows must be contiguous."""
        if self.num_points == 0:
            raise RuntimeError("append needs a non-empty index; use add first")
        self._check_data(data)
        if data.device.index != self._device:
            raise ValueError("data must be on the index's device")
        n_old, n_add = self.num_points, data.shape[0]
        if n_add == 0:
            return
        n_new = n_old + n_add
        with torch.cuda.device(self._device):
            store = self._store
            if store is None or store.shape[0] < n_new:
                store = torch.empty((max(n_new, n_old + n_old // 2), self._dim), dtype=torch.float32, device=data.device)
                store[:n_old].copy_(self._array[:n_old])
            store[n_old:n_new].copy_(data)
            try:
                _capi.check(_capi.lib().dci_b200_append(self._live(), C.c_void_p(store.data_ptr()), n_new,
                                                       _stream_ptr(self._device)))
            except Exception:
                # a failed append may have emptied the handle: follow it instead of keeping stale counts
                self.num_points = int(_capi.lib().dci_b200_num_points(self._live()))
                if self.num_points == 0:
                    self._array = None
                    self._store = None
                raise
        self._store = store
        self._array = store[:n_new]
        self.num_points = n_new

    def query(self, query, num_neighbours=-1, num_outer_iterations=5000, blind=False, *,
              max_num_candidates=None, return_int_ids=False):
        """query is [num_queries, dim] (or [dim]); returns ([num_queries, k] ids, [num_queries, k] distances)."""
        if len(query.shape) < 2:
            _query = query.unsqueeze(0)
        else:
            _query = query
        self._check_data(_query)
        if num_neighbours < 0:
            num_neighbours = self.num_points
        self._ensure_positive_integer(num_neighbours)
        if max_num_candidates is None:
            max_num_candidates = 10 * num_neighbours
        if self.num_points == 0:
            raise RuntimeError("the index is empty; add data first")
        nq = _query.shape[0]
        if blind:
            # Candidates in order of retrieval, no distances (reference dci_cuda_kernel.cu:398-399, :775-776);
            # returns ([nq, width] ids, [nq, width] promotion iterations), -1 in unused slots.
            width = _capi.lib().dci_b200_blind_width(int(num_outer_iterations), int(max_num_candidates))
            with torch.cuda.device(self._device):
                ids = torch.empty((nq, width), dtype=torch.int32, device=_query.device)
                iters = torch.empty((nq, width), dtype=torch.int32, device=_query.device)
                _capi.check(_capi.lib().dci_b200_query_blind(
                    self._live(), C.c_void_p(_query.data_ptr()), nq, num_neighbours, int(num_outer_iterations),
                    int(max_num_candidates), self._block_size, self._thread_size,
                    C.c_void_p(ids.data_ptr()), C.c_void_p(iters.data_ptr()), _stream_ptr(self._device)))
            return (ids, iters) if return_int_ids else (ids.to(torch.float32), iters)
        with torch.cuda.device(self._device):
            ids = torch.empty((nq, num_neighbours), dtype=torch.int32, device=_query.device)
            dists = torch.empty((nq, num_neighbours), dtype=torch.float32, device=_query.device)
            _capi.check(_capi.lib().dci_b200_query(
                self._live(), C.c_void_p(_query.data_ptr()), nq, num_neighbours, int(num_outer_iterations),
                int(max_num_candidates), 0, self._block_size, self._thread_size,
                C.c_void_p(ids.data_ptr()), C.c_void_p(dists.data_ptr()), _stream_ptr(self._device)))
            if return_int_ids:
                return ids, dists
            return ids.to(torch.float32), dists     # the reference returns ids as float32 (dci_cuda.cpp:111)

    def query_packed(self, query, num_neighbours, num_outer_iterations=5000, *, max_num_candidates=None):
        """The query's result as one [num_queries, k] int64 CUDA tensor of keys
        (fp32 distance bits << 32 | shard-local id; -1 in unused slots): the form MDCI gathers
        between GPUs (dci_b200_query_packed).  An index with fewer than k points (or none)
        answers with what it has."""
        _query = query.unsqueeze(0) if len(query.shape) < 2 else query
        self._check_data(_query)
        self._ensure_positive_integer(num_neighbours)
        if max_num_candidates is None:
            max_num_candidates = 10 * num_neighbours
        nq, k = _query.shape[0], num_neighbours
        kk = min(k, self.num_points)
        with torch.cuda.device(self._device):
            out = torch.empty((nq, kk), dtype=torch.int64, device=_query.device)
            if kk > 0:
                _capi.check(_capi.lib().dci_b200_query_packed(
                    self._live(), C.c_void_p(_query.data_ptr()), nq, kk, int(num_outer_iterations),
                    int(max_num_candidates), self._block_size, self._thread_size, C.c_void_p(out.data_ptr()),
                    _stream_ptr(self._device)))
            if kk < k:
                full = torch.full((nq, k), -1, dtype=torch.int64, device=_query.device)
                full[:, :kk] = out
                out = full
        return out

    def query_noalloc(self, query, ids_out, dists_out, num_outer_iterations=5000, *, max_num_candidates=None):
        """The same query through dci_b200_query_noalloc, for callers that must not
        trigger a device allocation (serving loops with a latency budget, processes
        whose device memory belongs to another allocator).  The caller supplies the
        outputs: ids_out int32 [num_queries, k] and dists_out float32 of the same
        shape, both CUDA and contiguous; k is taken from their shape.  Working
        memory comes from a fixed 32 MiB array inside the library, shared by all
        calls on the device, so calls must not overlap on the GPU; oversized
        problems raise NotImplementedError."""
        _query = query.unsqueeze(0) if len(query.shape) < 2 else query
        self._check_data(_query)
        nq, k = _query.shape[0], ids_out.shape[1]
        for t, dt in ((ids_out, torch.int32), (dists_out, torch.float32)):
            if t.dtype != dt or not t.is_cuda or not t.is_contiguous() or tuple(t.shape) != (nq, k) \
                    or t.device.index != self._device:
                raise TypeError("outputs must be contiguous CUDA tensors of shape [num_queries, k]: int32 ids, float32 distances")
        if max_num_candidates is None:
            max_num_candidates = 10 * k
        with torch.cuda.device(self._device):
            _capi.check(_capi.lib().dci_b200_query_noalloc(
                self._live(), C.c_void_p(_query.data_ptr()), nq, k, int(num_outer_iterations), int(max_num_candidates),
                self._block_size, self._thread_size, C.c_void_p(ids_out.data_ptr()), C.c_void_p(dists_out.data_ptr()),
                _stream_ptr(self._device)))
        return ids_out, dists_out

    def query_host(self, query, num_neighbours, num_outer_iterations=5000, *, max_num_candidates=None):
        """Same query from and to HOST memory through dci_b200_query_host: `query`
        is a CPU float32 tensor; returns CPU (int32 ids, float32 distances)."""
        q = query.reshape(-1, self._dim)
        if q.dtype != torch.float32 or q.is_cuda or not q.is_contiguous():
            raise TypeError("query_host takes a contiguous float32 CPU tensor")
        self._ensure_positive_integer(num_neighbours)
        if max_num_candidates is None:
            max_num_candidates = 10 * num_neighbours
        ids = torch.empty((q.shape[0], num_neighbours), dtype=torch.int32)
        dists = torch.empty((q.shape[0], num_neighbours), dtype=torch.float32)
        _capi.check(_capi.lib().dci_b200_query_host(
            self._live(), C.c_void_p(q.data_ptr()), q.shape[0], num_neighbours, int(num_outer_iterations),
            int(max_num_candidates), 0, self._block_size, self._thread_size,
            C.c_void_p(ids.data_ptr()), C.c_void_p(dists.data_ptr())))
        return ids, dists

    def clear(self):
        _capi.check(_capi.lib().dci_b200_clear(self._live()))
        self.num_points = 0
        self._array = None
        self._store = None

    def reset(self, *, seed=None):
        _capi.check(_capi.lib().dci_b200_reset(self._live(), _default_seed() if seed is None else int(seed)))
        self.num_points = 0
        self._array = None
        self._store = None

    def free(self):
        if self._handle:
            _capi.lib().dci_b200_destroy(self._handle)
            self._handle = C.c_void_p()
        self.num_points = 0
        self._array = None
        self._store = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    # -- inspection helpers used by tests and the benchmark
    def get_index(self):
        """(keys, ids): [L*S, N] float32 / int32 CPU tensors, each partition's segment sorted."""
        I = self._num_comp_indices * self._num_simp_indices
        keys = torch.empty(I, self.num_points, dtype=torch.float32)
        ids = torch.empty(I, self.num_points, dtype=torch.int32)
        _capi.check(_capi.lib().dci_b200_get_index(self._live(), C.c_void_p(keys.data_ptr()), C.c_void_p(ids.data_ptr())))
        return keys, ids

    def set_index(self, data, keys, ids):
        """Installs a sorted index built elsewhere (see get_index) for the CUDA tensor `data`."""
        if self.num_points > 0:
            raise RuntimeError("DCI class does not support insertion of more than one tensor. Must combine all tensors into one tensor before inserting")
        self._check_data(data)
        I = self._num_comp_indices * self._num_simp_indices
        keys = torch.as_tensor(keys, dtype=torch.float32).cpu().contiguous()
        ids = torch.as_tensor(ids, dtype=torch.int32).cpu().contiguous()
        if tuple(keys.shape) != (I, data.shape[0]) or tuple(ids.shape) != (I, data.shape[0]):
            raise ValueError("keys and ids must have shape [num_comp_indices * num_simp_indices, num_points]")
        with torch.cuda.device(self._device):
            _capi.check(_capi.lib().dci_b200_set_index(
                self._live(), C.c_void_p(data.data_ptr()), data.shape[0], self._block_size, self._thread_size,
                C.c_void_p(keys.data_ptr()), C.c_void_p(ids.data_ptr()), _stream_ptr(self._device)))
        self.num_points = data.shape[0]
        self._array = data

    def save(self, path):
        """Writes directions and sorted index to `path` (numpy .npz).  The data tensor is not saved."""
        import numpy as np
        keys, ids = self.get_index()
        np.savez(path, proj=self.get_proj().numpy(), keys=keys.numpy(), ids=ids.numpy(),
                 meta=np.array([self._dim, self._num_comp_indices, self._num_simp_indices, self._block_size,
                                self._thread_size, self.num_points], np.int64))

    @classmethod
    def load(cls, path, data, device=0):
        """Rebuilds an instance from save()'s file and the CUDA tensor the index was built on."""
        import numpy as np
        z = np.load(path)
        dim, L, S, bs, ts, n = [int(v) for v in z["meta"]]
        if data.shape[0] != n:
            raise ValueError("the saved index holds %d points, the tensor %d" % (n, data.shape[0]))
        g = cls(dim, L, S, bs, ts, device, proj=torch.from_numpy(z["proj"]))
        g.set_index(data, z["keys"], z["ids"])
        return g

    def project(self, x):
        """[L*S, n] projected keys of the rows of x (exact fp32 path)."""
        self._check_data(x)
        I = self._num_comp_indices * self._num_simp_indices
        out = torch.empty(I, x.shape[0], dtype=torch.float32, device=x.device)
        with torch.cuda.device(self._device):
            _capi.check(_capi.lib().dci_b200_project(self._live(), C.c_void_p(x.data_ptr()), x.shape[0],
                                                    C.c_void_p(out.data_ptr()), _stream_ptr(self._device)))
        return out

    def enable_work_stats(self, on=True, phases=False):
        """on: per-(query, partition) counters; phases: per-phase SM cycle sums."""
        _capi.check(_capi.lib().dci_b200_enable_work_stats(self._live(), (1 if on else 0) | (2 if phases else 0)))

    def get_work_stats(self, num_queries):
        """[num_queries, P, 6] int64: stop iteration, windows, entries, promoted, lane-0 promotions, exhausted."""
        out = torch.zeros(num_queries, self._block_size, 6, dtype=torch.int64)
        _capi.check(_capi.lib().dci_b200_get_work_stats(self._live(), C.c_void_p(out.data_ptr()),
                                                       num_queries * self._block_size))
        return out

    def get_phase_cycles(self):
        """SM cycles per traversal phase summed over the work items of the last query
        (needs enable_work_stats(..., phases=True))."""
        buf = (C.c_longlong * 16)()
        _capi.check(_capi.lib().dci_b200_get_phase_cycles(self._live(), buf))
        names = ["load_search", "priorities", "ordering_rank", "promotion", "stop_candidates", "distance", "topk",
                 None, "ordering_scan", "ordering_place", "counter_reset"]
        out = {n: int(buf[i]) for i, n in enumerate(names) if n}
        out["work_items"] = int(buf[15])
        out["queries_per_pass"] = int(buf[11])
        out["projection_tma"] = int(buf[13])
        return out

    def set_projection(self, mode):
        """'exact' (default; fixed fp32 summation order, rows streamed by TMA when the shapes allow),
        'exact_plain' (the same keys bit for bit, rows always staged by the computing threads),
        'tf32x3' (tcgen05 tensor cores, persistent TMA pipeline when the shapes allow), 'tf32x3_plain'
        (tensor cores, plain loads) or 'tf32x3_tile' (tensor cores, one TMA-fed tile per CTA)."""
        rc = _capi.lib().dci_b200_set_projection(
            self._live(), {"exact": 0, "tf32x3": 1, "tf32x3_plain": 2, "tf32x3_tile": 3, "exact_plain": 4}[mode])
        if rc == _capi.ERR_STATE:
            raise RuntimeError(_capi.lib().dci_b200_last_error().decode())
        _capi.check(rc)

    def set_max_ctas(self, max_ctas):
        """Caps the number of CTAs of the traversal kernel (0 = automatic).  For tests: with few CTAs
        every CTA works through many (query, partition) pairs one after the other."""
        _capi.check(_capi.lib().dci_b200_set_max_ctas(self._live(), int(max_ctas)))

    def enable_timing(self, on=True):
        _capi.check(_capi.lib().dci_b200_enable_timing(self._live(), 1 if on else 0))

    def last_projection_ms(self):
        """Device time of the kernels of the last projection that ran with timing on."""
        ms = C.c_float()
        _capi.check(_capi.lib().dci_b200_last_projection_ms(self._live(), C.byref(ms)))
        return float(ms.value)

    def get_timing(self):
        """dict of milliseconds spent by the last query per kernel group (timing must be enabled)."""
        buf = (C.c_float * 4)()
        _capi.check(_capi.lib().dci_b200_get_timing(self._live(), buf))
        return dict(project_ms=buf[0], traverse_ms=buf[1], merge_ms=buf[2], traverse_launches=int(buf[3]))

    def launch_count(self):
        return int(_capi.lib().dci_b200_launch_count(self._live()))


def shard_bounds(num_points, num_shards):
    """Row ranges of MDCI's shards (reference core.py:122-125): shard i holds
    rows [i*dpd, (i+1)*dpd) clipped to num_points, dpd = num_points // D + 1."""
    dpd = num_points // num_shards + 1
    return dpd, [(min(i * dpd, num_points), min((i + 1) * dpd, num_points)) for i in range(num_shards)]


def merge_shards(ids, dists, offsets, k):
    """ids/dists: [D, nq, k] int32/float32 CUDA tensors of per-shard results;
    returns ([nq, k] int64 global ids, [nq, k] float32) -- the k smallest per
    query, ties to the lower global id (reference core.py:153-157)."""
    D, nq, kk = ids.shape
    assert kk == k and dists.shape == ids.shape and ids.is_cuda and ids.is_contiguous() and dists.is_contiguous()
    dev = ids.device.index
    out_ids = torch.empty((nq, k), dtype=torch.int64, device=ids.device)
    out_dists = torch.empty((nq, k), dtype=torch.float32, device=ids.device)
    offs = (C.c_longlong * D)(*[int(o) for o in offsets])
    with torch.cuda.device(dev):
        _capi.check(_capi.lib().dci_b200_merge_shards(
            C.c_void_p(ids.data_ptr()), C.c_void_p(dists.data_ptr()), D, nq, k, offs,
            C.c_void_p(out_ids.data_ptr()), C.c_void_p(out_dists.data_ptr()), dev, _stream_ptr(dev)))
    return out_ids, out_dists


def merge_shards_packed(packed, offsets, k):
    """packed: [D, nq, k] int64 CUDA tensor of DCI.query_packed results; same output as merge_shards."""
    D, nq, kk = packed.shape
    assert kk == k and packed.is_cuda and packed.is_contiguous() and packed.dtype == torch.int64
    dev = packed.device.index
    out_ids = torch.empty((nq, k), dtype=torch.int64, device=packed.device)
    out_dists = torch.empty((nq, k), dtype=torch.float32, device=packed.device)
    offs = (C.c_longlong * D)(*[int(o) for o in offsets])
    with torch.cuda.device(dev):
        _capi.check(_capi.lib().dci_b200_merge_shards_packed(
            C.c_void_p(packed.data_ptr()), D, nq, k, offs, C.c_void_p(out_ids.data_ptr()),
            C.c_void_p(out_dists.data_ptr()), dev, _stream_ptr(dev)))
    return out_ids, out_dists


PACKED_MAX_K = 1024     # dci_b200_merge_shards_packed's limit; longer lists travel as two tensors


class MDCI(object):
    """Prioritized DCI sharded over several GPUs (reference: core.py:110-169).

    Two ways to run it:
      * MDCI(dim, ..., devices=[0, 1, ...]): one process drives every device, as
        the reference does; results land on devices[0].
      * MDCI(dim, ..., process_group=pg): one process per GPU (torch.distributed,
        NCCL); every rank calls add/query with the same arguments, holds shard
        `rank` on its current device and receives the merged result.
    Every shard answers every query with its local top-k; the lists are gathered
    and merged on the device by dci_b200_merge_shards.
    """

    def __init__(self, dim, num_comp_indices=2, num_simp_indices=7, bs=100, ts=10, devices=[0], *,
                 process_group=None, seeds=None, projs=None, _local_engine=None, _merge=None, _merge_packed=None):
        self._dim = dim
        self._pg = process_group
        self._merge = merge_shards if _merge is None else _merge
        self._merge_packed = merge_shards_packed if _merge_packed is None else _merge_packed
        self.data_per_device = 0
        if process_group is None:
            self.devices = [_device_index(d) for d in devices]
            self.num_devices = len(self.devices)
            self.dcis = [DCI(dim, num_comp_indices, num_simp_indices, bs, ts, dev,
                             seed=None if seeds is None else seeds[i],
                             proj=None if projs is None else projs[i])
                         for i, dev in enumerate(self.devices)]
        else:
            import torch.distributed as dist
            self._dist = dist
            self.rank = dist.get_rank(process_group)
            self.num_devices = dist.get_world_size(process_group)
            if _local_engine is not None:
                self.dcis = [_local_engine]
            else:
                dev = torch.cuda.current_device()
                self.devices = [dev]
                self.dcis = [DCI(dim, num_comp_indices, num_simp_indices, bs, ts, dev,
                                 seed=None if seeds is None else seeds[self.rank],
                                 proj=None if projs is None else projs[self.rank])]

    def add(self, data):
        # The reference's rule (core.py:122-125) can leave trailing shards without rows (9 points on
        # 4 devices: 3 + 3 + 3 + 0) and then fails inside its CUDA code; here such a shard stays empty
        # and contributes nothing to the merge.
        dpd, bounds = shard_bounds(data.shape[0], self.num_devices)
        self.data_per_device = dpd
        if self._pg is None:
            for i, dev in enumerate(self.devices):
                lo, hi = bounds[i]
                if hi > lo:
                    self.dcis[i].add(data[lo:hi].to(torch.device("cuda", dev)).contiguous())
        else:
            lo, hi = bounds[self.rank]
            if hi > lo:
                shard = data[lo:hi]
                eng = self.dcis[0]
                if isinstance(eng, DCI):
                    shard = shard.to(eng.device).contiguous()
                eng.add(shard)

    def add_local(self, shard, data_per_device):
        """process_group mode only: index `shard` (this rank's rows, already cut by
        the caller) and use `data_per_device` as the id stride between ranks, as
        add() would after slicing a full tensor."""
        if self._pg is None:
            raise RuntimeError("add_local needs MDCI(process_group=...)")
        self.data_per_device = int(data_per_device)
        self.dcis[0].add(shard)

    def query(self, query, num_neighbours=-1, num_outer_iterations=5000, blind=False, *,
              max_num_candidates=None, return_int_ids=False):
        if num_neighbours <= 0:
            raise RuntimeError('num_neighbours must be positive')
        if blind:
            raise NotImplementedError("blind querying is per index: the retrieval orders of different shards cannot be merged")
        _query = query.unsqueeze(0) if len(query.shape) < 2 else query
        k = num_neighbours
        offsets = [self.data_per_device * i for i in range(self.num_devices)]
        if self._pg is None:
            ids, dists = [], []
            home = torch.device("cuda", self.devices[0])
            nq = _query.shape[0]
            for i, dev in enumerate(self.devices):
                n_i = self.dcis[i].num_points
                a = torch.full((nq, k), -1, dtype=torch.int32, device=home)
                d = torch.full((nq, k), float("inf"), dtype=torch.float32, device=home)
                if n_i > 0:      # a shard shorter than k (or empty) answers with what it has
                    q = _query.to(torch.device("cuda", dev)).contiguous()
                    ai, di = self.dcis[i].query(q, min(k, n_i), num_outer_iterations,
                                                max_num_candidates=max_num_candidates, return_int_ids=True)
                    a[:, :ai.shape[1]] = ai.to(home)
                    d[:, :di.shape[1]] = di.to(home)
                ids.append(a)
                dists.append(d)
            out_ids, out_dists = self._merge(torch.stack(ids).contiguous(), torch.stack(dists).contiguous(), offsets, k)
        else:
            eng = self.dcis[0]
            q = _query.to(eng.device).contiguous() if isinstance(eng, DCI) else _query
            nq = q.shape[0]
            if k <= PACKED_MAX_K and hasattr(eng, "query_packed"):
                # one collective per query batch: every rank's lists as 64-bit (distance, id) keys
                mine = eng.query_packed(q, k, num_outer_iterations, max_num_candidates=max_num_candidates)
                packed = torch.empty((self.num_devices * nq, k), dtype=torch.int64, device=mine.device)
                self._dist.all_gather_into_tensor(packed, mine.contiguous(), group=self._pg)   # rank-major
                out_ids, out_dists = self._merge_packed(packed.view(self.num_devices, nq, k), offsets, k)
            else:
                a, d = eng.query(q, k, num_outer_iterations, max_num_candidates=max_num_candidates, return_int_ids=True)
                ids = torch.empty((self.num_devices * nq, k), dtype=a.dtype, device=a.device)
                dists = torch.empty((self.num_devices * nq, k), dtype=d.dtype, device=d.device)
                self._dist.all_gather_into_tensor(ids, a.contiguous(), group=self._pg)      # rank-major concatenation
                self._dist.all_gather_into_tensor(dists, d.contiguous(), group=self._pg)
                out_ids, out_dists = self._merge(ids.view(self.num_devices, nq, k), dists.view(self.num_devices, nq, k),
                                                 offsets, k)
        if return_int_ids:
            return out_ids, out_dists
        return out_ids.to(torch.float32), out_dists

    def clear(self):
        for dci in self.dcis:
            dci.clear()

    def reset(self):
        for dci in self.dcis:
            dci.reset()

    def free(self):
        for dci in self.dcis:
            dci.free()
