"""Search of the index and query parameters for a recall target.

The reference fixes ``max_num_candidates = 10 * num_neighbours`` inside ``DCI.query``
(dciknn_cuda/core.py:87, 141) and leaves the choice of (num_comp_indices, num_simp_indices,
block_size, thread_size, num_outer_iterations) to the caller with no guidance; its headline figure
is "queries per second at recall@k >= r".  This module measures that figure: it builds an index per
parameter set on the caller's data, answers a sample of the caller's queries, scores recall against
exact neighbours and reports the fastest set that reaches the target.

Everything here is host logic over the public ``DCI`` class; the exact neighbours used as ground
truth come from a chunked brute-force pass with torch and are not part of any timed region.
"""
from __future__ import annotations

import itertools
import random
import time
from dataclasses import dataclass, field, asdict

import torch

from .core import DCI


@dataclass(frozen=True)
class Params:
    """One point of the search space; field names follow the reference's arguments."""
    num_comp_indices: int = 2
    num_simp_indices: int = 7
    bs: int = 100
    ts: int = 10
    num_outer_iterations: int = 5000
    max_num_candidates: int | None = None      # None = the reference's 10 * num_neighbours

    def as_dict(self):
        return asdict(self)


@dataclass
class Trial:
    params: Params
    recall: float
    queries_per_s: float
    build_ms: float
    feasible: bool = field(default=False)

    def as_dict(self):
        d = {"recall": self.recall, "queries_per_s": self.queries_per_s, "build_ms": self.build_ms,
             "feasible": self.feasible}
        d.update(self.params.as_dict())
        return d


def default_grid(num_neighbours, num_points):
    """A coarse grid around the reference's defaults (L=2, S=7, P=100, T=10, outer=5000,
    max_num_candidates=10k).  Partition counts that would leave fewer than 4k points per
    partition are dropped: a partition can only return what it holds."""
    k = int(num_neighbours)
    grid = []
    for L, S, P, T, mult in itertools.product((1, 2, 3), (3, 5, 7, 10), (50, 100, 200, 400, 1000), (10, 20),
                                              (2, 5, 10, 20)):
        if -(-num_points // P) < 4 * k:
            continue
        grid.append(Params(L, S, P, T, 5000, mult * k))
    return grid


def exact_neighbours(data, query, k, chunk_bytes=1 << 30):
    """ids [nq, k] of the k nearest rows of `data` for every row of `query` (brute force)."""
    n = data.shape[0]
    rows = max(1, int(chunk_bytes // (4 * n)))
    out = []
    for lo in range(0, query.shape[0], rows):
        d = torch.cdist(query[lo:lo + rows], data)
        out.append(d.topk(k, dim=1, largest=False).indices)
    return torch.cat(out)


def recall(ids, truth):
    """Mean fraction of the true neighbours of a query that `ids` holds.  ids/truth: [nq, k]."""
    ids = ids.to(torch.int64)
    truth = truth.to(torch.int64)
    hit = (ids.unsqueeze(2) == truth.unsqueeze(1)).any(dim=2)
    return float(hit.float().mean())


def select(trials, target_recall):
    """The fastest trial whose recall reaches the target; when none does, the one with the
    highest recall (ties: faster).  Marks `feasible` on every trial."""
    for t in trials:
        t.feasible = t.recall >= target_recall
    ok = [t for t in trials if t.feasible]
    if ok:
        return max(ok, key=lambda t: t.queries_per_s)
    return max(trials, key=lambda t: (t.recall, t.queries_per_s)) if trials else None


def measure(data, query, truth, k, params, device, seed=1, repeats=2, dci_factory=DCI):
    """Builds one index with `params`, answers `query` `repeats` times, returns a Trial."""
    dci = dci_factory(data.shape[1], params.num_comp_indices, params.num_simp_indices, params.bs, params.ts,
                      device=device, seed=seed)
    try:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        dci.add(data)                       # first add sizes the buffers
        dci.clear()
        ev[0].record()
        dci.add(data)
        ev[1].record()
        kw = dict(num_outer_iterations=params.num_outer_iterations, return_int_ids=True)
        if params.max_num_candidates is not None:
            kw["max_num_candidates"] = params.max_num_candidates
        ids, _ = dci.query(query, k, **kw)  # warm-up
        ev[2].record()
        for _ in range(repeats):
            ids, _ = dci.query(query, k, **kw)
        ev[3].record()
        torch.cuda.synchronize(device)
        qps = repeats * query.shape[0] / (ev[2].elapsed_time(ev[3]) * 1e-3)
        return Trial(params, recall(ids, truth), qps, ev[0].elapsed_time(ev[1]))
    finally:
        dci.free()


def tune(data, query, num_neighbours=10, target_recall=0.9, grid=None, sample=1024, seed=1, repeats=2,
         truth=None, progress=None, budget_s=None, measure_fn=measure):
    """Returns (best Trial, all Trials).

    data   [N, dim] float32 CUDA tensor to index.
    query  [nq, dim] float32 CUDA tensor; the first `sample` rows are used.
    grid   iterable of Params (default: `default_grid`).
    truth  optional precomputed exact neighbour ids for the sampled queries.
    budget_s  optional wall-clock limit; the grid is visited in a seeded random order, so a
           search that the limit cuts short is an unbiased sample of the grid.
    A parameter set that the library rejects (for example more indices than it supports) is
    skipped.  `progress`, when given, is called with each finished Trial.
    """
    if not (torch.is_tensor(data) and data.is_cuda and data.dtype == torch.float32):
        raise TypeError("data must be a float32 CUDA tensor")
    if not 0.0 < target_recall <= 1.0:
        raise ValueError("target_recall must be in (0, 1]")
    k = int(num_neighbours)
    q = query[:sample].contiguous()
    device = data.device.index
    if truth is None:
        truth = exact_neighbours(data, q, k)
    grid = list(default_grid(k, data.shape[0]) if grid is None else grid)
    if budget_s is not None:
        random.Random(seed).shuffle(grid)
    trials = []
    t_end = None if budget_s is None else time.monotonic() + budget_s
    for p in grid:
        if t_end is not None and trials and time.monotonic() > t_end:
            break
        try:
            t = measure_fn(data, q, truth, k, p, device, seed=seed, repeats=repeats)
        except (ValueError, NotImplementedError):
            continue
        trials.append(t)
        if progress is not None:
            progress(t)
    return select(trials, target_recall), trials
