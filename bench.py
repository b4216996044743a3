"""Benchmark of the Prioritized DCI query hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (config.workload): 1M points of dim 128 (latent
randn(.,32) @ randn(32,128) + 0.01*randn), 10k queries of the same
distribution, k=10, L=2 composite x S=10 simple indices, P=100 partitions,
window T=10, num_outer_iterations=5000 -- seeded synthetic data.  One step =
one query() call over the whole 10k-query batch on an already built index
(the index build is timed once and reported as build_ms).

With N > 1 (launched by torchrun, one rank per GPU) every rank builds its own
1M-point shard of that distribution and answers all 10k queries on it; the
per-rank top-k lists are all-gathered with NCCL and merged on the device
(MDCI).  Per-GPU work is fixed, so scaling is "weak" and `value` counts (query,
shard) answers per second; `index_queries_per_s` is the query rate of the whole
N-million-point index.  After the timed region the merged lists are checked
against the reference's merge rule recomputed with torch, and recall is
measured against exact brute force over all shards.

At every N the line also carries `sharded_10m`: ONE 10M-point, 96-dimensional
Gaussian-mixture index cut into N shards by the reference's rule
(rows [i*(N//D+1), (i+1)*(N//D+1))), queried with a seeded sample of the
mixture -- the strong-scaling curve of the sharded index (queries/s of the whole
index at N = 1, 2, 4, 8), with recall against exact brute force and the same
merge check.

--impl reference runs the reference project's own CUDA build (oracle/_ref,
compiled from the reference's unmodified sources) on a bounded query sample of
the same workload: the reference has no CPU implementation.  With N > 1 every
rank runs it on the shard the other arm gives that rank, and rank 0 merges the
per-shard lists the way the reference's MDCI does (offset ids, concatenate in
device order, stable sort).  If that library is missing it times the CPU oracle
port instead.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(n_points=1_000_000, n_queries=10_000, dim=128, latent=32, noise=0.01, k=10, L=2, S=10, P=100, T=10,
           outer=5000)
METRIC = "queries/sec at recall@10>=0.9 (1M x 128 fp32 synthetic, k=10, L=2, S=10, P=100, T=10)"

# The sharded index of the `sharded_10m` block: 10M x 96 mixture of 256 Gaussians (centres 4*randn,
# unit noise), k=10, L=2, S=10, reference defaults P=100, T=10 per shard.
SHARDED = dict(n_points=10_000_000, n_queries=2_000, dim=96, kind="mixture", k=10, L=2, S=10, P=100, T=10, outer=5000)

# Other configurations, for manual runs (--workload); the default bench line is the headline workload.
WORKLOADS = {
    "configs1": dict(CFG),
    # 1M x 960, uniform[0,1) rows scaled to unit length, L=3, S=12, max candidates 10000
    "configs2": dict(n_points=1_000_000, n_queries=1_000, dim=960, kind="unit_uniform", k=10, L=3, S=12, P=100, T=10,
                     outer=5000, max_cand=10000),
    # one of 8 shards of the 10M-point mixture: 10M/8+1 points, dim 96
    "configs3_shard": dict(n_points=1_250_001, n_queries=10_000, dim=96, kind="mixture", k=10, L=2, S=10, P=100, T=10,
                           outer=5000),
    # one of 8 shards of 4M x 256: 4M/8+1 points from a 64-d latent, k=100, S=15, 20000 outer iterations
    "configs4_shard": dict(n_points=500_001, n_queries=2_000, dim=256, latent=64, noise=0.0, k=100, L=2, S=15, P=100,
                           T=10, outer=20000),
}

WORKLOAD_LABEL = {"configs1": "configs[1]", "configs2": "configs[2]", "configs3_shard": "configs[3] (one of 8 shards)",
                  "configs4_shard": "configs[4] (one of 8 shards)"}


def make_data(seed, n, nq, cfg, stream=0):
    """Seeded synthetic rows; the last nq rows are the queries.  Default kind: randn(., latent) @
    randn(latent, dim) + noise * randn.  `stream` > 0 draws other rows of the SAME distribution
    (same linear map, same centres): the shards of ranks above 0."""
    g = torch.Generator().manual_seed(seed)
    rows = g if stream == 0 else torch.Generator().manual_seed(seed + 1000 * stream)
    kind = cfg.get("kind", "latent")
    if kind == "unit_uniform":
        z = torch.rand(n + nq, cfg["dim"], generator=rows)
        z /= z.norm(dim=1, keepdim=True)
    elif kind == "mixture":
        centres = 4.0 * torch.randn(256, cfg["dim"], generator=g)
        z = centres[torch.randint(256, (n + nq,), generator=rows)] + torch.randn(n + nq, cfg["dim"], generator=rows)
    else:
        a = torch.randn(cfg["latent"], cfg["dim"], generator=g)
        z = torch.randn(n + nq, cfg["latent"], generator=rows) @ a
        if cfg.get("noise"):
            z += cfg["noise"] * torch.randn(n + nq, cfg["dim"], generator=rows)
    return z[:n].contiguous(), z[n:].contiguous()


MIX_BLOCK = 1 << 16


def mixture_rows(seed, lo, hi, dim, stream=0):
    """Rows [lo, hi) of a seeded 256-centre Gaussian mixture whose rows are drawn block by block
    (block j of 65 536 rows has its own generator), so that a rank can draw its shard of a large
    set without drawing the rest, and every rank count cuts the SAME point set.  `stream` selects an
    independent row sequence around the same centres (the queries)."""
    g = torch.Generator().manual_seed(seed)
    centres = 4.0 * torch.randn(256, dim, generator=g)
    seed = seed + 7919 * stream
    out = torch.empty(hi - lo, dim)
    for j in range(lo // MIX_BLOCK, (hi + MIX_BLOCK - 1) // MIX_BLOCK):
        gb = torch.Generator().manual_seed(seed * 1_000_003 + 17 + j)
        blk = centres[torch.randint(256, (MIX_BLOCK,), generator=gb)] + torch.randn(MIX_BLOCK, dim, generator=gb)
        a, b = max(lo, j * MIX_BLOCK), min(hi, (j + 1) * MIX_BLOCK)
        out[a - lo:b - lo] = blk[a - j * MIX_BLOCK:b - j * MIX_BLOCK]
    return out


def measured_peaks():
    """The pool's measured peaks (HBM copy GB/s, ...), or {} when the file is absent (fallback 6650 GB/s)."""
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.lines, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# ground truth and checks (torch on the GPU; never inside a timed region)

def shard_bruteforce(query, shard, k, id_offset, chunk=1 << 20):
    """Exact k nearest rows of `shard` per query: ([nq, k] distances, [nq, k] global ids)."""
    best_d = torch.full((query.shape[0], k), float("inf"), device=query.device)
    best_i = torch.full((query.shape[0], k), -1, dtype=torch.int64, device=query.device)
    for lo in range(0, shard.shape[0], chunk):
        d = torch.cdist(query, shard[lo:lo + chunk])
        kk = min(k, d.shape[1])
        dd, ii = d.topk(kk, largest=False)
        cat_d = torch.cat([best_d, dd], 1)
        cat_i = torch.cat([best_i, ii + (lo + id_offset)], 1)
        best_d, sel = cat_d.topk(k, largest=False)
        best_i = cat_i.gather(1, sel)
    return best_d, best_i


def gather_all(t, world, dist):
    if world == 1:
        return t.unsqueeze(0)
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous())
    return out


def recall_sharded(ids, query, shard, k, id_offset, world, dist):
    """recall@k of merged global ids against exact brute force over every rank's shard."""
    d, i = shard_bruteforce(query, shard, k, id_offset)
    dd, ii = gather_all(d, world, dist), gather_all(i, world, dist)            # [D, nq, k]
    dd = dd.permute(1, 0, 2).reshape(query.shape[0], -1)
    ii = ii.permute(1, 0, 2).reshape(query.shape[0], -1)
    truth = ii.gather(1, dd.topk(k, largest=False).indices)
    hit = (ids.long().unsqueeze(2) == truth.unsqueeze(1)).any(2).float().sum(1)
    return float((hit / k).mean())


def reference_merge(ids, dists, dpd, k):
    """The reference's MDCI merge (dciknn_cuda/core.py:146-157) with torch: per-device ids offset by
    data_per_device * device, lists concatenated in device order, stable sort by distance, first k.
    ids/dists: [D, nq, k]."""
    D, nq, _ = ids.shape
    off = (torch.arange(D, device=ids.device, dtype=torch.int64) * dpd).view(D, 1, 1)
    gid = torch.where(ids >= 0, ids.long() + off, ids.long())
    gid = gid.permute(1, 0, 2).reshape(nq, -1)
    d = dists.permute(1, 0, 2).reshape(nq, -1)
    order = torch.sort(d, dim=1, stable=True).indices[:, :k]
    return gid.gather(1, order), d.gather(1, order)


def merge_check(engine_ids, engine_dists, local_dci, query, cfg, mc, dpd, world, dist):
    """Compares the engine's merged lists with reference_merge of the per-shard lists."""
    a, d = local_dci.query(query, cfg["k"], cfg["outer"], max_num_candidates=mc, return_int_ids=True)
    aa, dd = gather_all(a, world, dist), gather_all(d, world, dist)
    want_i, want_d = reference_merge(aa, dd, dpd, cfg["k"])
    same_d = bool(torch.equal(want_d.view(torch.int32), engine_dists.view(torch.int32)))
    rows = float((want_i == engine_ids.long()).all(1).float().mean())
    return {"queries": int(query.shape[0]), "dist_bits_equal": same_d, "id_rows_equal": rows}


def cpu_baselines(dci, data_h, query_h, cfg, gpu_ids, gpu_dists, budget_s=12.0):
    """cpu_baseline: the sequential CPU restatement of the reference algorithm (oracle/dci_oracle.c,
    OpenMP over queries) on a bounded query sample, run on the index the GPU built.  Its answers are
    then compared with the GPU's for the same queries, bit for bit: full-size parity.
    cpu_bruteforce: torch.cdist + topk on the host cores."""
    from oracle import oracle
    cores = oracle.lib().dci_oracle_num_threads()
    keys, ids = dci.get_index()
    keys, ids = keys.numpy(), ids.numpy()
    proj = dci.get_proj().numpy()
    data = data_h.numpy()

    def run(nq):
        q = query_h[:nq].numpy()
        qproj = oracle.project(proj, q)
        t0 = time.perf_counter()
        oi, od = oracle.query_index(keys, ids, cfg["L"], cfg["S"], cfg["P"], cfg["T"], data, qproj, q, cfg["k"],
                                    cfg["outer"], 10 * cfg["k"])
        return time.perf_counter() - t0, oi, od

    t_probe, _, _ = run(cores)
    nq = int(max(cores, min(query_h.shape[0], cores * max(1, int(budget_s / max(t_probe, 1e-3))))))
    t, oi, od = run(nq)
    gi, gd = gpu_ids[:nq].cpu().numpy(), gpu_dists[:nq].cpu().numpy()
    parity = {"queries": nq, "against": "sequential CPU restatement of the reference on the same index",
              "id_rows_equal": float((gi == oi).all(1).mean()),
              "dist_bits_equal": bool(np.array_equal(gd.view(np.uint32), od.view(np.uint32)))}
    port = {"value": nq / t, "unit": "queries/s", "cores": cores, "kind": "port",
            "sample": "%d of the %d queries, sequential C restatement of the reference loop, %.1f s" % (nq, query_h.shape[0], t)}
    torch.set_num_threads(os.cpu_count() or 1)
    nb = min(256, query_h.shape[0])
    t0 = time.perf_counter()
    torch.cdist(query_h[:nb], data_h).topk(cfg["k"], largest=False)
    tb = time.perf_counter() - t0
    brute = {"value": nb / tb, "unit": "queries/s", "cores": os.cpu_count(), "kind": "torch.cdist+topk exact",
             "sample": "%d queries, %.1f s" % (nb, tb)}
    return port, brute, parity


def tuned_parameters(data, query, cfg, target=0.9):
    """Not the headline: the fastest of a few parameter sets near the configured one that still
    reaches the recall target on the same data (1 024 queries per trial), found by
    dciknn_cuda_b200.tuning.tune.  The headline `value` stays on the configured parameters."""
    from dciknn_cuda_b200 import tuning
    k = cfg["k"]
    grid = [tuning.Params(cfg["L"], cfg["S"], cfg["P"], cfg["T"], cfg["outer"], 10 * k)]
    grid += [tuning.Params(L, S, P, T, cfg["outer"], m * k)
             for (L, S, P, T, m) in ((1, 10, 100, 10, 20), (1, 10, 100, 20, 10), (1, 10, 400, 10, 5), (1, 10, 200, 10, 10),
                                     (2, 10, 100, 20, 5), (1, 7, 1000, 10, 5), (1, 10, 200, 20, 5))]
    best, trials = tuning.tune(data, query, k, target, grid=grid, sample=1024, seed=2024)
    return {"target_recall": target, "sample_queries": min(1024, query.shape[0]), "trials": len(trials),
            "configured": trials[0].as_dict(), "best": best.as_dict()}


# ---------------------------------------------------------------------------

class Ranks:
    """World description + collectives for one benchmark process."""

    def __init__(self, args, backend="nccl"):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if args.gpus > 1 and self.world != args.gpus:
            raise SystemExit("launch with torchrun --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group(backend, device_id=self.dev)

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        t = torch.tensor([float(x)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_values(self, x):
        t = torch.tensor([float(x)], device=self.dev)
        return [float(v) for v in gather_all(t, self.world, self.dist).flatten().tolist()]

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def time_steps(R, step, steps, warmup):
    """W untimed steps, then K steps between CUDA events, bracketed by barriers; returns
    (max-over-ranks ms per step, per-rank ms per step, result of the last step)."""
    for _ in range(warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    R.barrier()
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    R.barrier()
    mine = e0.elapsed_time(e1) / steps
    return R.max_over_ranks(mine), R.all_values(mine), out


def other_build_times(device):
    """Index build (`add`, warm buffers) of one shard of the two multi-GPU configurations, whose headline
    includes the build: device-generated rows of the same shape (the build does not depend on the values'
    distribution beyond the ties it meets)."""
    from dciknn_cuda_b200 import DCI
    res = {}
    for name in ("configs3_shard", "configs4_shard"):
        c = WORKLOADS[name]
        x = torch.randn(c["n_points"], c["dim"], device="cuda:%d" % device)
        g = DCI(c["dim"], c["L"], c["S"], c["P"], c["T"], device, seed=7)
        g.add(x); torch.cuda.synchronize()
        ts = []
        for _ in range(3):
            g.clear()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); g.add(x); e1.record(); torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        res[name] = {"points": c["n_points"], "dim": c["dim"], "simple_indices": c["L"] * c["S"], "add_ms": statistics.median(ts)}
        del g, x
        torch.cuda.empty_cache()
    return res


def sharded_10m(R, args):
    """The strong-scaling block: one 10M x 96 mixture index over the ranks (reference sharding rule)."""
    from dciknn_cuda_b200 import DCI, MDCI
    from dciknn_cuda_b200.core import shard_bounds
    cfg = dict(SHARDED)
    if args.sharded_points:
        cfg["n_points"] = args.sharded_points
    N, nq, k = cfg["n_points"], cfg["n_queries"], cfg["k"]
    dpd, bounds = shard_bounds(N, R.world)
    lo, hi = bounds[R.rank]
    shard = mixture_rows(3, lo, hi, cfg["dim"]).to(R.dev)
    query_h = mixture_rows(3, 0, nq, cfg["dim"], stream=1)
    query = query_h.to(R.dev)
    if R.world == 1:
        engine = DCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], R.local, seed=3030)
        local_dci = engine
        adder = lambda: engine.add(shard)
    else:
        engine = MDCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], process_group=R.dist.group.WORLD,
                      seeds=[3030 + r for r in range(R.world)])
        local_dci = engine.dcis[0]
        adder = lambda: engine.add_local(shard, dpd)
    adder(); torch.cuda.synchronize()
    local_dci.clear()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); adder(); e1.record(); torch.cuda.synchronize()
    build_ms = R.max_over_ranks(e0.elapsed_time(e1))

    def step():
        return engine.query(query, k, cfg["outer"], return_int_ids=True)

    steps = max(2, min(args.steps, 3))
    ms, per_rank, (ids, dists) = time_steps(R, step, steps, 3)
    q_pin = query_h.pin_memory()

    def e2e_step():
        a, d = engine.query(q_pin.to(R.dev, non_blocking=True), k, cfg["outer"], return_int_ids=True)
        return a.cpu(), d.cpu()
    e2e_step()
    R.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    R.barrier()
    e2e = nq * steps / R.max_over_ranks(time.perf_counter() - t0)
    nrec = min(500, nq)
    rec = recall_sharded(ids[:nrec], query[:nrec], shard, k, lo, R.world, R.dist)
    chk = merge_check(ids[:256], dists[:256], local_dci, query[:256], cfg, None, dpd, R.world, R.dist)
    out = {"workload": "ONE index of %d points x dim %d (256-centre Gaussian mixture) in %d shard(s) of %d rows "
                       "(reference rule N//D+1), %d queries per step, k=%d, L=%d, S=%d, P=%d, T=%d per shard"
                       % (N, cfg["dim"], R.world, dpd if R.world > 1 else N, nq, k, cfg["L"], cfg["S"], cfg["P"], cfg["T"]),
           "scaling": "strong", "queries_per_s": nq / (ms * 1e-3), "unit": "queries/s", "ms_per_step": ms, "steps": steps,
           "ms_per_step_by_rank": per_rank, "e2e_queries_per_s": e2e, "build_ms_per_shard": build_ms,
           "recall_at_10": rec, "merge_check": chk,
           "partition_points": int((hi - lo + cfg["P"] - 1) // cfg["P"])}
    del engine, local_dci, shard
    torch.cuda.empty_cache()
    return out


def bench_ours(args):
    from dciknn_cuda_b200 import DCI, MDCI
    R = Ranks(args)
    world, rank, local, dev = R.world, R.rank, R.local, R.dev
    cfg = dict(WORKLOADS[args.workload])
    if args.points:
        cfg["n_points"] = args.points
    if args.queries:
        cfg["n_queries"] = args.queries
    mc = cfg.get("max_cand")
    # every rank draws the same queries (seed 1); rank r > 0 draws its own shard of the same distribution
    data_h, query_h = make_data(1, cfg["n_points"], cfg["n_queries"], cfg)
    if rank > 0:
        data_h, _ = make_data(1, cfg["n_points"], 0, cfg, stream=rank)
    data = data_h.to(dev)
    query = query_h.to(dev)
    dpd = cfg["n_points"] + 1
    if world == 1:
        engine = DCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], local, seed=2024)
        engine.set_projection(args.projection)
        local_dci = engine
        adder = lambda: engine.add(data)
    else:
        engine = MDCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], process_group=R.dist.group.WORLD,
                      seeds=[2024 + r for r in range(world)])
        local_dci = engine.dcis[0]
        local_dci.set_projection(args.projection)
        adder = lambda: engine.add_local(data, dpd)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    adder(); torch.cuda.synchronize()            # first add also allocates the index buffers
    local_dci.clear(); local_dci.set_projection(args.projection)
    e0.record(); adder(); e1.record(); torch.cuda.synchronize()
    build_ms = e0.elapsed_time(e1)
    # projection of the indexed points alone (it is part of build_ms): HBM-bound, 4*dim bytes in and
    # 4*L*S bytes out per point; both the exact kernel and the tcgen05 3xTF32 kernel are timed
    proj_bytes = cfg["n_points"] * 4 * (cfg["dim"] + cfg["L"] * cfg["S"])
    projection = {"mode": args.projection}
    hbm_peak = measured_peaks().get("hbm_gbs", 6650.0)
    if rank == 0:
        probe = DCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], local, seed=2024)
        for mode in ("exact", "tf32x3"):
            try:
                probe.set_projection(mode)
                probe.enable_timing(True)
                t = []
                for _ in range(4):
                    probe.project(data); torch.cuda.synchronize()
                    t.append(probe.last_projection_ms())     # events right around the kernels
                probe.enable_timing(False)
                t = min(t[1:])
                projection[mode] = {"data_ms": t, "gbps": proj_bytes / (t * 1e-3) / 1e9,
                                    "hbm_frac": proj_bytes / (t * 1e-3) / 1e9 / hbm_peak}
            except Exception as e:      # a kernel that gave up on a bounded wait reports it instead of stopping the bench
                projection[mode] = {"error": str(e)[:200]}
        probe.free()
        projection.update({k: v for k, v in projection.get(args.projection, projection["exact"]).items()
                           if k in ("data_ms", "gbps")})

    def step():
        return engine.query(query, cfg["k"], cfg["outer"], max_num_candidates=mc, return_int_ids=True)

    for _ in range(args.warmup):
        step()
    launches0 = local_dci.launch_count()
    sampler = ClockSampler(local)
    R.barrier()
    if rank == 0:
        sampler.start()
    e0.record()
    for _ in range(args.steps):
        ids, dists = step()
    e1.record()
    R.barrier()
    clocks = sampler.stop() if rank == 0 else None
    mine_ms = e0.elapsed_time(e1) / args.steps
    ms_per_step = R.max_over_ranks(mine_ms)
    per_rank_ms = R.all_values(mine_ms)
    launches = local_dci.launch_count() - launches0 + (args.steps if world > 1 else 0)    # + one shard merge per step
    nq = cfg["n_queries"]
    value = world * nq / (ms_per_step * 1e-3)

    # end to end from host memory: pinned queries in, results back on the host
    q_pin = query_h.pin_memory()

    def e2e_step():
        if world == 1:
            return engine.query_host(q_pin, cfg["k"], cfg["outer"], max_num_candidates=mc)
        a, d = engine.query(q_pin.to(dev, non_blocking=True), cfg["k"], cfg["outer"], max_num_candidates=mc,
                            return_int_ids=True)
        return a.cpu(), d.cpu()
    e2e_step()
    R.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    R.barrier()
    e2e_value = world * nq * args.steps / R.max_over_ranks(time.perf_counter() - t0)
    id_bytes = 8 if world > 1 else 4

    # what the timed steps returned, checked (every rank takes part in the gathers)
    nrec = min(1000, nq)
    rec = recall_sharded(ids[:nrec], query[:nrec], data, cfg["k"], dpd * rank if world > 1 else 0, world, R.dist)
    chk = None
    if world > 1:
        chk = merge_check(ids[:512], dists[:512], local_dci, query[:512], cfg, mc, dpd, world, R.dist)

    out = None
    if rank == 0:
        # roofline of the dominant kernel (traversal): algorithmic bytes from the work counters
        local_dci.enable_work_stats(False, phases=True)
        local_dci.query(query, cfg["k"], cfg["outer"], max_num_candidates=mc)
        torch.cuda.synchronize()
        phases = local_dci.get_phase_cycles()
        local_dci.enable_work_stats(True)
        local_dci.query(query, cfg["k"], cfg["outer"], max_num_candidates=mc)
        torch.cuda.synchronize()
        st = local_dci.get_work_stats(nq)
        local_dci.enable_work_stats(False)
        entries, cands = int(st[:, :, 2].sum()), int(st[:, :, 3].sum())
        algo_bytes = 8 * entries + 4 * cfg["dim"] * cands + nq * (4 * cfg["dim"] + 4 * cfg["L"] * cfg["S"] + 8 * cfg["k"])
        local_dci.enable_timing(True)
        tr, pj, mg, nl = [], [], [], 0
        for _ in range(max(3, args.steps)):
            local_dci.query(query, cfg["k"], cfg["outer"], max_num_candidates=mc)
            t = local_dci.get_timing()
            tr.append(t["traverse_ms"]); pj.append(t["project_ms"]); mg.append(t["merge_ms"]); nl = t["traverse_launches"]
        local_dci.enable_timing(False)
        tr_ms = statistics.mean(tr) / max(nl, 1)
        peaks = measured_peaks()
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = algo_bytes / max(nl, 1) / (tr_ms * 1e-3) / 1e9
        work_items = max(phases["work_items"], 1)
        phase_pw = {k: v / work_items for k, v in phases.items()
                    if k not in ("work_items", "queries_per_pass", "projection_tma")}
        sm_mhz = (clocks or {}).get("sm_mhz") or 0.0
        # A second, honest bound.  The index and rows of a partition stay in L2 across the queries,
        # so the launch moves almost nothing through HBM; what it exhausts is instruction issue.
        # issue_slot_util = warp instructions per launch / (4 issue slots x SMs x SM cycles of the
        # launch), with the instruction count per work item taken from a profiler capture of the same
        # build (--ncu-warp-inst-per-work-item) and the cycles from this run's event time and clock.
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        launch_cycles = tr_ms * 1e-3 * sm_mhz * 1e6
        second = {"binding_resource": "instruction issue (SM front end) and the shared-memory pipe; not HBM",
                  "sm_cycles_per_work_item": sum(phase_pw.values()),
                  "launch_sm_cycles": launch_cycles,
                  "warp_inst_per_work_item": args.ncu_warp_inst_per_work_item,
                  "issue_slot_util": (args.ncu_warp_inst_per_work_item * (nq * cfg["P"] / max(nl, 1)) / (4.0 * sms * launch_cycles)
                                      if args.ncu_warp_inst_per_work_item and launch_cycles else None),
                  "l2_read_gbs": (args.ncu_l2_bytes_per_work_item * (nq * cfg["P"] / max(nl, 1)) / (tr_ms * 1e-3) / 1e9
                                  if args.ncu_l2_bytes_per_work_item else None),
                  "source": "profiler figures passed on the command line; null without them"}
        roofline = {"bound": "hbm", "kernel": "traverse_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_source": "measured" if peaks else "fallback",
                    "traffic": args.ncu_dram_bytes_per_launch, "algorithmic_bytes_per_launch": algo_bytes // max(nl, 1),
                    "launch_ms": tr_ms, "project_ms": statistics.mean(pj), "merge_ms": statistics.mean(mg),
                    "entries_per_query": entries / nq, "candidates_per_query": cands / nq,
                    "phase_cycles_per_work_item": phase_pw,
                    "queries_per_pass": phases["queries_per_pass"], "second_bound": second}
        cpu_port, cpu_brute, parity = (None, None, None)
        if world == 1 and not args.no_cpu_baseline and args.workload == "configs1":
            cpu_port, cpu_brute, parity = cpu_baselines(local_dci, data_h, query_h, cfg, ids, dists)
        tuned = None
        if world == 1 and not args.no_tune and args.workload == "configs1":
            tuned = tuned_parameters(data, query, cfg)
        out = {
            "metric": METRIC, "value": value, "unit": "queries/s" if world == 1 else "(query, shard) answers/s",
            "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s: %d points x dim %d per GPU, %d queries, k=%d, L=%d, S=%d, P=%d, T=%d, num_outer_iterations=%d"
                                   % (WORKLOAD_LABEL[args.workload],
                                      cfg["n_points"], cfg["dim"], nq, cfg["k"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], cfg["outer"]),
                       "points_total": world * cfg["n_points"], "queries_per_step": nq,
                       "l2": "inputs larger than L2 (index %d MB + data %d MB per GPU)"
                             % (cfg["n_points"] * cfg["L"] * cfg["S"] * 10 // 1_000_000, cfg["n_points"] * cfg["dim"] * 4 // 1_000_000),
                       "parallelism": "1 GPU" if world == 1 else "MDCI: %d shards, one NCCL all-gather of packed (distance, id) lists + device merge" % world,
                       "value_unit_note": "every GPU answers every query on its own 1M-point shard: value counts (query, shard) "
                                          "answers per second; index_queries_per_s is the rate of the whole %d-point index" % (world * cfg["n_points"])
                                          if world > 1 else "queries per second"},
            "index_queries_per_s": nq / (ms_per_step * 1e-3),
            "ms_per_step_by_rank": per_rank_ms,
            "build_ms": build_ms, "recall_at_10": rec, "merge_check": chk, "parity": parity,
            "projection": projection,
            "e2e": {"value": e2e_value, "unit": "queries/s" if world == 1 else "(query, shard) answers/s",
                    "h2d_bytes_per_step": nq * cfg["dim"] * 4, "d2h_bytes_per_step": nq * cfg["k"] * (4 + id_bytes)},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu_port, "cpu_bruteforce": cpu_brute, "tuned": tuned,
        }
    del engine, local_dci, data
    torch.cuda.empty_cache()
    if out is not None and world == 1 and args.workload == "configs1" and not args.no_sharded:
        out["build_ms_other_shapes"] = other_build_times(local)
    block = None
    if not args.no_sharded and args.workload == "configs1":
        block = sharded_10m(R, args)
    R.close()
    if out is not None:
        out["sharded_10m"] = block
        print(json.dumps(out), flush=True)


def bench_reference(args):
    """The reference's own CUDA build on the workload of the other arm.  Rank r of N builds a
    reference index on the shard the other arm gives rank r and answers the same query sample; rank 0
    merges the per-shard lists by the reference's MDCI rule.  One query at a time is all the reference
    can do (src/dci_cuda_kernel.cu:833), so its rate does not depend on the batch and a bounded sample
    per step stands for the full batch."""
    from oracle import reference
    cfg = dict(WORKLOADS[args.workload])
    if args.points:
        cfg["n_points"] = args.points
    if args.queries:
        cfg["n_queries"] = args.queries
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    base = {"impl": "reference", "metric": METRIC, "unit": "queries/s" if world == 1 else "(query, shard) answers/s",
            "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "%s: %d points x dim %d per GPU, %d queries, k=%d, L=%d, S=%d, P=%d, T=%d, num_outer_iterations=%d"
                                   % (WORKLOAD_LABEL[args.workload], cfg["n_points"], cfg["dim"], cfg["n_queries"], cfg["k"],
                                      cfg["L"], cfg["S"], cfg["P"], cfg["T"], cfg["outer"]),
                       "points_total": world * cfg["n_points"]}}
    if not reference.available():
        if rank != 0:
            return
        data_h, query_h = make_data(1, cfg["n_points"], cfg["n_queries"], cfg)
        from oracle import oracle
        cores = oracle.lib().dci_oracle_num_threads()
        rng = np.random.default_rng(0)
        proj = rng.standard_normal((cfg["L"] * cfg["S"], cfg["dim"])).astype(np.float32)
        proj /= np.linalg.norm(proj, axis=1, keepdims=True)
        o = oracle.OracleDCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], proj)
        o.add(data_h.numpy())
        nq = 2 * cores
        q = query_h.numpy()
        for w in range(args.warmup):
            o.query(q[:nq], cfg["k"], cfg["outer"])
        t0 = time.perf_counter()
        for s in range(args.steps):
            o.query(q[s * nq:(s + 1) * nq], cfg["k"], cfg["outer"])
        t = time.perf_counter() - t0
        value = nq * args.steps / t
        base.update({"value": value, "n_gpus": 1, "unit": "queries/s", "ms_per_step": 1e3 * t / args.steps, "gpu_launches": 0,
                     "cpu_baseline": {"value": value, "unit": "queries/s", "cores": cores, "kind": "port",
                                      "sample": "%d queries per step, CPU restatement (reference build absent)" % nq},
                     "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        base["config"]["sample_queries_per_step"] = nq
        print(json.dumps(base), flush=True)
        return

    R = Ranks(args)
    dev = R.dev
    data_h, query_h = make_data(1, cfg["n_points"], cfg["n_queries"], cfg)
    if rank > 0:
        data_h, _ = make_data(1, cfg["n_points"], 0, cfg, stream=rank)
    data, query = data_h.to(dev), query_h.to(dev)
    dpd = cfg["n_points"] + 1
    k = cfg["k"]
    ref = reference.ReferenceDCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], dev.index)
    t0 = time.perf_counter(); ref.add(data); build_s = time.perf_counter() - t0
    t0 = time.perf_counter(); ref.query(query[:4], k, cfg["outer"]); probe = (time.perf_counter() - t0) / 4
    nq = int(max(4, min(args.ref_queries, 6.0 / max(probe, 1e-4))))
    if world > 1:      # every rank must use the same sample size
        t = torch.tensor([nq], device=dev)
        R.dist.all_reduce(t, op=R.dist.ReduceOp.MIN)
        nq = int(t.item())

    def step(s):
        lo = (s * nq) % (cfg["n_queries"] - nq + 1)
        a, d = ref.query(query[lo:lo + nq], k, cfg["outer"])           # synchronous, as the reference is
        if world == 1:
            return lo, a.long(), d
        aa, dd = gather_all(a, world, R.dist), gather_all(d, world, R.dist)   # the reference gathers to one device
        mi, md = reference_merge(aa, dd, dpd, k)
        return lo, mi, md

    for w in range(args.warmup):
        step(w)
    R.barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        lo, ids, dists = step(args.warmup + s)
    R.barrier()
    t = R.max_over_ranks(time.perf_counter() - t0)
    rec = recall_sharded(ids, query[lo:lo + nq], data, k, dpd * rank if world > 1 else 0, world, R.dist)
    value = world * nq * args.steps / t
    if rank == 0:
        base.update({"value": value, "ms_per_step": 1e3 * t / args.steps, "build_ms": build_s * 1e3, "recall_at_10": rec,
                     "index_queries_per_s": nq * args.steps / t,
                     "gpu_launches": 0,
                     "cpu_baseline": {"value": value, "unit": base["unit"], "cores": 1, "kind": "reference",
                                      "sample": "the reference's own CUDA build (oracle/_ref/libdci_ref.so) on %d B200, "
                                                "%d queries per step; it has no CPU implementation and answers one query "
                                                "at a time" % (world, nq)},
                     "e2e": {"value": value, "unit": base["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        base["config"]["sample_queries_per_step"] = nq
        base["config"]["parallelism"] = "1 GPU" if world == 1 else \
            "one reference index per GPU on its own shard, lists gathered and merged with torch as the reference's MDCI does"
    ref.free()
    R.close()
    if rank == 0:
        print(json.dumps(base), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="configs1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-tune", action="store_true", help="skip the parameter search reported under 'tuned'")
    ap.add_argument("--no-sharded", action="store_true", help="skip the 10M-point sharded-index block")
    ap.add_argument("--sharded-points", type=int, default=0, help="override the sharded block's number of points")
    ap.add_argument("--points", type=int, default=0, help="override the workload's number of points (per GPU)")
    ap.add_argument("--queries", type=int, default=0, help="override the workload's number of queries")
    ap.add_argument("--ref-queries", type=int, default=256, help="cap on the reference arm's queries per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--projection", default="exact", choices=["exact", "tf32x3", "tf32x3_plain", "tf32x3_tile"],
                    help="exact fp32 projection (default) or the tcgen05 3xTF32 kernel")
    # figures of a profiler capture of the traversal kernel, for the lines that need them (null otherwise)
    ap.add_argument("--ncu-dram-bytes-per-launch", type=float, default=None,
                    help="dram__bytes_read.sum + dram__bytes_write.sum of one traversal launch of this run's size")
    ap.add_argument("--ncu-warp-inst-per-work-item", type=float, default=None,
                    help="warp instructions executed per (query, partition) work item")
    ap.add_argument("--ncu-l2-bytes-per-work-item", type=float, default=None,
                    help="bytes the SMs read from L2 per work item")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.impl == "reference":
        bench_reference(args)
    else:
        bench_ours(args)


if __name__ == "__main__":
    main()
