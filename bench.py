"""Benchmark of the Prioritized DCI query hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload): BASELINE.json configs[1] -- 1M points, dim 128
(latent randn(.,32) @ randn(32,128) + 0.01*randn), 10k queries of the same
distribution, k=10, L=2 composite x S=10 simple indices, P=100 partitions,
window T=10, num_outer_iterations=5000 -- seeded synthetic data.  One step =
one query() call over the whole 10k-query batch on an already built index
(the index build is timed once and reported as build_ms).

With N > 1 (launched by torchrun, one rank per GPU) every rank builds its own
1M-point shard of that distribution and answers all 10k queries on it; the
per-rank top-k lists are all-gathered with NCCL and merged on the device
(MDCI).  Per-GPU work is fixed, so scaling is "weak" and `value` counts (query,
shard) answers per second; `index_queries_per_s` is the query rate of the whole
N-million-point index.

--impl reference runs the reference project's own CUDA build (oracle/_ref,
compiled from the reference's unmodified sources) on a bounded query sample of
the same workload: the reference has no CPU implementation.  If that library is
missing it times the CPU oracle port instead.
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


# Other BASELINE.json configurations, for manual runs (--workload); the default bench line is configs[1].
WORKLOADS = {
    "configs1": dict(CFG),
    # configs[2]: 1M x 960, uniform[0,1) rows scaled to unit length, L=3, S=12, max candidates 10000
    "configs2": dict(n_points=1_000_000, n_queries=1_000, dim=960, kind="unit_uniform", k=10, L=3, S=12, P=100, T=10,
                     outer=5000, max_cand=10000),
    # configs[3], one of 8 shards: 10M/8+1 points of a 256-centre Gaussian mixture, dim 96
    "configs3_shard": dict(n_points=1_250_001, n_queries=10_000, dim=96, kind="mixture", k=10, L=2, S=10, P=100, T=10,
                           outer=5000),
    # configs[4], one of 8 shards: 4M/8+1 points, dim 256 from a 64-d latent, k=100, S=15, 20000 outer iterations
    "configs4_shard": dict(n_points=500_001, n_queries=2_000, dim=256, latent=64, noise=0.0, k=100, L=2, S=15, P=100,
                           T=10, outer=20000),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one traversal launch from an ncu capture
# (profiles/traverse_kernel_configs1.md).  The index and the rows are read about once per launch and
# everything else hits L2, so the figure does not grow with the number of queries.
NCU_DRAM_BYTES_PER_LAUNCH = {"configs1": 723_818_000}

WORKLOAD_LABEL = {"configs1": "configs[1]", "configs2": "configs[2]", "configs3_shard": "configs[3] (one of 8 shards)",
                  "configs4_shard": "configs[4] (one of 8 shards)"}


def make_data(seed, n, nq, cfg):
    """Seeded synthetic rows; the last nq rows are the queries.  Default kind: randn(., latent) @
    randn(latent, dim) + noise * randn."""
    g = torch.Generator().manual_seed(seed)
    kind = cfg.get("kind", "latent")
    if kind == "unit_uniform":
        z = torch.rand(n + nq, cfg["dim"], generator=g)
        z /= z.norm(dim=1, keepdim=True)
    elif kind == "mixture":
        centres = 4.0 * torch.randn(256, cfg["dim"], generator=g)
        z = centres[torch.randint(256, (n + nq,), generator=g)] + torch.randn(n + nq, cfg["dim"], generator=g)
    else:
        a = torch.randn(cfg["latent"], cfg["dim"], generator=g)
        z = torch.randn(n + nq, cfg["latent"], generator=g) @ a
        if cfg.get("noise"):
            z += cfg["noise"] * torch.randn(n + nq, cfg["dim"], generator=g)
    return z[:n].contiguous(), z[n:].contiguous()


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


def recall_at_k(ids, data, query, k):
    """recall against exact brute force computed with torch on the GPU (ground truth only)."""
    d2 = torch.cdist(query, data)
    truth = d2.topk(k, largest=False).indices
    hit = (ids.long().unsqueeze(2) == truth.unsqueeze(1)).any(2).float().sum(1)
    return float((hit / k).mean())


def cpu_baselines(dci, data_h, query_h, cfg, budget_s=12.0):
    """cpu_baseline: the sequential CPU restatement of the reference algorithm
    (oracle/dci_oracle.c, OpenMP over queries) on a bounded query sample, using
    the index the GPU built (tests show it is identical to the oracle's own).
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
        oracle.query_index(keys, ids, cfg["L"], cfg["S"], cfg["P"], cfg["T"], data, qproj, q, cfg["k"],
                           cfg["outer"], 10 * cfg["k"])
        return time.perf_counter() - t0

    t_probe = run(cores)
    nq = int(max(cores, min(query_h.shape[0], cores * max(1, int(budget_s / max(t_probe, 1e-3))))))
    t = run(nq)
    port = {"value": nq / t, "unit": "queries/s", "cores": cores, "kind": "port",
            "sample": "%d of the %d queries, sequential C restatement of the reference loop, %.1f s" % (nq, query_h.shape[0], t)}
    torch.set_num_threads(os.cpu_count() or 1)
    nb = min(256, query_h.shape[0])
    t0 = time.perf_counter()
    torch.cdist(query_h[:nb], data_h).topk(cfg["k"], largest=False)
    tb = time.perf_counter() - t0
    brute = {"value": nb / tb, "unit": "queries/s", "cores": os.cpu_count(), "kind": "torch.cdist+topk exact",
             "sample": "%d queries, %.1f s" % (nb, tb)}
    return port, brute


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


def bench_ours(args):
    import torch.distributed as dist
    from dciknn_cuda_b200 import DCI, MDCI
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit("launch with torchrun --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = dict(WORKLOADS[args.workload])
    if args.points:
        cfg["n_points"] = args.points
    if args.queries:
        cfg["n_queries"] = args.queries
    mc = cfg.get("max_cand")
    # every rank draws the same queries (seed 1); rank r > 0 draws its own shard
    data_h, query_h = make_data(1, cfg["n_points"], cfg["n_queries"], cfg)
    if rank > 0:
        data_h, _ = make_data(1 + 1000 * rank, cfg["n_points"], 0, cfg)
    data = data_h.to(dev)
    query = query_h.to(dev)
    if world == 1:
        engine = DCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], local, seed=2024)
        engine.set_projection(args.projection)
        local_dci = engine
        adder = lambda: engine.add(data)
    else:
        engine = MDCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], process_group=dist.group.WORLD,
                      seeds=[2024 + r for r in range(world)])
        local_dci = engine.dcis[0]
        local_dci.set_projection(args.projection)
        adder = lambda: engine.add_local(data, cfg["n_points"] + 1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    adder(); torch.cuda.synchronize()            # first add also allocates the index buffers
    local_dci.clear(); local_dci.set_projection(args.projection)
    e0.record(); adder(); e1.record(); torch.cuda.synchronize()
    build_ms = e0.elapsed_time(e1)
    # projection of the indexed points alone (it is part of build_ms): HBM-bound, 4*dim bytes in and
    # 4*L*S bytes out per point
    proj_ms = []
    local_dci.enable_timing(True)
    for _ in range(4):
        local_dci.project(data); torch.cuda.synchronize()
        proj_ms.append(local_dci.last_projection_ms())     # events right around the kernels
    local_dci.enable_timing(False)
    proj_ms = min(proj_ms[1:])
    proj_bytes = cfg["n_points"] * 4 * (cfg["dim"] + cfg["L"] * cfg["S"])

    def step():
        return engine.query(query, cfg["k"], cfg["outer"], max_num_candidates=mc, return_int_ids=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    launches0 = local_dci.launch_count()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    e0.record()
    for _ in range(args.steps):
        ids, dists = step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms.item())
    launches = local_dci.launch_count() - launches0 + (args.steps if world > 1 else 0)
    ms_per_step = total_ms / args.steps
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
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_t = torch.tensor([time.perf_counter() - t0], device=dev)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_value = world * nq * args.steps / float(e2e_t.item())
    id_bytes = 8 if world > 1 else 4

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
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = algo_bytes / max(nl, 1) / (tr_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "traverse_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_source": "measured" if peaks else "fallback",
                    "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload), "algorithmic_bytes_per_launch": algo_bytes // max(nl, 1),
                    "launch_ms": tr_ms, "project_ms": statistics.mean(pj), "merge_ms": statistics.mean(mg),
                    "entries_per_query": entries / nq, "candidates_per_query": cands / nq,
                    "phase_cycles_per_work_item": {k: v / max(phases["work_items"], 1) for k, v in phases.items()
                                                   if k not in ("work_items", "queries_per_pass", "projection_tma")},
                    "queries_per_pass": phases["queries_per_pass"]}
        nrec = min(1000, nq)
        rec = recall_at_k(ids[:nrec] if world == 1 else ids[:nrec], data, query[:nrec], cfg["k"]) if world == 1 else None
        cpu_port, cpu_brute = (None, None)
        if world == 1 and not args.no_cpu_baseline and args.workload == "configs1":
            cpu_port, cpu_brute = cpu_baselines(local_dci, data_h, query_h, cfg)
        tuned = None
        if world == 1 and not args.no_tune and args.workload == "configs1":
            tuned = tuned_parameters(data, query, cfg)
        out = {
            "metric": METRIC, "value": value, "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s: %d points x dim %d per GPU, %d queries, k=%d, L=%d, S=%d, P=%d, T=%d, num_outer_iterations=%d"
                                   % (WORKLOAD_LABEL[args.workload],
                                      cfg["n_points"], cfg["dim"], nq, cfg["k"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], cfg["outer"]),
                       "points_total": world * cfg["n_points"], "queries_per_step": nq,
                       "l2": "inputs larger than L2 (index %d MB + data %d MB per GPU)"
                             % (cfg["n_points"] * cfg["L"] * cfg["S"] * 10 // 1_000_000, cfg["n_points"] * cfg["dim"] * 4 // 1_000_000),
                       "parallelism": "1 GPU" if world == 1 else "MDCI: %d shards, NCCL all-gather + device merge" % world,
                       "value_unit_note": "(query, shard) answers per second" if world > 1 else "queries per second"},
            "index_queries_per_s": nq / (ms_per_step * 1e-3),
            "build_ms": build_ms, "recall_at_10": rec,
            "projection": {"mode": args.projection, "data_ms": proj_ms, "gbps": proj_bytes / (proj_ms * 1e-3) / 1e9},
            "e2e": {"value": e2e_value, "unit": "queries/s", "h2d_bytes_per_step": nq * cfg["dim"] * 4,
                    "d2h_bytes_per_step": nq * cfg["k"] * (4 + id_bytes)},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu_port, "cpu_bruteforce": cpu_brute, "tuned": tuned,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if out is not None:
        print(json.dumps(out), flush=True)


def bench_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(WORKLOADS[args.workload])
    if args.points:
        cfg["n_points"] = args.points
    if args.queries:
        cfg["n_queries"] = args.queries
    data_h, query_h = make_data(1, cfg["n_points"], cfg["n_queries"], cfg)
    base = {"impl": "reference", "metric": METRIC, "unit": "queries/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "configs[1]: %d points x dim %d, k=%d, L=%d, S=%d, P=%d, T=%d, num_outer_iterations=%d"
                                   % (cfg["n_points"], cfg["dim"], cfg["k"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], cfg["outer"])}}
    from oracle import reference
    if reference.available():
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        data, query = data_h.to(dev), query_h.to(dev)
        ref = reference.ReferenceDCI(cfg["dim"], cfg["L"], cfg["S"], cfg["P"], cfg["T"], dev.index)
        t0 = time.perf_counter(); ref.add(data); build_s = time.perf_counter() - t0
        t0 = time.perf_counter(); ref.query(query[:4], cfg["k"], cfg["outer"]); probe = (time.perf_counter() - t0) / 4
        nq = int(max(4, min(args.ref_queries, 6.0 / max(probe, 1e-4))))
        for w in range(args.warmup):
            ref.query(query[w * nq:(w + 1) * nq], cfg["k"], cfg["outer"])
        t0 = time.perf_counter()
        for s in range(args.steps):
            lo = ((args.warmup + s) * nq) % (cfg["n_queries"] - nq + 1)
            ids, dists = ref.query(query[lo:lo + nq], cfg["k"], cfg["outer"])
        t = time.perf_counter() - t0
        rec = recall_at_k(ids, data, query[lo:lo + nq], cfg["k"])
        value = nq * args.steps / t
        base.update({"value": value, "ms_per_step": 1e3 * t / args.steps, "build_ms": build_s * 1e3, "recall_at_10": rec,
                     "gpu_launches": 0,
                     "cpu_baseline": {"value": value, "unit": "queries/s", "cores": 1, "kind": "reference",
                                      "sample": "the reference's own CUDA build (oracle/_ref/libdci_ref.so) on one B200, "
                                                "%d queries per step; it has no CPU implementation and answers one query at a time" % nq},
                     "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        base["config"]["queries_per_step"] = nq
    else:
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
        base.update({"value": value, "ms_per_step": 1e3 * t / args.steps, "gpu_launches": 0,
                     "cpu_baseline": {"value": value, "unit": "queries/s", "cores": cores, "kind": "port",
                                      "sample": "%d queries per step, CPU restatement (reference build absent)" % nq},
                     "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        base["config"]["queries_per_step"] = nq
    print(json.dumps(base), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="configs1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-tune", action="store_true", help="skip the parameter search reported under 'tuned'")
    ap.add_argument("--points", type=int, default=0, help="override the workload's number of points (per GPU)")
    ap.add_argument("--queries", type=int, default=0, help="override the workload's number of queries")
    ap.add_argument("--ref-queries", type=int, default=256, help="cap on the reference arm's queries per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--projection", default="exact", choices=["exact", "tf32x3", "tf32x3_plain", "tf32x3_tile"],
                    help="exact fp32 projection (default) or the tcgen05 3xTF32 kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.impl == "reference":
        bench_reference(args)
    else:
        bench_ours(args)


if __name__ == "__main__":
    main()
