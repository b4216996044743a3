"""Generates tests/golden/*.npz by running the reference project's own CUDA
build (oracle/_ref, see oracle/build_ref.py) on a GPU.

Run on a machine with a GPU from the repository root:
    python tests/golden/make_golden.py <output directory>
For every case it records the inputs (data, queries, directions), what the
reference built (its sorted index: keys and ids per simple index, read back
from its `indices` array), the queries as the reference's own cuBLAS call
projects them, and the neighbours it returns: from the unmodified build
(`asis_*`; subject to its top-k scratch race) and from the build whose scratch
offset is patched to be per-thread (`fixed_*`; deterministic).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.reference import ReferenceDCI  # noqa: E402

CASES = [
    # name,           N,    d,  L, S, P,  T,  k, outer, max_cand, nq
    ("insertion_sort", 600, 32, 2, 5, 12, 10, 5, 5000, 50, 40),
    ("quick_sort",    1000, 32, 2, 5, 4,  10, 5, 5000, 50, 40),
    ("quota_stops",   4000, 16, 2, 3, 2,  10, 3, 5000, 30, 24),
    ("outer_cap",     4000, 16, 2, 3, 2,  10, 3, 40,   3000, 24),
    ("ragged_t7",      997, 20, 3, 4, 10, 7,  4, 5000, 40, 32),
]


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda", 0)
    for name, N, d, L, S, P, T, k, outer, mc, nq in CASES:
        rng = np.random.default_rng(abs(hash(name)) % (2 ** 31) if False else sum(map(ord, name)))
        z = (rng.standard_normal((N + nq, 12)) @ rng.standard_normal((12, d))).astype(np.float32)
        z += np.float32(0.05) * rng.standard_normal((N + nq, d)).astype(np.float32)
        data, query = np.ascontiguousarray(z[:N]), np.ascontiguousarray(z[N:])
        rec = dict(data=data, query=query, params=np.array([L, S, P, T, k, outer, mc], np.int64))
        tdata, tquery = torch.from_numpy(data).to(dev), torch.from_numpy(query).to(dev)
        proj = None
        for tag, fixed in (("asis", False), ("fixed", True)):
            ref = ReferenceDCI(d, L, S, P, T, 0, race_fixed=fixed)
            if proj is None:
                proj = ref.get_proj()          # the reference's own cuRAND directions
                rec["proj"] = proj
            else:
                ref.set_proj(proj)
            ref.add(tdata)
            if tag == "asis":
                rec["ref_keys"], rec["ref_ids"] = ref.get_index()
                rec["ref_qproj"] = ref.project_queries(tquery)
            ids, dists = ref.query(tquery, k, outer, mc)
            rec[tag + "_ids"] = ids.cpu().numpy()
            rec[tag + "_dists"] = dists.cpu().numpy()
            ref.free()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **rec)
        same = float((rec["asis_ids"] == rec["fixed_ids"]).all(1).mean())
        print("%s: N=%d P=%d  as-is == race-fixed on %.1f%% of queries" % (name, N, P, 100 * same), flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "golden_out"))
