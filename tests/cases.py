"""Seeded synthetic inputs shared by the tests (shapes follow the benchmark
configurations; sizes are cut down so the sequential oracle finishes in seconds)."""
import numpy as np


def unit_rows(rng, rows, dim):
    p = rng.standard_normal((rows, dim)).astype(np.float32)
    return (p / np.linalg.norm(p, axis=1, keepdims=True)).astype(np.float32)


def latent_linear(rng, n, latent, dim, noise=0.0):
    z = rng.standard_normal((n, latent)).astype(np.float32) @ rng.standard_normal((latent, dim)).astype(np.float32)
    if noise:
        z = z + np.float32(noise) * rng.standard_normal((n, dim)).astype(np.float32)
    return np.ascontiguousarray(z, dtype=np.float32)


def example_config(seed=0, n=2000, nq=500):
    """configs[0]: 2000 points, dim 100 from a 50-d latent, 500 queries, L=2, S=7, P=100, T=10, k=10."""
    rng = np.random.default_rng(seed)
    z = latent_linear(rng, n + nq, 50, 100)
    return dict(data=z[:n], query=z[n:], L=2, S=7, P=100, T=10, k=10, outer=5000,
                proj=unit_rows(rng, 14, 100))


def c2_shaped(seed=1, n=40000, nq=24, P=4):
    """configs[1] cut down: partitions of 10 000 points, dim 128 from a 32-d latent + noise, L=2, S=10."""
    rng = np.random.default_rng(seed)
    z = latent_linear(rng, n + nq, 32, 128, noise=0.01)
    return dict(data=z[:n], query=z[n:], L=2, S=10, P=P, T=10, k=10, outer=5000,
                proj=unit_rows(rng, 20, 128))


def mixture(rng, n, dim, centres=256):
    """Rows around `centres` Gaussian centres (4 * randn), unit noise: the sharded 10M-point
    configuration's distribution."""
    c = (4.0 * rng.standard_normal((centres, dim))).astype(np.float32)
    z = c[rng.integers(0, centres, n)] + rng.standard_normal((n, dim)).astype(np.float32)
    return np.ascontiguousarray(z, dtype=np.float32)


def unit_uniform(rng, n, dim):
    """uniform[0, 1) entries, every row scaled to unit length: the high-dimensional configuration."""
    z = rng.random((n, dim), dtype=np.float32)
    return np.ascontiguousarray(z / np.linalg.norm(z, axis=1, keepdims=True), dtype=np.float32)


def high_dim_shaped(seed=2, n=8000, nq=32, P=4):
    """configs[2] cut down: dim 960 unit-length uniform rows, L=3, S=12 (36 simple indices), quota 10 000."""
    rng = np.random.default_rng(seed)
    z = unit_uniform(rng, n + nq, 960)
    return dict(data=z[:n], query=z[n:], L=3, S=12, P=P, T=10, k=10, outer=5000, max_cand=10000,
                proj=unit_rows(rng, 36, 960))


def mixture_shaped(seed=3, n=40000, nq=96, P=4):
    """configs[3] cut down: 256-centre Gaussian mixture in dim 96, L=2, S=10."""
    rng = np.random.default_rng(seed)
    z = mixture(rng, n + nq, 96)
    return dict(data=z[:n], query=z[n:], L=2, S=10, P=P, T=10, k=10, outer=5000, max_cand=100,
                proj=unit_rows(rng, 20, 96))


def large_k_shaped(seed=4, n=4800, nq=8, P=4):
    """configs[4] cut down: dim 256 from a 64-d latent, k=100, L=2, S=15, 20 000 outer iterations."""
    rng = np.random.default_rng(seed)
    z = latent_linear(rng, n + nq, 64, 256)
    return dict(data=z[:n], query=z[n:], L=2, S=15, P=P, T=10, k=100, outer=20000, max_cand=1000,
                proj=unit_rows(rng, 30, 256))


EDGE_CASES = [
    # name,                N,    d, L, S, P,  T,  k, outer, max_cand, nq, special
    ("tiny_one_point",      1,    5, 1, 1, 1,  1,  1, 10,    10,       4, None),
    ("n_less_than_T",       7,    9, 2, 3, 1, 10,  3, 50,    30,       6, None),
    ("ragged_partitions", 103,   16, 2, 4, 10, 4,  5, 100,   50,       8, None),
    ("more_parts_than_pts", 13,   8, 2, 2, 40, 3,  2, 20,    20,       5, None),
    ("T_equals_1",         200,  12, 2, 5, 3,  1,  4, 30,    40,       6, None),
    ("wide_window",        300,  12, 1, 4, 2, 64,  4, 30,    40,       6, None),
    ("many_indices",       400,  24, 3, 12, 4, 10, 10, 5000, 100,      6, None),
    ("dim_not_multiple_4", 500,  37, 2, 6, 5, 10,  8, 5000,  80,       6, None),
    ("duplicate_keys",     600,  10, 2, 4, 3,  7,  6, 40,    60,       8, "round"),
    ("far_queries",        500,  16, 2, 5, 4, 10,  5, 200,   50,       8, "far"),
    ("k_equals_partition", 240,  16, 2, 3, 8, 10, 30, 5000,  300,      5, None),
    ("quota_reached_early", 5000, 16, 2, 3, 2, 10, 2, 5000,  4,        8, None),
    ("outer_cap_hits",     5000, 16, 2, 3, 2, 10,  2, 3,     1000000,  8, None),
    ("max_cand_zero",      800,  16, 2, 3, 2, 10,  2, 5000,  0,        6, None),
    ("big_k",              900,  16, 2, 3, 3, 10, 700, 5000, 7000,     4, None),
    ("identical_points",   700,  8,  2, 3, 2, 10, 5, 5000,  50,       4, "identical"),
    ("two_clusters_equal", 3000, 8,  2, 4, 1, 10, 5, 5000,  50,       4, "clusters"),
    # few windows (a small CTA) and two distinct priorities with many ties: the radix-sort fallback
    ("two_clusters_small",  600, 8,  2, 4, 2, 10, 5, 5000,  50,       4, "clusters"),
    ("three_values_small",  400, 6,  1, 5, 1,  7, 4, 5000,  40,       4, "round"),
]


def edge_case(row, seed=7):
    name, N, d, L, S, P, T, k, outer, mc, nq, special = row
    rng = np.random.default_rng(seed + len(name))
    data = rng.standard_normal((N, d)).astype(np.float32)
    query = rng.standard_normal((nq, d)).astype(np.float32)
    if special == "round":
        data, query = np.round(data), np.round(query * 2) / 2
    if special == "identical":     # every key equal: the ordering falls back to the radix sort
        data[:] = data[0]
    if special == "clusters":      # two groups of identical points
        data[: N // 2] = data[0]
        data[N // 2:] = data[1]
    if special == "far":
        query[: nq // 2] *= 30.0
    return dict(name=name, data=np.ascontiguousarray(data), query=np.ascontiguousarray(query), L=L, S=S, P=P, T=T,
                k=k, outer=outer, max_cand=mc, proj=unit_rows(rng, L * S, d))
