/*
 * dci_oracle.c -- TEST INFRASTRUCTURE ONLY.  Not part of the shipped library.
 *
 * A plain-C, single-work-item-at-a-time restatement of the Prioritized DCI
 * algorithm as the reference CUDA code executes it.  It exists so that the
 * CUDA path can be checked value by value; nothing in the product may call it.
 *
 * Every function cites the reference source it follows (paths are relative to
 * the reference project root).  The restatement deliberately keeps the
 * reference's sequential structure (one prioritized loop per partition) and is
 * therefore slow; the CUDA library uses a different, parallel formulation and
 * is compared against this one.
 *
 * Deliberate differences from the reference, all unobservable in its results
 * or documented in the tests:
 *   - the per-thread top-k scratch lists of src/dci_cuda_kernel.cu:513-553 are
 *     indexed there by (blockIdx.x + threadIdx.x) * k, so lists of different
 *     blocks overlap and race.  Here every promoted candidate takes part in
 *     one race-free global top-k ordered by (distance, id).
 *   - once every simple index of a partition is exhausted the reference keeps
 *     looping with no effect (:458, :481); here the loop leaves early.
 *   - equal projected keys are ordered by point id (the reference's quicksort,
 *     :206-235, leaves their order unspecified).
 *   - slots of the result that no candidate fills hold (+inf, -1); the
 *     reference leaves a stale id there (:691-701).
 *
 * Parity pin: the reference ships no tests or golden vectors.  This file is
 * pinned against outputs of the reference's own CUDA build (see
 * tests/golden/README.md and tests/test_oracle_golden.py).
 *
 * Arithmetic: fp32 throughout, no contraction except where written as fmaf
 * (build with -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- projection ---------------------------------------------------------
 * keys[i][p] = sum_k proj[i][k] * x[p][k], accumulated in fp32 with one fused
 * multiply-add per term, k ascending from an accumulator of +0.
 * Reference: util_kernel.cu:45-80 (cublasSgemm) called from
 * dci_cuda_kernel.cu:167-169 (data) and :802-803 (queries).  cuBLAS does not
 * document its summation order, so this order is this project's definition of
 * the "exact fp32" projection; the CUDA library's exact path uses the same one.
 */
int dci_oracle_project(const float *proj, const float *x, long long n, int dim,
                       int num_indices, float *out /* [num_indices][n] */) {
    if (!proj || !x || !out || n < 0 || dim <= 0 || num_indices <= 0) return -1;
#pragma omp parallel for schedule(static)
    for (long long p = 0; p < n; ++p) {
        const float *row = x + p * (long long)dim;
        for (int i = 0; i < num_indices; ++i) {
            const float *d = proj + (long long)i * dim;
            float acc = 0.0f;
            for (int k = 0; k < dim; ++k) acc = fmaf(d[k], row[k], acc);
            out[(long long)i * n + p] = acc;
        }
    }
    return 0;
}

/* ---- index build --------------------------------------------------------
 * Reference: copy_to_indices (dci_cuda_kernel.cu:132-146) fills {key, id} with
 * id = the row number inside this instance; sort_indices (:113-129) sorts
 * every (simple index, partition) segment ascending by key, the partition b
 * being the id range [b*ppb, min((b+1)*ppb, N)), ppb = ceil(N / P) (:178).
 */
typedef struct { float key; int id; } entry_t;

static int entry_cmp(const void *a, const void *b) {
    const entry_t *x = (const entry_t *)a, *y = (const entry_t *)b;
    if (x->key < y->key) return -1;
    if (x->key > y->key) return 1;
    return (x->id > y->id) - (x->id < y->id);
}

int dci_oracle_build(const float *keys_unsorted /* [I][N] */, int N, int I, int P,
                     float *skeys /* [I][N] */, int *sids /* [I][N] */) {
    if (!keys_unsorted || !skeys || !sids || N <= 0 || I <= 0 || P <= 0) return -1;
    int ppb = (N + P - 1) / P;
    int err = 0;
#pragma omp parallel for schedule(dynamic)
    for (int i = 0; i < I; ++i) {
        entry_t *buf = (entry_t *)malloc(sizeof(entry_t) * (size_t)ppb);
        if (!buf) { err = 1; continue; }
        for (int b = 0; b < P; ++b) {
            long long lo = (long long)b * ppb;
            long long n = (long long)N - lo;
            if (n > ppb) n = ppb;
            if (n <= 0) break;
            for (int x = 0; x < n; ++x) {
                buf[x].key = keys_unsorted[(long long)i * N + lo + x];
                buf[x].id = (int)(lo + x);
            }
            qsort(buf, (size_t)n, sizeof(entry_t), entry_cmp);
            for (int x = 0; x < n; ++x) {
                skeys[(long long)i * N + lo + x] = buf[x].key;
                sids[(long long)i * N + lo + x] = buf[x].id;
            }
        }
        free(buf);
    }
    return err ? -2 : 0;
}

/* ---- traversal helpers -------------------------------------------------- */

/* dci_search_index, dci_cuda_kernel.cu:279-297: position of the last key that
 * is < q, in -1..n-1. */
static int search_last_less(const float *keys, float q, int n) {
    int start = -1, end = n - 1, cur = (start + end + 2) / 2;
    while (start < end) {
        if (keys[cur] < q) start = cur; else end = cur - 1;
        cur = (start + end + 2) / 2;
    }
    return start;
}

/* dci_next_closest_proj, dci_cuda_kernel.cu:250-273.  T is blockDim.x there. */
static int next_window(const float *keys, int *left, int *right, float q, int n, int T) {
    int lb = -T, ub = n + T - 1, cur;
    if (*left <= lb && *right >= ub) {
        cur = lb;
    } else if (*left <= lb) {
        cur = *right; *right += T;
    } else if (*right >= ub) {
        cur = *left; *left -= T;
    } else {
        int r = *right < n - 1 ? *right : n - 1;
        int l = *left > 0 ? *left : 0;
        if (keys[r] - q < q - keys[l]) { cur = *right; *right += T; }
        else { cur = *left; *left -= T; }
    }
    return cur;
}

/* position used for the priority of a window, dci_cuda_kernel.cu:339-346 and
 * :572-580. */
static int clamp_pos(int cur, int n, int T) {
    if (cur < 0 && cur > -T) return 0;
    if (cur < n + T - 1 && cur >= n) return n - 1;
    return cur;
}

/* abs_d, dci_cuda_kernel.cu:47-49 */
static float abs_d(float x) { return x > 0 ? x : -x; }

/* compute_dist_device, dci_cuda_kernel.cu:36-44.  nvcc contracts
 * sq += d*d into one fused multiply-add; sqrt is the IEEE one. */
static float dist_seq(const float *a, const float *b, int dim) {
    float sq = 0.0f;
    for (int i = 0; i < dim; ++i) {
        float d = a[i] - b[i];
        sq = fmaf(d, d, sq);
    }
    return sqrtf(sq);
}

typedef struct {
    long long stop_iter;   /* value of the outer counter when the loop ended  */
    long long visits;      /* windows popped (including empty ones)           */
    long long entries;     /* in-range index entries looked at                */
    int candidates;        /* points promoted                                 */
    int lane0;             /* promotions that happened in lane 0              */
    int exhausted;         /* 1 if the loop ended because nothing was left    */
} work_stats_t;

/* One (query, partition) work item: dci_query_single_point_by_block,
 * dci_cuda_kernel.cu:401-626, for the partition whose segment starts at
 * column `lo` of every simple index and holds n points.  Marks promoted
 * points in cand[0..n) (indexed by id - lo). */
static void traverse_partition(const float *skeys, const int *sids, int N, int L, int S,
                               long long lo, int n, int T, const float *qproj /* [I] */,
                               int knn, long long outer, int max_cand,
                               unsigned char *cand, int *counts /* [L][n] scratch */,
                               int *left, int *right, int *cur, float *prio,
                               work_stats_t *st, long long *when /* optional [n]: iteration of promotion */) {
    int I = L * S;
    memset(cand, 0, (size_t)n);
    memset(counts, 0, sizeof(int) * (size_t)L * n);
    memset(st, 0, sizeof(*st));
    /* search_index :300-318 */
    for (int i = 0; i < I; ++i) {
        int s = search_last_less(skeys + (long long)i * N + lo, qproj[i], n);
        left[i] = s - T + 1;
        right[i] = left[i] + T;
    }
    /* init_index_priority :320-355 */
    for (int i = 0; i < I; ++i) {
        const float *keys = skeys + (long long)i * N + lo;
        cur[i] = next_window(keys, &left[i], &right[i], qproj[i], n, T);
        int pos = clamp_pos(cur[i], n, T);
        /* the reference asserts 0 <= pos < n here (:347-348) */
        prio[i] = abs_d(keys[pos] - qproj[i]);
    }
    int c0 = 0;
    long long k = 0;
    long long limit = (long long)n * S * T;      /* :458 */
    while (k < limit) {
        int any = 0;
        for (int m = 0; m < L; ++m) {
            /* :466-478, strict '<' so the lowest h wins ties; +inf never wins */
            float top = INFINITY; int top_h = -1;
            for (int h = 0; h < S; ++h) {
                if (prio[m * S + h] < top) { top = prio[m * S + h]; top_h = h; }
            }
            if (top_h < 0) continue;
            any = 1;
            int i = top_h + m * S;
            const float *keys = skeys + (long long)i * N + lo;
            const int *ids = sids + (long long)i * N + lo;
            int position = cur[i];
            st->visits++;
            for (int t = 0; t < T; ++t) {          /* lanes, :487-562 */
                int ci = position + t;
                if (ci < 0 || ci >= n) continue;
                int p = (int)(ids[ci] - lo);
                st->entries++;
                if (++counts[(long long)m * n + p] == S && !cand[p]) {
                    cand[p] = 1;
                    if (when) when[p] = k;
                    st->candidates++;
                    if (t == 0) { c0++; }
                }
            }
            /* :566-591 */
            cur[i] = next_window(keys, &left[i], &right[i], qproj[i], n, T);
            int pos = clamp_pos(cur[i], n, T);
            if (pos >= 0 && pos < n) {
                prio[i] = abs_d(keys[pos] - qproj[i]);
            } else {
                prio[i] = INFINITY;
                cur[i] = -T;
            }
        }
        /* :598-607, evaluated by lane 0 on its own promotion count */
        if (c0 >= knn) {
            if (k + 1 >= outer * S || c0 >= max_cand) break;
        }
        if (!any) { st->exhausted = 1; break; }
        k++;
    }
    st->stop_iter = k;
    st->lane0 = c0;
}

typedef struct { float dist; int id; } nn_t;

static int nn_cmp(const void *a, const void *b) {
    const nn_t *x = (const nn_t *)a, *y = (const nn_t *)b;
    if (x->dist < y->dist) return -1;
    if (x->dist > y->dist) return 1;
    return (x->id > y->id) - (x->id < y->id);
}

/*
 * dci_query, dci_cuda_kernel.cu:777-875, for nq queries over an index built
 * with P partitions and window width T.
 *   skeys/sids  [I][N]   sorted segments (dci_oracle_build)
 *   data        [N][dim] the indexed points
 *   qproj       [I][nq]  projected queries (dci_oracle_project layout)
 *   query       [nq][dim]
 *   out_ids/out_dists [nq][knn], rows ascending by (distance, id)
 *   stats       optional, [nq][P][6] long long:
 *               stop_iter, visits, entries, candidates, lane0, exhausted
 *   cand_mask   optional, [nq][N] bytes: 1 where the point was promoted
 */
int dci_oracle_query(const float *skeys, const int *sids, int N, int L, int S, int P, int T,
                     const float *data, int dim, const float *qproj, const float *query,
                     int nq, int knn, long long outer, int max_cand,
                     int *out_ids, float *out_dists, long long *stats,
                     unsigned char *cand_mask) {
    if (!skeys || !sids || !data || !qproj || !query || !out_ids || !out_dists) return -1;
    if (N <= 0 || L <= 0 || S <= 0 || P <= 0 || T <= 0 || dim <= 0 || nq < 0 || knn <= 0) return -1;
    int I = L * S;
    int ppb = (N + P - 1) / P;
    int err = 0;
#pragma omp parallel
    {
        unsigned char *cand = (unsigned char *)malloc((size_t)ppb);
        int *counts = (int *)malloc(sizeof(int) * (size_t)L * ppb);
        int *lr = (int *)malloc(sizeof(int) * 3 * (size_t)I);
        float *prio = (float *)malloc(sizeof(float) * (size_t)I);
        float *qp = (float *)malloc(sizeof(float) * (size_t)I);
        nn_t *list = (nn_t *)malloc(sizeof(nn_t) * (size_t)N);
        if (!cand || !counts || !lr || !prio || !qp || !list) {
#pragma omp atomic write
            err = 1;
        } else {
#pragma omp for schedule(dynamic)
            for (int q = 0; q < nq; ++q) {
                const float *qv = query + (long long)q * dim;
                for (int i = 0; i < I; ++i) qp[i] = qproj[(long long)i * nq + q];
                int cnt = 0;
                for (int b = 0; b < P; ++b) {
                    long long lo = (long long)b * ppb;
                    long long n = (long long)N - lo;
                    if (n > ppb) n = ppb;
                    work_stats_t st;
                    memset(&st, 0, sizeof(st));
                    if (n > 0) {
                        traverse_partition(skeys, sids, N, L, S, lo, (int)n, T, qp, knn, outer,
                                           max_cand, cand, counts, lr, lr + I, lr + 2 * I, prio, &st, NULL);
                        for (int x = 0; x < n; ++x) {
                            if (!cand[x]) continue;
                            int p = (int)(lo + x);
                            list[cnt].id = p;
                            list[cnt].dist = dist_seq(data + (long long)p * dim, qv, dim);
                            cnt++;
                            if (cand_mask) cand_mask[(long long)q * N + p] = 1;
                        }
                    }
                    if (stats) {
                        long long *s = stats + ((long long)q * P + b) * 6;
                        s[0] = st.stop_iter; s[1] = st.visits; s[2] = st.entries;
                        s[3] = st.candidates; s[4] = st.lane0; s[5] = st.exhausted;
                    }
                }
                qsort(list, (size_t)cnt, sizeof(nn_t), nn_cmp);
                for (int j = 0; j < knn; ++j) {
                    if (j < cnt) {
                        out_ids[(long long)q * knn + j] = list[j].id;
                        out_dists[(long long)q * knn + j] = list[j].dist;
                    } else {
                        out_ids[(long long)q * knn + j] = -1;
                        out_dists[(long long)q * knn + j] = INFINITY;
                    }
                }
            }
        }
        free(cand); free(counts); free(lr); free(prio); free(qp); free(list);
    }
    return err ? -2 : 0;
}

typedef struct { long long when; int id; } blind_t;

static int blind_cmp(const void *a, const void *b) {
    const blind_t *x = (const blind_t *)a, *y = (const blind_t *)b;
    if (x->when != y->when) return x->when < y->when ? -1 : 1;
    return (x->id > y->id) - (x->id < y->id);
}

/*
 * Blind querying as the reference's comments specify it (dci_cuda_kernel.cu:398-399, :775-776):
 * the same traversal with the same stop rule, no distance is computed and no indexed vector is
 * read; the result is the promoted points "in the order of retrieval".  Partitions are traversed
 * side by side (one CUDA block each, :843), so the order is defined here as ascending
 * (iteration of the partition's loop at which the point was promoted, point id).  The reference's
 * own blind path cannot be run (unsynchronised counter :498-505, host reads of device memory
 * :770-772), so this restatement is the specification, not a transcription.
 *   out_ids / out_when  [nq][width]; unused slots hold -1 / -1.
 */
int dci_oracle_query_blind(const float *skeys, const int *sids, int N, int L, int S, int P, int T,
                           const float *qproj, int nq, int knn, long long outer, int max_cand,
                           int width, int *out_ids, long long *out_when) {
    if (!skeys || !sids || !qproj || !out_ids) return -1;
    if (N <= 0 || L <= 0 || S <= 0 || P <= 0 || T <= 0 || nq < 0 || knn <= 0 || width <= 0) return -1;
    int I = L * S;
    int ppb = (N + P - 1) / P;
    int err = 0;
#pragma omp parallel
    {
        unsigned char *cand = (unsigned char *)malloc((size_t)ppb);
        int *counts = (int *)malloc(sizeof(int) * (size_t)L * ppb);
        int *lr = (int *)malloc(sizeof(int) * 3 * (size_t)I);
        float *prio = (float *)malloc(sizeof(float) * (size_t)I);
        float *qp = (float *)malloc(sizeof(float) * (size_t)I);
        long long *when = (long long *)malloc(sizeof(long long) * (size_t)ppb);
        blind_t *list = (blind_t *)malloc(sizeof(blind_t) * (size_t)N);
        if (!cand || !counts || !lr || !prio || !qp || !when || !list) {
#pragma omp atomic write
            err = 1;
        } else {
#pragma omp for schedule(dynamic)
            for (int q = 0; q < nq; ++q) {
                for (int i = 0; i < I; ++i) qp[i] = qproj[(long long)i * nq + q];
                int cnt = 0;
                for (int b = 0; b < P; ++b) {
                    long long lo = (long long)b * ppb;
                    long long n = (long long)N - lo;
                    if (n > ppb) n = ppb;
                    if (n <= 0) continue;
                    work_stats_t st;
                    traverse_partition(skeys, sids, N, L, S, lo, (int)n, T, qp, knn, outer, max_cand,
                                       cand, counts, lr, lr + I, lr + 2 * I, prio, &st, when);
                    for (int x = 0; x < n; ++x) {
                        if (!cand[x]) continue;
                        list[cnt].id = (int)(lo + x);
                        list[cnt].when = when[x];
                        cnt++;
                    }
                }
                qsort(list, (size_t)cnt, sizeof(blind_t), blind_cmp);
                for (int j = 0; j < width; ++j) {
                    out_ids[(long long)q * width + j] = j < cnt ? list[j].id : -1;
                    if (out_when) out_when[(long long)q * width + j] = j < cnt ? list[j].when : -1;
                }
            }
        }
        free(cand); free(counts); free(lr); free(prio); free(qp); free(when); free(list);
    }
    return err ? -2 : 0;
}

/* Exact brute-force k-NN with the same distance arithmetic and tie order,
 * used for recall figures in tests. */
int dci_oracle_bruteforce(const float *data, int N, int dim, const float *query, int nq,
                          int knn, int *out_ids, float *out_dists) {
    if (!data || !query || !out_ids || !out_dists || N <= 0 || dim <= 0 || knn <= 0) return -1;
    int err = 0;
#pragma omp parallel
    {
        nn_t *list = (nn_t *)malloc(sizeof(nn_t) * (size_t)N);
        if (!list) {
#pragma omp atomic write
            err = 1;
        } else {
#pragma omp for schedule(dynamic)
            for (int q = 0; q < nq; ++q) {
                for (int p = 0; p < N; ++p) {
                    list[p].id = p;
                    list[p].dist = dist_seq(data + (long long)p * dim, query + (long long)q * dim, dim);
                }
                qsort(list, (size_t)N, sizeof(nn_t), nn_cmp);
                for (int j = 0; j < knn; ++j) {
                    out_ids[(long long)q * knn + j] = j < N ? list[j].id : -1;
                    out_dists[(long long)q * knn + j] = j < N ? list[j].dist : INFINITY;
                }
            }
        }
        free(list);
    }
    return err ? -2 : 0;
}

int dci_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void dci_oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
