// Query hot path: prioritized traversal, distances and per-partition top-k for
// one (query, partition) work item per CTA pass.
//
// The reference walks a partition with one sequential loop
// (dci_query_single_point_by_block, src/dci_cuda_kernel.cu:401-626): every
// outer iteration pops, per composite index, the simple index whose next
// T-wide window is nearest to the query (:466-478), bumps a counter for the T
// points of that window (:487-495), promotes a point when all S simple indices
// of a composite index have seen it (:494-555), and stops on a test of how many
// promotions lane 0 of the window has made (:598-607).
//
// The visiting order does not depend on the counters, only on the sorted keys:
// inside one composite index it is all windows of its S simple indices ordered
// by (priority, simple index, order inside the index).  So this kernel
//   1. finds every simple index's split position with a warp-wide 32-ary search
//      (replaces dci_search_index, :279-297),
//   2. enumerates all windows with their priorities (dci_next_closest_proj,
//      :250-273, and the priority rule :338-352, :572-590) and radix-sorts the
//      windows of each composite index: the rank of a window IS the outer
//      iteration in which the reference visits it,
//   3. for every point takes, per composite index, the largest rank among the
//      S windows that contain it (= the iteration of its S-th visit, i.e. its
//      promotion) with the lane it occupies in that window, and then the
//      smallest such rank over the composite indices (the first promotion wins,
//      :497),
//   4. derives the stop iteration from the order statistics of the promotion
//      iterations of lane-0 points (the reference's stop test), and
//   5. computes true distances of the points promoted up to the stop iteration
//      (compute_dist_device, :36-44, same summation order) and keeps the k
//      nearest (replaces the racy per-thread lists :513-553 and the Thrust sort
//      :691-701).
// All buffers of a work item live in shared memory when they fit, otherwise in
// a per-CTA slab of global scratch.
#pragma once
#include "common.cuh"

namespace dci {

struct TraverseParams {
    const float *skeys;        // [I][N] sorted keys
    const int *sids;           // [I][N] point ids
    const float *data;         // [N][dim]
    const float *qproj;        // [I][nq_total]
    const float *query;        // [nq_total][dim]
    uint64_t *part_topk;       // [nq][num_parts][knn]
    long long *work_stats;     // nullptr or [nq_total][P][6]
    unsigned char *gscratch;   // per-CTA slabs (global-scratch variant)
    size_t gscratch_per_cta;
    long long outer_s;         // num_outer_iterations * S
    int N, dim, L, S, P, T, ppb, num_parts;
    int nq, nq_total, q0;      // this launch covers queries [q0, q0 + nq)
    int knn, max_cand;
    int wcap;                  // capacity of one composite's window list
    int topk_cap;              // power of two >= knn + blockDim.x
    int tshift;                // bits that hold the lane in an encoded promotion
    int vec4;                  // rows of data/query can be read as float4
    FastDiv divT;
};

template <typename ValT>
struct TraverseLayout {
    // dynamic shared memory, always: [hist][qvec][topk buf]
    size_t hist_bytes, qvec_bytes, topk_bytes, fixed_bytes;
    // "big" region (shared or global): [rank tables][union(sort buffers, point arrays)]
    size_t rank_bytes, sortk_bytes, sortv_bytes, point_bytes, big_bytes;
    __host__ __device__ static size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }
    __host__ __device__ static TraverseLayout make(int nthreads, int dim, int topk_cap, int L,
                                                   int wcap, int ppb) {
        TraverseLayout l;
        l.hist_bytes = align16((size_t)256 * (nthreads / 32) * sizeof(ValT));
        l.qvec_bytes = align16((size_t)dim * 4);
        l.topk_bytes = align16((size_t)topk_cap * 8);
        l.fixed_bytes = l.hist_bytes + l.qvec_bytes + l.topk_bytes;
        l.rank_bytes = align16((size_t)L * wcap * sizeof(ValT));
        l.sortk_bytes = align16((size_t)wcap * 4);
        l.sortv_bytes = align16((size_t)wcap * sizeof(ValT));
        l.point_bytes = align16((size_t)ppb * 4);
        const size_t sort_total = 2 * l.sortk_bytes + 2 * l.sortv_bytes;
        const size_t point_total = 3 * l.point_bytes;
        l.big_bytes = l.rank_bytes + (sort_total > point_total ? sort_total : point_total);
        return l;
    }
};

// Sum of v over the CTA, returned to every thread.  scratch: 33 shared words.
__device__ __forceinline__ int cta_sum(int v, uint32_t *scratch) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    if (lane == 0) scratch[w] = (uint32_t)v;
    __syncthreads();
    if (w == 0) {
        int x = lane < nw ? (int)scratch[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, o);
        if (lane == 0) scratch[32] = (uint32_t)x;
    }
    __syncthreads();
    const int r = (int)scratch[32];
    __syncthreads();
    return r;
}

// Smallest v in [0, vmax] such that at least `kth` entries of list[0..cnt) are
// <= v (the kth smallest, 1-based).  Requires 1 <= kth <= cnt.
__device__ __forceinline__ uint32_t cta_kth_smallest(const uint32_t *list, int cnt, int kth,
                                                     uint32_t vmax, uint32_t *scratch) {
    uint32_t lo = 0, hi = vmax;
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        int c = 0;
        for (int j = threadIdx.x; j < cnt; j += blockDim.x) c += (list[j] <= mid);
        c = cta_sum(c, scratch);
        if (c >= kth) hi = mid; else lo = mid + 1;
    }
    return lo;
}

// Euclidean distance with the reference's summation order
// (compute_dist_device, src/dci_cuda_kernel.cu:36-44): sq = fma(d, d, sq) for
// ascending coordinate, then an IEEE square root.
__device__ __forceinline__ float dist_sequential(const float *__restrict__ row, const float *qv,
                                                 int dim, int vec4) {
    float sq = 0.0f;
    if (vec4) {
        const float4 *r4 = reinterpret_cast<const float4 *>(row);
        const float4 *q4 = reinterpret_cast<const float4 *>(qv);
        const int n4 = dim >> 2;
#pragma unroll 4
        for (int c = 0; c < n4; ++c) {
            const float4 a = __ldg(r4 + c);
            const float4 b = q4[c];
            float d = __fsub_rn(a.x, b.x); sq = __fmaf_rn(d, d, sq);
            d = __fsub_rn(a.y, b.y); sq = __fmaf_rn(d, d, sq);
            d = __fsub_rn(a.z, b.z); sq = __fmaf_rn(d, d, sq);
            d = __fsub_rn(a.w, b.w); sq = __fmaf_rn(d, d, sq);
        }
    } else {
        for (int c = 0; c < dim; ++c) {
            const float d = __fsub_rn(__ldg(row + c), qv[c]);
            sq = __fmaf_rn(d, d, sq);
        }
    }
    return __fsqrt_rn(sq);
}

template <typename ValT, bool SMEM>
__global__ void __launch_bounds__(1024, 1)
traverse_kernel(const TraverseParams prm) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ int s_pos[kMaxIndices];       // last position with key < q
    __shared__ int s_nl[kMaxIndices];        // number of left windows
    __shared__ int s_cnt[kMaxIndices];       // number of windows
    __shared__ int s_sp[kMaxIndices];        // 1: the only right window precedes the left ones
    __shared__ float s_qp[kMaxIndices];      // projected query
    __shared__ int s_woff[kMaxIndices + 64]; // per composite: S+1 window offsets
    __shared__ uint32_t s_scratch[40];
    __shared__ int s_count[2];
    __shared__ uint64_t s_thresh;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int L = prm.L, S = prm.S, T = prm.T, I = L * S, N = prm.N, dim = prm.dim;
    const TraverseLayout<ValT> lay =
        TraverseLayout<ValT>::make(blockDim.x, dim, prm.topk_cap, L, prm.wcap, prm.ppb);
    ValT *hist = reinterpret_cast<ValT *>(dyn_smem);
    float *qvec = reinterpret_cast<float *>(dyn_smem + lay.hist_bytes);
    uint64_t *topk_buf = reinterpret_cast<uint64_t *>(dyn_smem + lay.hist_bytes + lay.qvec_bytes);
    unsigned char *big = SMEM ? dyn_smem + lay.fixed_bytes
                              : prm.gscratch + (size_t)blockIdx.x * prm.gscratch_per_cta;
    ValT *rank = reinterpret_cast<ValT *>(big);
    unsigned char *uni = big + lay.rank_bytes;
    // sort view of the union region
    uint32_t *kA = reinterpret_cast<uint32_t *>(uni);
    uint32_t *kB = reinterpret_cast<uint32_t *>(uni + lay.sortk_bytes);
    ValT *vA = reinterpret_cast<ValT *>(uni + 2 * lay.sortk_bytes);
    ValT *vB = reinterpret_cast<ValT *>(uni + 2 * lay.sortk_bytes + lay.sortv_bytes);
    // point view of the union region
    uint32_t *kenc = reinterpret_cast<uint32_t *>(uni);                       // best promotion per point
    uint32_t *mr = reinterpret_cast<uint32_t *>(uni + lay.point_bytes);       // promotion in this composite
    uint32_t *list = reinterpret_cast<uint32_t *>(uni + 2 * lay.point_bytes); // lane-0 ranks, then candidates

    const uint32_t tmask = (1u << prm.tshift) - 1u;
    const long long nwork = (long long)prm.nq * prm.num_parts;

    for (long long wi = blockIdx.x; wi < nwork; wi += gridDim.x) {
        const int b = (int)(wi / prm.nq), ql = (int)(wi % prm.nq), q = prm.q0 + ql;
        const long long lo = (long long)b * prm.ppb;
        const int n = (int)min((long long)prm.ppb, (long long)N - lo);

        for (int i = tid; i < I; i += blockDim.x) s_qp[i] = prm.qproj[(size_t)i * prm.nq_total + q];
        for (int c = tid; c < dim; c += blockDim.x) qvec[c] = prm.query[(size_t)q * dim + c];
        __syncthreads();

        // ---- 1. split positions: warp-wide 32-ary lower bound per simple index
        for (int i = warp; i < I; i += nw) {
            const float *keys = prm.skeys + (size_t)i * N + lo;
            const float qv = s_qp[i];
            int lo_ = 0, hi_ = n;
            while (lo_ < hi_) {
                const int len = hi_ - lo_, chunk = (len + 31) >> 5;
                const int idx = lo_ + lane * chunk;
                const bool pred = idx < hi_ && keys[idx] < qv;
                const int c = __popc(__ballot_sync(0xFFFFFFFFu, pred));
                if (c == 0) {
                    hi_ = lo_;
                } else {
                    const int last = lo_ + (c - 1) * chunk;
                    lo_ = last + 1;
                    hi_ = min(hi_, last + chunk);
                }
            }
            if (lane == 0) {
                const int s = lo_ - 1;
                const int nl = (s + 1 + T - 1) / T;           // left starts s-T+1-jT > -T
                const int nr = (n + T - 2 - s + T - 1) / T;    // right starts s+1+jT < n+T-1
                s_pos[i] = s;
                s_nl[i] = nl;
                s_cnt[i] = nl + nr;
                s_sp[i] = (s == n - 1 && nr > 0) ? 1 : 0;
            }
        }
        __syncthreads();
        if (tid < L) {
            int acc = 0;
            for (int h = 0; h < S; ++h) { s_woff[tid * (S + 1) + h] = acc; acc += s_cnt[tid * S + h]; }
            s_woff[tid * (S + 1) + S] = acc;
        }
        __syncthreads();
        int maxW = 0;
        for (int m = 0; m < L; ++m) maxW = max(maxW, s_woff[m * (S + 1) + S]);

        // ---- 2. windows, priorities, visiting order of every composite index
        for (int m = 0; m < L; ++m) {
            const int *woff = s_woff + m * (S + 1);
            const int Wm = woff[S];
            for (int w = tid; w < Wm; w += blockDim.x) {
                int h = 0;
                while (w >= woff[h + 1]) ++h;
                const int i = m * S + h, t = w - woff[h];
                const int s = s_pos[i], nl = s_nl[i];
                bool right; int j;
                if (s_sp[i]) { right = (t == 0); j = right ? 0 : t - 1; }
                else { right = (t >= nl); j = right ? t - nl : t; }
                const int start = right ? s + 1 + j * T : s - T + 1 - j * T;
                const int kp = right ? min(start, n - 1) : max(start, 0);
                const float pri = fabsf(prm.skeys[(size_t)i * N + lo + kp] - s_qp[i]);
                kA[w] = __float_as_uint(pri);
                vA[w] = (ValT)w;
            }
            __syncthreads();
            cta_radix_sort<ValT, ValT, true>(kA, vA, kB, vB, Wm, hist, s_scratch, rank + (size_t)m * prm.wcap);
        }

        // ---- 3. promotion iteration and lane of every point
        for (int p = tid; p < n; p += blockDim.x) kenc[p] = 0xFFFFFFFFu;
        for (int m = 0; m < L; ++m) {
            const int *woff = s_woff + m * (S + 1);
            const ValT *rk = rank + (size_t)m * prm.wcap;
            for (int p = tid; p < n; p += blockDim.x) mr[p] = 0u;
            __syncthreads();
            for (int h = 0; h < S; ++h) {
                const int i = m * S + h;
                const int s = s_pos[i], nl = s_nl[i], sp = s_sp[i], base = woff[h];
                const int *ids = prm.sids + (size_t)i * N + lo;
                for (int y = tid; y < n; y += blockDim.x) {
                    const int p = ids[y] - (int)lo;
                    uint32_t wloc, t;
                    if (y <= s) {
                        const uint32_t x = (uint32_t)(s - y), j = prm.divT.div(x);
                        t = (uint32_t)(T - 1) - (x - j * (uint32_t)T);
                        wloc = sp ? 1u + j : j;
                    } else {
                        const uint32_t x = (uint32_t)(y - s - 1), j = prm.divT.div(x);
                        t = x - j * (uint32_t)T;
                        wloc = (uint32_t)nl + j;
                    }
                    const uint32_t r = (uint32_t)rk[base + wloc];
                    atomicMax(&mr[p], (r << prm.tshift) | t);
                }
            }
            __syncthreads();
            for (int p = tid; p < n; p += blockDim.x) {
                const uint32_t cur = kenc[p], v = mr[p];
                if ((v >> prm.tshift) < (cur >> prm.tshift)) kenc[p] = v;   // ties keep the lower composite
            }
            __syncthreads();
        }

        // ---- 4. stop iteration from lane-0 promotions (reference :598-607)
        if (tid == 0) { s_count[0] = 0; s_count[1] = 0; }
        __syncthreads();
        for (int p = tid; p < n; p += blockDim.x) {
            const uint32_t v = kenc[p];
            if ((v & tmask) == 0u) list[atomicAdd(&s_count[0], 1)] = v >> prm.tshift;
        }
        __syncthreads();
        const int cnt0 = s_count[0];
        const long long limit = (long long)n * S * T;
        long long stop = limit - 1;
        if (cnt0 >= prm.knn) {
            const long long a = cta_kth_smallest(list, cnt0, prm.knn, (uint32_t)maxW, s_scratch);
            const long long bcap = max(a, prm.outer_s - 1);
            long long ccap;
            if (prm.max_cand <= prm.knn) ccap = a;
            else if (cnt0 >= prm.max_cand)
                ccap = max(a, (long long)cta_kth_smallest(list, cnt0, prm.max_cand, (uint32_t)maxW, s_scratch));
            else ccap = limit;
            stop = min(min(bcap, ccap), limit - 1);
        }
        int lane0_stat = 0;
        if (prm.work_stats) {
            int c = 0;
            for (int j = tid; j < cnt0; j += blockDim.x) c += ((long long)list[j] <= stop);
            lane0_stat = cta_sum(c, s_scratch);
        }
        __syncthreads();
        for (int p = tid; p < n; p += blockDim.x) {
            if ((long long)(kenc[p] >> prm.tshift) <= stop) list[atomicAdd(&s_count[1], 1)] = (uint32_t)p;
        }
        __syncthreads();
        const int ncand = s_count[1];

        if (prm.work_stats) {
            long long visits = 0;
            int entries = 0;
            for (int m = 0; m < L; ++m) {
                const int *woff = s_woff + m * (S + 1);
                const int Wm = woff[S];
                visits += min((long long)Wm, stop + 1);
                const ValT *rk = rank + (size_t)m * prm.wcap;
                for (int w = tid; w < Wm; w += blockDim.x) {
                    if ((long long)rk[w] > stop) continue;
                    int h = 0;
                    while (w >= woff[h + 1]) ++h;
                    const int i = m * S + h, t = w - woff[h];
                    const int s = s_pos[i], nl = s_nl[i];
                    bool right; int j;
                    if (s_sp[i]) { right = (t == 0); j = right ? 0 : t - 1; }
                    else { right = (t >= nl); j = right ? t - nl : t; }
                    const int start = right ? s + 1 + j * T : s - T + 1 - j * T;
                    entries += max(0, min(start + T, n) - max(start, 0));
                }
            }
            entries = cta_sum(entries, s_scratch);
            if (tid == 0) {
                long long *st = prm.work_stats + ((size_t)q * prm.P + b) * 6;
                const bool exhausted = stop > (long long)maxW;
                st[0] = exhausted ? (long long)maxW : stop;
                st[1] = visits; st[2] = entries; st[3] = ncand; st[4] = lane0_stat; st[5] = exhausted ? 1 : 0;
            }
        }

        // ---- 5. distances of the promoted points and the partition's top-k
        CtaTopK topk;
        topk.init(topk_buf, &s_count[0], &s_thresh, prm.topk_cap, prm.knn);
        for (int base = 0; base < ncand; base += blockDim.x) {
            uint64_t key = kEmptySlot;
            const int j = base + tid;
            if (j < ncand) {
                const long long gid = lo + (long long)list[j];
                const float d = dist_sequential(prm.data + (size_t)gid * dim, qvec, dim, prm.vec4);
                key = ((uint64_t)__float_as_uint(d) << 32) | (uint32_t)gid;
            }
            topk.offer(key);
        }
        topk.finish();
        uint64_t *out = prm.part_topk + ((size_t)ql * prm.num_parts + b) * prm.knn;
        for (int j = tid; j < prm.knn; j += blockDim.x) out[j] = topk_buf[j];
        __syncthreads();
    }
}

// Final top-k of one query over the per-partition lists (replaces
// get_top_candidates, src/dci_cuda_kernel.cu:691-701).  One CTA per query.
__global__ void merge_partitions_kernel(const uint64_t *__restrict__ part_topk, int num_parts,
                                        int knn, int topk_cap, int q0, int *__restrict__ out_ids,
                                        float *__restrict__ out_dists) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ int s_count;
    __shared__ uint64_t s_thresh;
    uint64_t *buf = reinterpret_cast<uint64_t *>(dyn_smem);
    const int ql = blockIdx.x;
    const uint64_t *in = part_topk + (size_t)ql * num_parts * knn;
    const long long total = (long long)num_parts * knn;
    CtaTopK topk;
    topk.init(buf, &s_count, &s_thresh, topk_cap, knn);
    for (long long base = 0; base < total; base += blockDim.x) {
        const long long j = base + threadIdx.x;
        topk.offer(j < total ? in[j] : kEmptySlot);
    }
    topk.finish();
    for (int j = threadIdx.x; j < knn; j += blockDim.x) {
        const uint64_t key = buf[j];
        const size_t o = (size_t)(q0 + ql) * knn + j;
        if (key == kEmptySlot) {
            out_ids[o] = -1;
            out_dists[o] = __int_as_float(0x7F800000);
        } else {
            out_ids[o] = (int)(uint32_t)key;
            out_dists[o] = __uint_as_float((uint32_t)(key >> 32));
        }
    }
}

// Merge of per-shard result lists for MDCI (replaces the cat/sort/gather of
// dciknn_cuda/core.py:153-157).  One CTA per query.
struct ShardOffsets { long long v[64]; };

__global__ void merge_shards_kernel(const int *__restrict__ ids_in, const float *__restrict__ dists_in,
                                    int num_shards, int nq, int k, int topk_cap,
                                    const ShardOffsets offsets,
                                    long long *__restrict__ out_ids, float *__restrict__ out_dists) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ int s_count;
    __shared__ uint64_t s_thresh;
    uint64_t *buf = reinterpret_cast<uint64_t *>(dyn_smem);
    const int q = blockIdx.x;
    const long long total = (long long)num_shards * k;
    CtaTopK topk;
    topk.init(buf, &s_count, &s_thresh, topk_cap, k);
    for (long long base = 0; base < total; base += blockDim.x) {
        const long long j = base + threadIdx.x;
        uint64_t key = kEmptySlot;
        if (j < total) {
            const int s = (int)(j / k), r = (int)(j % k);
            const size_t src = ((size_t)s * nq + q) * k + r;
            const int id = ids_in[src];
            if (id >= 0) {
                const float d = dists_in[src];
                key = ((uint64_t)__float_as_uint(d) << 32) | (uint32_t)((long long)id + offsets.v[s]);
            }
        }
        topk.offer(key);
    }
    topk.finish();
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const uint64_t key = buf[j];
        const size_t o = (size_t)q * k + j;
        if (key == kEmptySlot) {
            out_ids[o] = -1;
            out_dists[o] = __int_as_float(0x7F800000);
        } else {
            out_ids[o] = (long long)(uint32_t)key;
            out_dists[o] = __uint_as_float((uint32_t)(key >> 32));
        }
    }
}

}  // namespace dci
