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
//      :250-273, and the priority rule :338-352, :572-590) and ranks the windows
//      of each composite index in that order (a counting rank over value
//      buckets; a stable radix sort when many priorities are equal): the rank of
//      a window IS the outer iteration in which the reference visits it,
//   3. for every point looks up (through the inverse permutation built by add)
//      the window that contains it in each simple index and takes, per
//      composite index, the largest rank among those S windows (= the iteration
//      of its S-th visit, i.e. its promotion) with the lane it occupies in that
//      window, and then the smallest such rank over the composite indices (the
//      first promotion wins, :497),
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
    // index arrays, partition-major: the segment of (partition b, simple index i) starts at
    // I * b * ppb + i * n_b, n_b = points of partition b (see segment_start in build_index.cuh)
    const float *skeys;        // sorted keys
    const float *skeysT;       // the same keys, every segment stride-T transposed
    const int *sids;           // point ids
    const void *spos;          // position of each point in its sorted segment (u16 or u32)
    const float *data;         // [N][dim]
    const float *qproj;        // [I][nq_total]
    const float *query;        // [nq_total][dim]
    uint64_t *part_topk;       // [nq][num_parts][knn]
    long long *work_stats;     // nullptr or [nq_total][P][6]
    long long *phase_cycles;   // nullptr or [16]: SM cycles summed over work items, per phase
    unsigned char *gscratch;   // per-CTA slabs
    size_t gscratch_per_cta;
    long long outer_s;         // num_outer_iterations * S
    int N, dim, L, S, P, T, ppb, num_parts;
    int nq, nq_total, q0;      // this launch covers queries [q0, q0 + nq)
    int knn, max_cand;
    int wcap;                  // capacity of one composite's window list
    int nbuckets;              // value buckets of the window ordering
    int bkey;                  // 1: the ordering keeps a bucket-ordered copy of the keys (needs wcap more words)
    int kpart;                 // length of a partition's result list: min(knn, ppb)
    int topk_cap;              // power of two >= kpart + blockDim.x
    int topk_global;           // 1: the top-k buffers live in the CTA's global slab (large k)
    size_t topk_global_off;    // their offset inside the slab
    int tshift;                // bits that hold the lane in an encoded promotion
    int vec4;                  // rows of data/query can be read as float4
    int vec8;                  // rows of data start on 32-byte boundaries: one full sector per load
    int qbatch;                // queries of one partition a CTA takes together (1..kMaxQBatch)
    int dense_cap;             // capacity of the dense pass's selection buffers: power of two >= kpart + blockDim/4
    uint32_t *qbound;          // nullptr or [nq]: per query of this launch, fp32 bits of an upper bound of its k-th
                               // smallest distance found so far (any partition); candidates beyond it are dropped
    int blind;                 // 1: no distances; a promoted point's key is its promotion iteration (needs topk_global)
    FastDiv divT;
};

constexpr int kMaxQBatch = 8;                  // queries whose exhaustive distance phases share row loads
constexpr int kPriWidth = 5;                   // window keys a thread loads together in the priority pass
constexpr int kDistChunk = 16;                 // floats of a row staged per step of the distance phase
constexpr int kDistStride = kDistChunk + 4;    // padded row stride of the staging tile (floats)

template <typename ValT>
struct TraverseLayout {
    // dynamic shared memory, always: [counters][qvec]
    size_t cnt_bytes, qvec_bytes, fixed_bytes;
    int nbuckets;
    // "big" region (shared or global): [rank table per composite][union]
    //   union, ordering view : kA u32[wcap] | bval ValT[wcap] | slot u8[wcap] | bkey u32[wcap]
    //   union, point view    : kenc u32[ppb] | ... | list ValT[ppb] at list_off
    //   union, distance view : top-k 2 x u64[topk_cap] | staging tiles | ... | list (kept)
    size_t rank_bytes, wk_bytes, wv_bytes, ws_bytes, point_bytes, list_bytes, topk_bytes, tile_bytes,
        list_off, big_bytes;
    // per-CTA global slab for the radix-sort fallback: 2 x u32[wcap] | 2 x ValT[wcap]
    size_t fallback_bytes;
    __host__ __device__ static size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }
    __host__ __device__ static TraverseLayout make(int nthreads, int dim, int topk_cap, int L,
                                                   int wcap, int ppb, int nbuckets, bool tiles, bool bkey) {
        TraverseLayout l;
        const size_t radix_hist = (size_t)256 * (nthreads / 32) * sizeof(ValT);
        l.nbuckets = nbuckets;
        const size_t bucket_cnt = sizeof(ValT) * (size_t)(nbuckets + 16);   // zero padding for vector scans
        l.cnt_bytes = align16(radix_hist > bucket_cnt ? radix_hist : bucket_cnt);
        l.qvec_bytes = align16((size_t)dim * 4);
        l.fixed_bytes = l.cnt_bytes + l.qvec_bytes;
        l.rank_bytes = align16((size_t)L * wcap * sizeof(ValT));
        l.wk_bytes = align16((size_t)wcap * 4);
        l.wv_bytes = align16((size_t)wcap * sizeof(ValT));
        l.ws_bytes = align16((size_t)wcap);
        l.point_bytes = align16((size_t)ppb * 4);
        l.list_bytes = align16((size_t)ppb * sizeof(ValT));
        l.topk_bytes = align16((size_t)topk_cap * 8) * 2;
        // staging tiles: shared-memory variant only, and only when rows cannot be read sector by sector
        l.tile_bytes = tiles ? (size_t)(nthreads / 32) * 32 * kDistStride * 4 : 0;
        const size_t need = l.topk_bytes + l.tile_bytes;
        l.list_off = l.point_bytes > need ? l.point_bytes : need;
        const size_t sort_total = (bkey ? 2 : 1) * l.wk_bytes + l.wv_bytes + l.ws_bytes;
        const size_t point_total = l.list_off + l.list_bytes;
        l.big_bytes = l.rank_bytes + (sort_total > point_total ? sort_total : point_total);
        l.fallback_bytes = 2 * l.wk_bytes + 2 * l.wv_bytes;
        return l;
    }
};

template <int V> struct IntTag { static constexpr int value = V; };
struct TrueTag { static constexpr bool value = true; };
struct FalseTag { static constexpr bool value = false; };

// Positions of two neighbouring points of one sorted segment, read with one load (the segment
// starts on an aligned boundary and its padding is zero, see pos_segment_start).  A pair that is
// not loaded reads as position 0.
template <typename PosT> struct PosPair;
template <> struct PosPair<uint16_t> {
    uint32_t w;
    __device__ __forceinline__ void load(const uint16_t *p, bool live) {
        w = live ? __ldg(reinterpret_cast<const uint32_t *>(p)) : 0u;
    }
    __device__ __forceinline__ uint32_t first() const { return w & 0xFFFFu; }
    __device__ __forceinline__ uint32_t second() const { return w >> 16; }
};
template <> struct PosPair<uint32_t> {
    uint2 w;
    __device__ __forceinline__ void load(const uint32_t *p, bool live) {
        w = live ? __ldg(reinterpret_cast<const uint2 *>(p)) : make_uint2(0u, 0u);
    }
    __device__ __forceinline__ uint32_t first() const { return w.x; }
    __device__ __forceinline__ uint32_t second() const { return w.y; }
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

// Same distance with one 256-bit load per step: each lane fetches one whole
// 32-byte sector of its own row (sm_100 has 256-bit global loads), so no bytes
// are fetched that the lane does not use and no shared staging is needed.
// Requires dim % 8 == 0 and rows on 32-byte boundaries.
// The partial sums only grow (every term is a square), so a row is abandoned -- the rest of it is
// not even loaded -- as soon as its sum exceeds bound_sq; the result is then -1.
__device__ __forceinline__ void ld_row8(const float *p, float (&a)[8]) {
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(a[0]), "=f"(a[1]), "=f"(a[2]), "=f"(a[3]), "=f"(a[4]), "=f"(a[5]), "=f"(a[6]), "=f"(a[7])
                 : "l"(p));
}
__device__ __forceinline__ float sq_accumulate8(float sq, const float (&a)[8], const float *q) {
    const float4 b0 = *reinterpret_cast<const float4 *>(q);
    const float4 b1 = *reinterpret_cast<const float4 *>(q + 4);
    float d = __fsub_rn(a[0], b0.x); sq = __fmaf_rn(d, d, sq);
    d = __fsub_rn(a[1], b0.y); sq = __fmaf_rn(d, d, sq);
    d = __fsub_rn(a[2], b0.z); sq = __fmaf_rn(d, d, sq);
    d = __fsub_rn(a[3], b0.w); sq = __fmaf_rn(d, d, sq);
    d = __fsub_rn(a[4], b1.x); sq = __fmaf_rn(d, d, sq);
    d = __fsub_rn(a[5], b1.y); sq = __fmaf_rn(d, d, sq);
    d = __fsub_rn(a[6], b1.z); sq = __fmaf_rn(d, d, sq);
    d = __fsub_rn(a[7], b1.w); sq = __fmaf_rn(d, d, sq);
    return sq;
}
__device__ __forceinline__ float dist_sequential_v8(const float *__restrict__ row, const float *qv, int dim,
                                                    float bound_sq) {
    float sq = 0.0f;
    const int n8 = dim >> 3;
    int c = 0;
    // two loads in flight per check: a check after every load would expose one memory latency per
    // 8 coordinates
    for (; c + 2 <= n8; c += 2) {
        if (sq > bound_sq) return -1.0f;
        float a[8], b[8];
        ld_row8(row + c * 8, a);
        ld_row8(row + c * 8 + 8, b);
        sq = sq_accumulate8(sq, a, qv + c * 8);
        sq = sq_accumulate8(sq, b, qv + c * 8 + 8);
    }
    if (c < n8 && !(sq > bound_sq)) {
        float a[8];
        ld_row8(row + c * 8, a);
        sq = sq_accumulate8(sq, a, qv + c * 8);
    }
    return sq > bound_sq ? -1.0f : __fsqrt_rn(sq);
}

// Packed fp32 arithmetic of sm_100: two independent IEEE operations per instruction, so the
// results are those of the scalar operations.
__device__ __forceinline__ float2 sub2(const float2 a, const float2 b) {
    unsigned long long r;
    asm("sub.rn.f32x2 %0, %1, %2;"
        : "=l"(r)
        : "l"(*reinterpret_cast<const unsigned long long *>(&a)), "l"(*reinterpret_cast<const unsigned long long *>(&b)));
    return *reinterpret_cast<float2 *>(&r);
}
__device__ __forceinline__ float2 fma2sq(const float2 d, const float2 acc) {      // d * d + acc
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %1, %2;"
        : "=l"(r)
        : "l"(*reinterpret_cast<const unsigned long long *>(&d)), "l"(*reinterpret_cast<const unsigned long long *>(&acc)));
    return *reinterpret_cast<float2 *>(&r);
}

// Same distances for 32 rows at a time by one warp: lane r owns row r.  The
// rows are read from global memory in 64-byte pieces, four lanes per piece so
// that every 32-byte sector fetched is used in full, staged through a padded
// shared tile, and each lane then walks its own row in ascending coordinate
// order, so the result has exactly the summation order of dist_sequential.
// Requires dim % 4 == 0 and 16-byte aligned rows.  `row_id` is this lane's row
// (any valid row for lanes without a candidate).
__device__ __forceinline__ float dist_rows_tiled(const float *__restrict__ data, long long row_id,
                                                 const float *qv, int dim, float *tile) {
    const int lane = threadIdx.x & 31;
    const int sub = lane & 3, rsel = lane >> 2;            // 4 lanes per 64-byte piece, 8 rows per load
    const float *src[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const long long rid = __shfl_sync(0xFFFFFFFFu, row_id, rsel + 8 * u);
        src[u] = data + (size_t)rid * dim + sub * 4;
    }
    float4 ld[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
        ld[u] = (sub * 4 < dim) ? __ldg(reinterpret_cast<const float4 *>(src[u])) : make_float4(0.f, 0.f, 0.f, 0.f);
    float sq = 0.0f;
    for (int c0 = 0; c0 < dim; c0 += kDistChunk) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
            *reinterpret_cast<float4 *>(tile + (rsel + 8 * u) * kDistStride + sub * 4) = ld[u];
        __syncwarp();
        const int cn = c0 + kDistChunk;
        if (cn < dim) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (cn + sub * 4 < dim) ld[u] = __ldg(reinterpret_cast<const float4 *>(src[u] + cn));
        }
        const float *mine = tile + lane * kDistStride;
#pragma unroll
        for (int k4 = 0; k4 < kDistChunk / 4; ++k4) {
            if (c0 + k4 * 4 < dim) {
                const float4 a = *reinterpret_cast<const float4 *>(mine + k4 * 4);
                const float4 b = *reinterpret_cast<const float4 *>(qv + c0 + k4 * 4);
                float d = __fsub_rn(a.x, b.x); sq = __fmaf_rn(d, d, sq);
                d = __fsub_rn(a.y, b.y); sq = __fmaf_rn(d, d, sq);
                d = __fsub_rn(a.z, b.z); sq = __fmaf_rn(d, d, sq);
                d = __fsub_rn(a.w, b.w); sq = __fmaf_rn(d, d, sq);
            }
        }
        __syncwarp();
    }
    return __fsqrt_rn(sq);
}

// Windows of one simple index are numbered in spatial order: window g covers the
// sorted positions [g*T - c, g*T - c + T), c = nl*T - s - 1, where s is the last
// position with key < q and nl the number of windows left of the query; windows
// g < nl lie left of the query, the others right.  The order in which the
// reference visits the windows of one index (used only to break ties between
// equal priorities): left windows from the nearest outwards, then right windows
// outwards -- except that the single right window that exists when every key is
// below the query comes first (its signed difference is negative,
// src/dci_cuda_kernel.cu:264-265).
__device__ __forceinline__ int window_visit_order(int g, int nl, int sp) {
    return g >= nl ? (sp ? 0 : g) : (nl - 1 - g + sp);
}

// BATCH: compile the query-group path (Q > 1 with the dense distance pass).  The host picks it
// when the configuration makes exhaustive work items likely; without it the kernel is the plain
// one-query-per-pass loop.
// LEAN: the instance for the common case -- distances wanted (not blind), selection buffers in shared
// memory, 256-bit row loads, T > 1, no work statistics and no phase counters -- so that the code of
// the rarer paths does not weigh on its register allocation and instruction cache.
template <typename ValT, typename PosT, bool SMEM, bool BATCH, bool LEAN = false>
__global__ void __launch_bounds__(1024, 1)
traverse_kernel(const TraverseParams prm) {
    const bool f_blind = LEAN ? false : prm.blind != 0;
    const bool f_topk_global = LEAN ? false : prm.topk_global != 0;
    const bool f_vec8 = LEAN ? true : prm.vec8 != 0;
    long long *const f_work_stats = LEAN ? nullptr : prm.work_stats;
    unsigned long long *const f_phase_cycles = LEAN ? nullptr : (unsigned long long *)prm.phase_cycles;
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ int s_pos[kMaxIndices];       // last position with key < q
    __shared__ int s_nl[kMaxIndices];        // number of left windows
    __shared__ int s_cnt[kMaxIndices];       // number of windows
    __shared__ int s_sp[kMaxIndices];        // 1: the only right window precedes the left ones
    __shared__ int2 s_cb[kMaxIndices];       // x: c (window 0 starts at -c), y: first window id in its composite
    __shared__ int s_kt[kMaxIndices];        // index into the stride-T keys of window 0's start (may be -1)
    __shared__ float s_qp[kMaxIndices];      // projected query
    __shared__ int s_woff[kMaxIndices + 64]; // per composite: S+1 window offsets
    __shared__ uint32_t s_scratch[40];
    __shared__ uint32_t s_sel[2][256];
    __shared__ uint32_t s_res[4];
    __shared__ uint32_t s_maxpri;
    __shared__ int s_count[2];
    __shared__ uint64_t s_thresh;
    __shared__ TopKSlot s_slot[kMaxQBatch];  // dense distance phase: one top-k per deferred query
    __shared__ float s_bd[kMaxQBatch], s_bsq[kMaxQBatch];   // ... and its distance bound (plain and squared)
    __shared__ int s_dense[kMaxQBatch];      // local query numbers deferred to the dense phase

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int L = prm.L, S = prm.S, T = prm.T, I = L * S, N = prm.N, dim = prm.dim;
    const TraverseLayout<ValT> lay =
        TraverseLayout<ValT>::make(blockDim.x, dim, f_topk_global ? 0 : prm.topk_cap, L, prm.wcap, prm.ppb,
                                   prm.nbuckets, SMEM && prm.vec4 && !f_vec8, prm.bkey != 0);
    ValT *cnt = reinterpret_cast<ValT *>(dyn_smem);                    // bucket counters / radix histogram
    float *qvec = reinterpret_cast<float *>(dyn_smem + lay.cnt_bytes);
    unsigned char *slab = prm.gscratch + (size_t)blockIdx.x * prm.gscratch_per_cta;
    unsigned char *big = SMEM ? dyn_smem + lay.fixed_bytes : slab + lay.fallback_bytes;
    ValT *rank = reinterpret_cast<ValT *>(big);
    unsigned char *uni = big + lay.rank_bytes;
    // ordering view of the union region
    uint32_t *kA = reinterpret_cast<uint32_t *>(uni);
    ValT *bval = reinterpret_cast<ValT *>(uni + lay.wk_bytes);
    uint8_t *slot = reinterpret_cast<uint8_t *>(uni + lay.wk_bytes + lay.wv_bytes);
    uint32_t *bkey = prm.bkey ? reinterpret_cast<uint32_t *>(uni + lay.wk_bytes + lay.wv_bytes + lay.ws_bytes)
                              : nullptr;                                                               // keys, bucket by bucket
    // radix-sort fallback buffers (global)
    uint32_t *fb_k0 = reinterpret_cast<uint32_t *>(slab);
    uint32_t *fb_k1 = reinterpret_cast<uint32_t *>(slab + lay.wk_bytes);
    ValT *fb_v0 = reinterpret_cast<ValT *>(slab + 2 * lay.wk_bytes);
    ValT *fb_v1 = reinterpret_cast<ValT *>(slab + 2 * lay.wk_bytes + lay.wv_bytes);
    // point view of the union region
    uint32_t *kenc = reinterpret_cast<uint32_t *>(uni);                       // best promotion per point
    ValT *list = reinterpret_cast<ValT *>(uni + lay.list_off);                // lane-0 ranks, then candidates
    // distance view
    uint64_t *topk_bufs = f_topk_global ? reinterpret_cast<uint64_t *>(slab + prm.topk_global_off)
                                          : reinterpret_cast<uint64_t *>(uni);   // over kenc, phase 5 only
    float *tiles = reinterpret_cast<float *>(uni + lay.topk_bytes);           // staging, shared variant only
    const PosT *spos = reinterpret_cast<const PosT *>(prm.spos);

    const uint32_t tmask = (1u << prm.tshift) - 1u;
    // A CTA takes Q consecutive queries of one partition together.  Queries whose traversal
    // promotes every point of the partition (the exhaustive case of the reference's stop rule) are
    // deferred and their distances computed in one pass that loads each row once for all of them.
    const int Q = BATCH ? (prm.qbatch > 0 ? prm.qbatch : 1) : 1;
    const int ngroups = (prm.nq + Q - 1) / Q;
    const long long nwork = (long long)ngroups * prm.num_parts;
    long long t_last = 0;
#define DCI_PHASE_MARK(slot_)                                                             \
    if (f_phase_cycles && tid == 0) {                                                   \
        const long long now_ = clock64();                                                 \
        atomicAdd(&f_phase_cycles[slot_], (unsigned long long)(now_ - t_last)); \
        t_last = now_;                                                                    \
    }

    for (long long wi = blockIdx.x; wi < nwork; wi += gridDim.x) {
      const int b = (int)(wi / ngroups), grp = (int)(wi % ngroups);
      const long long lo = (long long)b * prm.ppb;
      const int n = (int)min((long long)prm.ppb, (long long)N - lo);
      int ndense = 0;
      for (int jq = 0; jq < Q; ++jq) {
        const int ql = grp * Q + jq;
        if (ql >= prm.nq) break;
        const int q = prm.q0 + ql;
        if (f_phase_cycles && tid == 0) t_last = clock64();

        for (int i = tid; i < I; i += blockDim.x) s_qp[i] = prm.qproj[(size_t)i * prm.nq_total + q];
        for (int c = tid; c < dim; c += blockDim.x) qvec[c] = prm.query[(size_t)q * dim + c];
        if (tid == 0) { s_maxpri = 0u; s_count[0] = 0; s_count[1] = 0; }
        __syncthreads();

        // ---- 1. split positions: warp-wide 32-ary lower bound per simple index
        for (int i = warp; i < I; i += nw) {
            const float *keys = prm.skeys + segment_start(lo, i, I, n);
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
                const int c = nl * T - s - 1;                  // 0 <= c < T
                s_cb[i].x = c;
                const int r0 = c ? T - c : 0;                  // residue class of every window start
                s_kt[i] = r0 * (n / T) + min(r0, n % T) - (c ? 1 : 0);
                // no window priority exceeds the distance to the farthest key
                const float far = fmaxf(fabsf(keys[0] - qv), fabsf(keys[n - 1] - qv));
                atomicMax(&s_maxpri, __float_as_uint(far));
            }
        }
        __syncthreads();
        if (tid < L) {
            int acc = 0;
            for (int h = 0; h < S; ++h) {
                s_woff[tid * (S + 1) + h] = acc;
                s_cb[tid * S + h].y = acc;
                acc += s_cnt[tid * S + h];
            }
            s_woff[tid * (S + 1) + S] = acc;
        }
        __syncthreads();
        int maxW = 0;
        for (int m = 0; m < L; ++m) maxW = max(maxW, s_woff[m * (S + 1) + S]);
        const float maxpri = __uint_as_float(s_maxpri);
        const bool buckets_ok = maxpri > 0.0f && maxpri < 3.0e38f;
        const float scale = buckets_ok ? (float)lay.nbuckets / maxpri : 0.0f;
        const int last_bucket = lay.nbuckets - 1;
        DCI_PHASE_MARK(0)

        // ---- 2. windows, priorities, visiting order of every composite index
        for (int m = 0; m < L; ++m) {
            const int *woff = s_woff + m * (S + 1);
            const int Wm = woff[S];
            cta_zero16(cnt, lay.cnt_bytes);
            __syncthreads();
            DCI_PHASE_MARK(10)
            const int last_t = ((n - 1) % T) * (n / T) + min((n - 1) % T, n % T) + (n - 1) / T;
            // The threads are split among the simple indices, so that a thread keeps one index's
            // constants in registers and walks that index's windows, kPriWidth key loads in flight.
            // A bucket that grows beyond kMaxBucket is noticed by the arrival that exceeds it.
            int over = buckets_ok ? 0 : 1;
            {
                const int tpi = max(1, (int)blockDim.x / S), slots = (int)blockDim.x / tpi;
                const int sl = tid / tpi, r = tid - sl * tpi;
                if (sl < slots)
                for (int h = sl; h < S; h += slots) {
                    const int i = m * S + h;
                    const int cnt_i = s_cnt[i], c = s_cb[i].x, kt = s_kt[i], wbase = woff[h];
                    const float qp = s_qp[i];
                    const float *kT = prm.skeysT + segment_start(lo, i, I, n);
                    for (int g0 = r; g0 < cnt_i; g0 += tpi * kPriWidth) {
                        float kv[kPriWidth];
#pragma unroll
                        for (int u = 0; u < kPriWidth; ++u) {
                            const int g = g0 + u * tpi;
                            kv[u] = 0.0f;
                            if (g < cnt_i) {
                                // window starts are contiguous in the stride-T layout; the two clamped
                                // cases read the segment's first / last key
                                const int start = g * T - c;
                                const int at = start < 0 ? 0 : (start >= n ? last_t : kt + g);
                                kv[u] = __ldg(kT + at);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < kPriWidth; ++u) {
                            const int g = g0 + u * tpi;
                            if (g < cnt_i) {
                                const uint32_t bits = __float_as_uint(fabsf(kv[u] - qp));
                                const int w = wbase + g;
                                kA[w] = bits;
                                if (buckets_ok) {
                                    const uint32_t arrival = bucket_arrive(cnt, bucket_of(bits, scale, last_bucket));
                                    over |= (arrival >= (uint32_t)kMaxBucket);
                                    slot[w] = (uint8_t)min(arrival, 255u);
                                }
                            }
                        }
                    }
                }
            }
            over = __syncthreads_or(over);
            DCI_PHASE_MARK(1)
            ValT *rk = rank + (size_t)m * prm.wcap;
            if (!over) {
                const int *nlv = s_nl + m * S, *spv = s_sp + m * S;
                auto tie_less = [woff, nlv, spv](uint32_t a, uint32_t b2) {
                    int ha = 0, hb = 0;
                    while ((int)a >= woff[ha + 1]) ++ha;
                    while ((int)b2 >= woff[hb + 1]) ++hb;
                    if (ha != hb) return ha < hb;
                    return window_visit_order((int)a - woff[ha], nlv[ha], spv[ha]) <
                           window_visit_order((int)b2 - woff[ha], nlv[ha], spv[ha]);
                };
                auto mark = [&](int slot_) { DCI_PHASE_MARK(slot_) };
                auto bucket = [scale, last_bucket](uint32_t k) { return bucket_of(k, scale, last_bucket); };
                cta_bucket_place_and_rank<ValT, ValT>(kA, Wm, slot, bval, bkey, cnt, lay.nbuckets, bucket, s_scratch,
                                                      rk, tie_less, mark);
            } else {
                // many equal priorities: stable radix sort of the windows laid out in visiting order
                for (int h = 0; h < S; ++h) {
                    const int i = m * S + h, base = woff[h], nl = s_nl[i], sp = s_sp[i];
                    for (int g = tid; g < s_cnt[i]; g += blockDim.x) {
                        const int at = base + window_visit_order(g, nl, sp);
                        fb_k0[at] = kA[base + g];
                        fb_v0[at] = (ValT)(base + g);
                    }
                }
                __syncthreads();
                cta_radix_sort<ValT, ValT, true>(fb_k0, fb_v0, fb_k1, fb_v1, Wm, cnt,
                                                 s_scratch, rk);
            }
            DCI_PHASE_MARK(2)
        }

        // ---- 3. promotion iteration and lane of every point; lane-0 promotions listed
        // Each thread carries a few pairs of neighbouring points through all simple indices, so
        // that the per-index constants stay in registers, one load brings the positions of two points
        // and the loads of the next index are in flight while this one's ranks are looked up.
        const uint32_t tmul = 1u << prm.tshift;
        // one pass: this thread's kPairs pairs, pair j = points p0 + 2 * (j * blockDim + tid) and the next one
        // `pair_step` is twice the number of threads that take part (a multiple of 32); the others sit
        // the pass out, whole warps at a time.
        auto promote_pass = [&](auto t_is_one, auto pairs_tag, const int p0, const int pair_step) {
            constexpr bool kT1 = decltype(t_is_one)::value;
            constexpr int kPairs = decltype(pairs_tag)::value;
            const size_t pstride = (size_t)pos_stride(prm.ppb);
            if (2 * tid < pair_step) {
                const int pt = p0 + 2 * tid;                       // first point of this thread's pair 0
                uint32_t best[2 * kPairs];
#pragma unroll
                for (int j = 0; j < 2 * kPairs; ++j) best[j] = 0xFFFFFFFFu;
                // 16-bit ranks and positions with windows of several points: the running maximum keeps
                // the rank in its high half and the relative position (below 65536: the host uses
                // 16-bit positions only while ppb + T <= 65536) in its low half.  The windows of one
                // composite index have distinct ranks, so the largest packed word is the largest
                // rank, and the lane (position mod T) is worked out once per composite from the
                // winner's position.  Two simple indices per trip: the loads of one are in flight
                // while the other's ranks are looked up, without register moves.
                constexpr bool kPacked = !BATCH && !kT1 && sizeof(PosT) == 2 && sizeof(ValT) == 2;   // (the query-group variants have no registers to spare)
                if constexpr (kPacked) {
                    unsigned livemask = 0;
#pragma unroll
                    for (int j = 0; j < kPairs; ++j) livemask |= (pt + j * pair_step < n) ? (1u << j) : 0u;
                    for (int m = 0; m < L; ++m) {
                        const uint16_t *rkm = reinterpret_cast<const uint16_t *>(rank) + (size_t)m * prm.wcap;
                        const uint16_t *rp = reinterpret_cast<const uint16_t *>(spos) + pos_segment_start(b, m * S, I, prm.ppb) + pt;
                        uint32_t mx[2 * kPairs];
#pragma unroll
                        for (int j = 0; j < 2 * kPairs; ++j) mx[j] = 0u;
                        uint32_t wa[kPairs], wb[kPairs];
#pragma unroll
                        for (int j = 0; j < kPairs; ++j)
                            wa[j] = ((livemask >> j) & 1u) ? __ldg(reinterpret_cast<const uint32_t *>(rp + j * pair_step)) : 0u;
                        auto lookups = [&](const uint32_t (&pw)[kPairs], const int h) {
                            const int2 cb = s_cb[m * S + h];
                            const uint16_t *rkb = rkm + cb.y;
                            const uint32_t c2 = (uint32_t)cb.x * 0x10001u;
#pragma unroll
                            for (int j = 0; j < kPairs; ++j) {
                                const uint32_t w2 = pw[j] + c2;        // both positions made relative to window 0 at once
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const uint32_t x = e ? (w2 >> 16) : (w2 & 0xFFFFu);
                                    const uint32_t g = __umulhi(x, prm.divT.magic);
                                    mx[2 * j + e] = max(mx[2 * j + e], ((uint32_t)rkb[g] << 16) | x);
                                }
                            }
                        };
                        int h = 0;
                        for (; h + 2 <= S; h += 2) {
                            rp += pstride;
#pragma unroll
                            for (int j = 0; j < kPairs; ++j)
                                wb[j] = ((livemask >> j) & 1u) ? __ldg(reinterpret_cast<const uint32_t *>(rp + j * pair_step)) : 0u;
                            lookups(wa, h);
                            if (h + 2 < S) {
                                rp += pstride;
#pragma unroll
                                for (int j = 0; j < kPairs; ++j)
                                    wa[j] = ((livemask >> j) & 1u) ? __ldg(reinterpret_cast<const uint32_t *>(rp + j * pair_step)) : 0u;
                            }
                            lookups(wb, h + 1);
                        }
                        if (h < S) lookups(wa, h);
#pragma unroll
                        for (int j = 0; j < 2 * kPairs; ++j) {
                            if ((mx[j] >> 16) < (best[j] >> prm.tshift)) {     // ties keep the lower composite
                                const uint32_t x = mx[j] & 0xFFFFu, g = __umulhi(x, prm.divT.magic);
                                best[j] = (mx[j] >> 16) * tmul + (x - g * (uint32_t)T);
                            }
                        }
                    }
                } else {
                for (int m = 0; m < L; ++m) {
                    const ValT *rkm = rank + (size_t)m * prm.wcap;
                    const PosT *row = spos + pos_segment_start(b, m * S, I, prm.ppb) + pt;
                    uint32_t mx[2 * kPairs];
#pragma unroll
                    for (int j = 0; j < 2 * kPairs; ++j) mx[j] = 0u;
                    PosPair<PosT> cur[kPairs], nxt[kPairs];
#pragma unroll
                    for (int j = 0; j < kPairs; ++j) cur[j].load(row + j * pair_step, pt + j * pair_step < n);
                    for (int h = 0; h < S; ++h) {
                        if (h + 1 < S) {
#pragma unroll
                            for (int j = 0; j < kPairs; ++j)
                                nxt[j].load(row + (size_t)(h + 1) * pstride + j * pair_step, pt + j * pair_step < n);
                        }
                        const int2 cb = s_cb[m * S + h];
                        const ValT *rkb = rkm + cb.y;
#pragma unroll
                        for (int j = 0; j < kPairs; ++j) {
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const uint32_t x = (e ? cur[j].second() : cur[j].first()) + (uint32_t)cb.x;   // position relative to window 0
                                uint32_t enc;
                                if (kT1) {
                                    enc = (uint32_t)rkb[x];
                                } else {
                                    const uint32_t g = __umulhi(x, prm.divT.magic);
                                    const uint32_t t = x - g * (uint32_t)T;
                                    enc = (uint32_t)rkb[g] * tmul + t;
                                }
                                mx[2 * j + e] = max(mx[2 * j + e], enc);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < kPairs; ++j) cur[j] = nxt[j];
                    }
#pragma unroll
                    for (int j = 0; j < 2 * kPairs; ++j)
                        if ((mx[j] >> prm.tshift) < (best[j] >> prm.tshift)) best[j] = mx[j];   // ties keep the lower composite
                }
                }
                // one reservation per warp for the lane-0 promotions of all its points (every warp of
                // the CTA appends to the same counter)
                unsigned m0[2 * kPairs];
                int total0 = 0;
#pragma unroll
                for (int j = 0; j < 2 * kPairs; ++j) {
                    const int p = pt + (j >> 1) * pair_step + (j & 1);
                    const bool live = p < n;
                    if (live) kenc[p] = best[j];
                    m0[j] = __ballot_sync(0xFFFFFFFFu, live && (best[j] & tmask) == 0u);
                    total0 += __popc(m0[j]);
                }
                int base0 = 0;
                if (lane == 0 && total0) base0 = atomicAdd(&s_count[0], total0);
                base0 = __shfl_sync(0xFFFFFFFFu, base0, 0);
#pragma unroll
                for (int j = 0; j < 2 * kPairs; ++j) {
                    if ((m0[j] >> lane) & 1u) list[base0 + __popc(m0[j] & lanemask_lt())] = (ValT)(best[j] >> prm.tshift);
                    base0 += __popc(m0[j]);
                }
            }
        };
        // a pass of several pairs per thread while the points still to do fill most of it, passes of
        // one pair for the rest and for small partitions (32-bit positions take two registers a pair,
        // so their large pass has fewer pairs; so has the one for T = 1, whose five-pair instance
        // made the compiler spill registers in the instance that every T > 1 uses)
        auto promote = [&](auto t_is_one) {
            const int pair_step = 2 * (int)blockDim.x;
            for (int p0 = 0; p0 < n;) {
                const int units = (n - p0 + pair_step - 1) / pair_step;
                // pairs of the large pass; none where the registers are needed elsewhere (query groups)
                constexpr int kBig = BATCH ? 0 : ((decltype(t_is_one)::value || sizeof(PosT) != 2) ? 2 : (SMEM ? 5 : 4));
                if (kBig > 1 && units >= 2) {
                    // a full pass, or for a short rest the same pass by as many warps as it takes
                    int step = pair_step;
                    if (units < kBig - 1) step = 2 * ((((n - p0 + 1) / 2 + kBig - 1) / max(kBig, 1) + 31) & ~31);
                    promote_pass(t_is_one, IntTag<(kBig > 1 ? kBig : 1)>{}, p0, step);
                    p0 += kBig * step;
                } else { promote_pass(t_is_one, IntTag<1>{}, p0, pair_step); p0 += pair_step; }
            }
        };
        if (!LEAN && T == 1) promote(TrueTag{}); else promote(FalseTag{});
        __syncthreads();

        DCI_PHASE_MARK(3)
        // ---- 4. stop iteration from lane-0 promotions (reference :598-607)
        const int cnt0 = s_count[0];
        const long long limit = (long long)n * S * T;
        long long stop = limit - 1;
        long long stop_rule = 0x7FFFFFFFFFFFFFFFll;      // iteration at which the stop test fires (statistics)
        if (cnt0 >= prm.knn) {
            const bool need_c = prm.max_cand > prm.knn && cnt0 >= prm.max_cand;
            int bits = 1;
            while ((1 << bits) <= maxW && bits < 31) ++bits;
            uint32_t sel[2];
            const ValT *lst = list;
            cta_select2([lst](int j) { return (uint32_t)lst[j]; }, cnt0, prm.knn,
                        need_c ? prm.max_cand : prm.knn, bits, s_sel, s_res, sel);
            const long long a = sel[0];
            const long long bcap = max(a, prm.outer_s - 1);
            long long ccap;
            if (prm.max_cand <= prm.knn) ccap = a;
            else if (need_c) ccap = max(a, (long long)sel[1]);
            else ccap = limit;
            stop_rule = min(bcap, ccap);
            stop = min(stop_rule, limit - 1);
        }
        int lane0_stat = 0;
        if (f_work_stats) {
            int c = 0;
            for (int j = tid; j < cnt0; j += blockDim.x) c += ((long long)list[j] <= stop);
            lane0_stat = cta_sum(c, s_scratch);
        }
        __syncthreads();
        // candidates = points promoted no later than `stop`; a warp reserves list slots for eight
        // rounds of its points at once (all warps append to one counter)
        const uint32_t stop_enc = stop >= (long long)(0xFFFFFFFFu >> prm.tshift) ? 0xFFFFFFFFu
                                                                                 : (((uint32_t)stop + 1u) << prm.tshift) - 1u;
        for (int p0 = 0; p0 < n; p0 += 8 * blockDim.x) {
            unsigned mk[8];
            int tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int p = p0 + j * blockDim.x + tid;
                mk[j] = __ballot_sync(0xFFFFFFFFu, p < n && kenc[p] <= stop_enc);
                tot += __popc(mk[j]);
            }
            int base = 0;
            if (lane == 0 && tot) base = atomicAdd(&s_count[1], tot);
            base = __shfl_sync(0xFFFFFFFFu, base, 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if ((mk[j] >> lane) & 1u) list[base + __popc(mk[j] & lanemask_lt())] = (ValT)(p0 + j * blockDim.x + tid);
                base += __popc(mk[j]);
            }
        }
        __syncthreads();
        const int ncand = s_count[1];

        if (f_work_stats) {
            long long visits = 0;
            int entries = 0;
            for (int m = 0; m < L; ++m) {
                const int *woff = s_woff + m * (S + 1);
                visits += min((long long)woff[S], stop + 1);
                const ValT *rk = rank + (size_t)m * prm.wcap;
                for (int h = 0; h < S; ++h) {
                    const int i = m * S + h, base = woff[h], c = s_cb[i].x;
                    for (int g = tid; g < s_cnt[i]; g += blockDim.x) {
                        if ((long long)rk[base + g] > stop) continue;
                        const int start = g * T - c;
                        entries += max(0, min(start + T, n) - max(start, 0));
                    }
                }
            }
            entries = cta_sum(entries, s_scratch);
            if (tid == 0) {
                long long *st = f_work_stats + ((size_t)q * prm.P + b) * 6;
                // the reference's loop runs out of windows at iteration maxW unless its stop test or its
                // iteration bound ends it first
                const bool exhausted = stop_rule > (long long)maxW && (long long)maxW < limit;
                st[0] = exhausted ? (long long)maxW : stop;
                st[1] = visits; st[2] = entries; st[3] = ncand; st[4] = lane0_stat; st[5] = exhausted ? 1 : 0;
            }
        }

        DCI_PHASE_MARK(4)
        if (BATCH && Q > 1 && ncand == n) {   // every point promoted: distances in the shared pass below
            if (tid == 0) {
                s_dense[ndense] = ql;
                if (f_phase_cycles) atomicAdd(&f_phase_cycles[15], 1ull);
            }
            ++ndense;
            __syncthreads();
            continue;
        }
        // ---- 5. distances of the promoted points and the partition's top-k
        // Only the query's k nearest candidates over all partitions reach the result, and the k-th
        // best of any one partition bounds that distance from above: candidates farther than the
        // best such bound published so far can be dropped (strictly farther, so ties are kept).
        // Which partitions have published depends on timing; the merged result does not.
        float bound_d = __int_as_float(0x7F800000), bound_sq = bound_d;
        if (prm.qbound && !f_blind) {
            const uint32_t bb = *reinterpret_cast<volatile uint32_t *>(prm.qbound + ql);
            if (bb < 0x7F7F7F7Fu) {                                  // the buffer starts as 0x7F7F7F7F: no bound yet
                bound_d = __uint_as_float(bb);
                const float up = __uint_as_float(bb + 1u);           // next float above the bound
                bound_sq = __fmul_ru(up, up);                        // sq > bound_sq  =>  sqrt(sq) > bound_d
            }
        }
        CtaTopK topk;
        topk.init(topk_bufs, &s_count[0], &s_thresh, s_sel, s_res, prm.topk_cap, prm.kpart);
        for (int base = 0; base < ncand; base += blockDim.x) {
            uint64_t key = kEmptySlot;
            const int j = base + tid;
            if (f_blind) {             // blind querying (reference :398-399): order of retrieval, no row is read
                if (j < ncand) {
                    const uint32_t p = (uint32_t)list[j];
                    key = ((uint64_t)(kenc[p] >> prm.tshift) << 32) | (uint32_t)(lo + p);
                }
            } else if (f_vec8) {
                if (j < ncand) {
                    const long long gid = lo + (long long)list[j];
                    const float d = dist_sequential_v8(prm.data + (size_t)gid * dim, qvec, dim, bound_sq);
                    if (d >= 0.0f && d <= bound_d) key = ((uint64_t)__float_as_uint(d) << 32) | (uint32_t)gid;
                }
            } else if (SMEM && prm.vec4) {
                const long long gid = lo + (long long)list[j < ncand ? j : 0];
                const float d = dist_rows_tiled(prm.data, gid, qvec, dim, tiles + warp * (32 * kDistStride));
                if (j < ncand && d <= bound_d) key = ((uint64_t)__float_as_uint(d) << 32) | (uint32_t)gid;
            } else if (j < ncand) {
                const long long gid = lo + (long long)list[j];
                const float d = dist_sequential(prm.data + (size_t)gid * dim, qvec, dim, prm.vec4);
                if (d <= bound_d) key = ((uint64_t)__float_as_uint(d) << 32) | (uint32_t)gid;
            }
            DCI_PHASE_MARK(5)
            topk.offer(key);
            DCI_PHASE_MARK(6)
        }
        topk.finish();
        uint64_t *out = prm.part_topk + ((size_t)ql * prm.num_parts + b) * prm.kpart;
        const uint64_t *res = topk.result();
        for (int j = tid; j < prm.kpart; j += blockDim.x) out[j] = res[j];
        if (tid == 0 && prm.qbound && !f_blind && prm.kpart == prm.knn && res[prm.knn - 1] != kEmptySlot)
            atomicMin(prm.qbound + ql, (uint32_t)(res[prm.knn - 1] >> 32));
        __syncthreads();
        DCI_PHASE_MARK(6)
        if (f_phase_cycles && tid == 0) atomicAdd(&f_phase_cycles[15], 1ull);
      }   // queries of the group

      // ---- 5'. dense distance pass for the deferred queries (host enables Q > 1 only with
      // 256-bit row loads, shared-memory buffers and room for Q selection buffer pairs)
      if (BATCH && ndense > 0) {
        if (f_phase_cycles && tid == 0) t_last = clock64();
        const size_t tk_bytes = (size_t)prm.dense_cap * 16;                      // two halves of u64[dense_cap]
        // the query vectors coordinate-major, kMaxQBatch slots per coordinate: one 128-bit load brings
        // one coordinate of four queries, i.e. two packed operands
        float *dq = reinterpret_cast<float *>(big + (size_t)Q * tk_bytes);
        for (int e = tid; e < dim * kMaxQBatch; e += blockDim.x) {
            const int t = e % kMaxQBatch, c = e / kMaxQBatch;
            dq[e] = t < ndense ? prm.query[(size_t)(prm.q0 + s_dense[t]) * dim + c] : 0.0f;
        }
        if (tid < ndense) {
            const int t = tid;
            s_slot[t].count = 0; s_slot[t].half = 0; s_slot[t].thresh = kEmptySlot;
            float bd = __int_as_float(0x7F800000), bsq = bd;     // the query's bound, as in phase 5
            if (prm.qbound) {
                const uint32_t bb = *reinterpret_cast<volatile uint32_t *>(prm.qbound + s_dense[t]);
                if (bb < 0x7F7F7F7Fu) {
                    bd = __uint_as_float(bb);
                    const float up = __uint_as_float(bb + 1u);
                    bsq = __fmul_ru(up, up);
                }
            }
            s_bd[t] = bd; s_bsq[t] = bsq;
        }
        __syncthreads();
        const int n8 = dim >> 3;
        for (int base = 0; base < n; base += blockDim.x) {
            const int r = base + tid;
            const bool live = r < n;
            float2 sq2[kMaxQBatch / 2];          // the sums of queries 2j and 2j + 1, each in the reference's order
#pragma unroll
            for (int t = 0; t < kMaxQBatch / 2; ++t) sq2[t] = make_float2(0.0f, 0.0f);
            if (live) {
                const float *row = prm.data + (size_t)(lo + r) * dim;
                for (int c = 0; c < n8; ++c) {
                    if ((c & 3) == 0 && c) {     // every 32 coordinates: is the row still within some query's bound?
                        bool any = false;
#pragma unroll
                        for (int t = 0; t < kMaxQBatch; ++t)
                            any |= (t < ndense && ((t & 1) ? sq2[t >> 1].y : sq2[t >> 1].x) <= s_bsq[t]);
                        if (!any) break;
                    }
                    float a[8];
                    ld_row8(row + c * 8, a);
                    const float4 *qc = reinterpret_cast<const float4 *>(dq + (size_t)c * 8 * kMaxQBatch);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float2 ab = make_float2(a[e], a[e]);
#pragma unroll
                        for (int h4 = 0; h4 < kMaxQBatch / 4; ++h4) {
                            if (4 * h4 < ndense) {               // the same for every thread
                                const float4 b = qc[e * (kMaxQBatch / 4) + h4];
                                sq2[2 * h4] = fma2sq(sub2(ab, make_float2(b.x, b.y)), sq2[2 * h4]);
                                if (4 * h4 + 2 < ndense) sq2[2 * h4 + 1] = fma2sq(sub2(ab, make_float2(b.z, b.w)), sq2[2 * h4 + 1]);
                            }
                        }
                    }
                }
            }
            float sq[kMaxQBatch];
#pragma unroll
            for (int t = 0; t < kMaxQBatch; ++t) sq[t] = (t & 1) ? sq2[t >> 1].y : sq2[t >> 1].x;
            DCI_PHASE_MARK(5)
            // the keys of a round are offered a quarter of the CTA at a time, so that a selection
            // buffer only needs room for blockDim/4 appends
            const int quarter = blockDim.x >> 2;
#pragma unroll
            for (int t = 0; t < kMaxQBatch; ++t) {
                if (t < ndense) {
                    uint64_t *bufs = reinterpret_cast<uint64_t *>(big + (size_t)t * tk_bytes);
                    CtaTopK topk = topk_slot_open(&s_slot[t], bufs, s_sel, s_res, prm.dense_cap, prm.kpart);
                    const float dfin = __fsqrt_rn(sq[t]);
                    const uint64_t key = (live && sq[t] <= s_bsq[t] && dfin <= s_bd[t])
                                             ? (((uint64_t)__float_as_uint(dfin) << 32) | (uint32_t)(lo + r)) : kEmptySlot;
                    for (int part = 0; part < 4; ++part)
                        topk.offer_from((tid / quarter) == part ? key : kEmptySlot, quarter);
                    topk_slot_close(&s_slot[t], topk, bufs);
                }
            }
            DCI_PHASE_MARK(6)
        }
        for (int t = 0; t < ndense; ++t) {
            uint64_t *bufs = reinterpret_cast<uint64_t *>(big + (size_t)t * tk_bytes);
            CtaTopK topk = topk_slot_open(&s_slot[t], bufs, s_sel, s_res, prm.dense_cap, prm.kpart);
            topk.finish();
            uint64_t *out = prm.part_topk + ((size_t)s_dense[t] * prm.num_parts + b) * prm.kpart;
            const uint64_t *res = topk.result();
            for (int j = tid; j < prm.kpart; j += blockDim.x) out[j] = res[j];
            if (tid == 0 && prm.qbound && prm.kpart == prm.knn && res[prm.knn - 1] != kEmptySlot)
                atomicMin(prm.qbound + s_dense[t], (uint32_t)(res[prm.knn - 1] >> 32));
            __syncthreads();
        }
        DCI_PHASE_MARK(6)
      }
    }
#undef DCI_PHASE_MARK
}

// Final top-k of a query over its per-partition lists (replaces
// get_top_candidates, src/dci_cuda_kernel.cu:691-701).  CTAs loop over queries.
// The selection buffers are dynamic shared memory, or -- for large k -- the
// CTA's slab of `gbufs` (2 * topk_cap entries each).
// blind: the high word of a key is a promotion iteration; out_dists then receives int32 values
// (-1 in empty slots) and may be null.
// out_packed (may be null; then out_ids is written): the merged keys themselves, (fp32 distance bits
// << 32 | id), kEmptySlot in unused slots -- the form in which MDCI ships a shard's lists.
__global__ void merge_partitions_kernel(const uint64_t *__restrict__ part_topk, int num_parts, int kpart,
                                        int knn, int topk_cap, int q0, int nq, uint64_t *gbufs,
                                        int *__restrict__ out_ids, float *__restrict__ out_dists, int blind,
                                        uint64_t *__restrict__ out_packed = nullptr) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ int s_count;
    __shared__ uint64_t s_thresh;
    __shared__ uint32_t s_sel[2][256];
    __shared__ uint32_t s_res[4];
    uint64_t *bufs = gbufs ? gbufs + (size_t)blockIdx.x * 2 * topk_cap : reinterpret_cast<uint64_t *>(dyn_smem);
    const long long total = (long long)num_parts * kpart;
    for (int ql = blockIdx.x; ql < nq; ql += gridDim.x) {
        const uint64_t *in = part_topk + (size_t)ql * total;
        CtaTopK topk;
        topk.init(bufs, &s_count, &s_thresh, s_sel, s_res, topk_cap, knn);
        for (long long base = 0; base < total; base += blockDim.x) {
            const long long j = base + threadIdx.x;
            topk.offer(j < total ? in[j] : kEmptySlot);
        }
        topk.finish();
        const uint64_t *buf = topk.result();
        for (int j = threadIdx.x; j < knn; j += blockDim.x) {
            const uint64_t key = buf[j];
            const size_t o = (size_t)(q0 + ql) * knn + j;
            if (out_packed) { out_packed[o] = key; continue; }
            if (key == kEmptySlot) {
                out_ids[o] = -1;
                if (out_dists) out_dists[o] = blind ? __int_as_float(-1) : __int_as_float(0x7F800000);
            } else {
                out_ids[o] = (int)(uint32_t)key;
                if (out_dists) out_dists[o] = __uint_as_float((uint32_t)(key >> 32));   // blind: the iteration as int32 bits
            }
        }
        __syncthreads();
    }
}

struct ShardOffsets { long long v[64]; };

// Merge of per-shard result lists for MDCI (replaces the cat/sort/gather of
// dciknn_cuda/core.py:153-157).  One CTA per query.
__global__ void merge_shards_kernel(const int *__restrict__ ids_in, const float *__restrict__ dists_in,
                                    int num_shards, int nq, int k, int topk_cap,
                                    const ShardOffsets offsets,
                                    long long *__restrict__ out_ids, float *__restrict__ out_dists) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ int s_count;
    __shared__ uint64_t s_thresh;
    __shared__ uint32_t s_sel[2][256];
    __shared__ uint32_t s_res[4];
    const int q = blockIdx.x;
    const long long total = (long long)num_shards * k;
    CtaTopK topk;
    topk.init(reinterpret_cast<uint64_t *>(dyn_smem), &s_count, &s_thresh, s_sel, s_res, topk_cap, k);
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
    const uint64_t *buf = topk.result();
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

// The same merge for shard lists in packed form (merge_partitions_kernel's out_packed): in is
// [num_shards][nq][k] keys, local id in the low word.  One CTA per query.
__global__ void merge_shards_packed_kernel(const uint64_t *__restrict__ in, int num_shards, int nq, int k, int topk_cap,
                                           const ShardOffsets offsets, long long *__restrict__ out_ids,
                                           float *__restrict__ out_dists) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ int s_count;
    __shared__ uint64_t s_thresh;
    __shared__ uint32_t s_sel[2][256];
    __shared__ uint32_t s_res[4];
    const int q = blockIdx.x;
    const long long total = (long long)num_shards * k;
    CtaTopK topk;
    topk.init(reinterpret_cast<uint64_t *>(dyn_smem), &s_count, &s_thresh, s_sel, s_res, topk_cap, k);
    for (long long base = 0; base < total; base += blockDim.x) {
        const long long j = base + threadIdx.x;
        uint64_t key = kEmptySlot;
        if (j < total) {
            const int s = (int)(j / k), r = (int)(j % k);
            const uint64_t v = in[((size_t)s * nq + q) * k + r];
            if (v != kEmptySlot)
                key = (v & 0xFFFFFFFF00000000ull) | (uint32_t)((long long)(uint32_t)v + offsets.v[s]);
        }
        topk.offer(key);
    }
    topk.finish();
    const uint64_t *buf = topk.result();
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

// The same merge for k above the selection buffers' limit.  Needs every shard's list sorted
// ascending by (distance, id) with its empty slots (id < 0) last, which is what a query returns:
// the place of an entry in the merged list is then the number of entries of all lists that
// precede it, found with one binary search per shard.  One CTA per query.
__global__ void merge_shards_sorted_kernel(const int *__restrict__ ids_in, const float *__restrict__ dists_in,
                                           int num_shards, int nq, int k, const ShardOffsets offsets,
                                           long long *__restrict__ out_ids, float *__restrict__ out_dists) {
    __shared__ int s_valid[64];
    __shared__ int s_total;
    const int q = blockIdx.x;
    auto key_at = [&](int s, int r) {
        const size_t src = ((size_t)s * nq + q) * k + r;
        return ((uint64_t)__float_as_uint(dists_in[src]) << 32) | (uint32_t)((long long)ids_in[src] + offsets.v[s]);
    };
    for (int s = threadIdx.x; s < num_shards; s += blockDim.x) {   // entries before the first empty slot
        int lo = 0, hi = k;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (ids_in[((size_t)s * nq + q) * k + mid] >= 0) lo = mid + 1; else hi = mid;
        }
        s_valid[s] = lo;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int s = 0; s < num_shards; ++s) t += s_valid[s];
        s_total = t;
    }
    __syncthreads();
    const long long total = (long long)num_shards * k;
    for (long long j = threadIdx.x; j < total; j += blockDim.x) {
        const int s = (int)(j / k), r = (int)(j % k);
        if (r >= s_valid[s]) continue;
        const uint64_t key = key_at(s, r);
        int place = r;
        for (int s2 = 0; s2 < num_shards && place < k; ++s2) {
            if (s2 == s) continue;
            int lo = 0, hi = s_valid[s2];
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (key_at(s2, mid) < key) lo = mid + 1; else hi = mid;
            }
            place += lo;
        }
        if (place < k) {
            out_ids[(size_t)q * k + place] = (long long)(uint32_t)key;
            out_dists[(size_t)q * k + place] = __uint_as_float((uint32_t)(key >> 32));
        }
    }
    for (int j = s_total + threadIdx.x; j < k; j += blockDim.x) {
        out_ids[(size_t)q * k + j] = -1;
        out_dists[(size_t)q * k + j] = __int_as_float(0x7F800000);
    }
}

}  // namespace dci

namespace dci {

// Small partitions: one WARP per (query, partition) work item, no CTA-wide barrier.
// Same computation as traverse_kernel (steps 1-5 of the comment at the top of this
// file), for partitions of at most 32 points whose composite indices have at most
// 32 windows each and at most 32 simple indices: lane = point, lane = window and
// lane = simple index in turn, everything else moves through shuffles.  The
// reference's own example (2 000 points in 100 partitions of 20, 7 simple indices
// per composite index, windows of 10) is of this kind; traverse_kernel spends its
// time there on barriers of a CTA that has almost nothing to do.
constexpr int kSmallWarps = 8;        // warps (work items in flight) per CTA

__global__ void __launch_bounds__(kSmallWarps * 32)
traverse_small_kernel(const TraverseParams prm) {
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xFFFFFFFFu;
    const int L = prm.L, S = prm.S, T = prm.T, I = L * S, dim = prm.dim;
    const uint16_t *spos = reinterpret_cast<const uint16_t *>(prm.spos);
    const uint32_t tmask = (1u << prm.tshift) - 1u;
    const long long nwork = (long long)prm.nq * prm.num_parts;
    const long long nwarps = (long long)gridDim.x * kSmallWarps;
    for (long long wi = (long long)blockIdx.x * kSmallWarps + (threadIdx.x >> 5); wi < nwork; wi += nwarps) {
        const int b = (int)(wi / prm.nq), ql = (int)(wi % prm.nq), q = prm.q0 + ql;
        const long long lo = (long long)b * prm.ppb;
        const int n = (int)min((long long)prm.ppb, (long long)prm.N - lo);
        uint32_t best = 0xFFFFFFFFu;             // this lane's point: promotion iteration << tshift | lane of the window
        int maxW = 0;
        uint32_t rank_a = 0xFFFFFFFFu, rank_b = 0xFFFFFFFFu;   // rank of this lane's window in the first two composite indices (statistics)
        int span_a = 0, span_b = 0;                            // in-range positions of that window
        for (int m = 0; m < L; ++m) {
            // ---- 1. split positions: lane h keeps the constants of simple index h of this composite
            int my_nl = 0, my_cnt = 0, my_c = 0, my_sp = 0;
            float my_qp = 0.0f;
            for (int h = 0; h < S; ++h) {
                const int i = m * S + h;
                const float qp = __ldg(prm.qproj + (size_t)i * prm.nq_total + q);
                const float key = lane < n ? __ldg(prm.skeys + segment_start(lo, i, I, n) + lane) : 0.0f;
                const int s = __popc(__ballot_sync(full, lane < n && key < qp)) - 1;     // last position with key < q
                if (lane == h) {
                    my_nl = (s + 1 + T - 1) / T;
                    const int nr = (n + T - 2 - s + T - 1) / T;
                    my_cnt = my_nl + nr;
                    my_c = my_nl * T - s - 1;
                    my_sp = (s == n - 1 && nr > 0) ? 1 : 0;
                    my_qp = qp;
                }
            }
            // first window of every simple index inside the composite's window list (exclusive scan over lanes)
            int my_off = my_cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(full, my_off, o);
                if (lane >= o) my_off += t;
            }
            const int W = __shfl_sync(full, my_off, 31);
            my_off -= my_cnt;
            maxW = max(maxW, W);
            // ---- 2. lane w = window w: its simple index, priority and place in the visiting order
            int wh = 0;
            for (int h = 1; h < S; ++h) wh += (__shfl_sync(full, my_off, h) <= lane) ? 1 : 0;
            const int w_off = __shfl_sync(full, my_off, wh), w_nl = __shfl_sync(full, my_nl, wh);
            const int w_c = __shfl_sync(full, my_c, wh), w_sp = __shfl_sync(full, my_sp, wh);
            const float w_qp = __shfl_sync(full, my_qp, wh);
            uint64_t okey = ~0ull;                // (priority, simple index, order inside the index): the visiting order
            int span = 0;
            if (lane < W) {
                const int g = lane - w_off, start = g * T - w_c;
                const int at = min(max(start, 0), n - 1);
                const float kv = __ldg(prm.skeys + segment_start(lo, m * S + wh, I, n) + at);
                okey = ((uint64_t)__float_as_uint(fabsf(kv - w_qp)) << 32) |
                       (uint32_t)((wh << 8) | window_visit_order(g, w_nl, w_sp));
                span = max(0, min(start + T, n) - max(start, 0));
            }
            uint32_t rk = 0u;                     // rank = number of windows that come earlier
            for (int j = 0; j < W; ++j) rk += (__shfl_sync(full, okey, j) < okey) ? 1u : 0u;
            if (m == 0) { rank_a = lane < W ? rk : 0xFFFFFFFFu; span_a = span; }
            if (m == 1) { rank_b = lane < W ? rk : 0xFFFFFFFFu; span_b = span; }
            // ---- 3. lane p = point p: the iteration at which its last simple index visits it
            uint32_t mx = 0u;
            for (int h = 0; h < S; ++h) {
                const int i = m * S + h;
                const uint32_t y = lane < n ? (uint32_t)__ldg(spos + pos_segment_start(b, i, I, prm.ppb) + lane) : 0u;
                const uint32_t x = y + (uint32_t)__shfl_sync(full, my_c, h);
                const uint32_t g = prm.divT.div(x);
                const uint32_t t = x - g * (uint32_t)T;
                const uint32_t r = __shfl_sync(full, rk, (__shfl_sync(full, my_off, h) + (int)g) & 31);
                mx = max(mx, (r << prm.tshift) | t);
            }
            if (lane < n && (mx >> prm.tshift) < (best >> prm.tshift)) best = mx;     // ties keep the lower composite
        }
        // ---- 4. stop iteration from the lane-0 promotions (reference :598-607)
        const uint32_t K = best >> prm.tshift;
        const bool is0 = lane < n && (best & tmask) == 0u;
        const unsigned m0 = __ballot_sync(full, is0);
        const int cnt0 = __popc(m0);
        const long long limit = (long long)n * S * T;
        long long stop = limit - 1;
        long long stop_rule = 0x7FFFFFFFFFFFFFFFll;      // iteration at which the stop test fires (statistics)
        if (cnt0 >= prm.knn) {
            const bool need_c = prm.max_cand > prm.knn && cnt0 >= prm.max_cand;
            int lt = 0, le = 0;                   // lane-0 promotions before / not after this lane's
            for (int j = 0; j < 32; ++j) {
                const uint32_t kj = __shfl_sync(full, K, j);
                if ((m0 >> j) & 1u) { lt += kj < K ? 1 : 0; le += kj <= K ? 1 : 0; }
            }
            const unsigned ma = __ballot_sync(full, is0 && lt < prm.knn && prm.knn <= le);
            const long long a = (long long)__shfl_sync(full, K, __ffs(ma) - 1);
            const long long bcap = max(a, prm.outer_s - 1);
            long long ccap;
            if (prm.max_cand <= prm.knn) ccap = a;
            else if (need_c) {
                const unsigned mc = __ballot_sync(full, is0 && lt < prm.max_cand && prm.max_cand <= le);
                ccap = max(a, (long long)__shfl_sync(full, K, __ffs(mc) - 1));
            } else ccap = limit;
            stop_rule = min(bcap, ccap);
            stop = min(stop_rule, limit - 1);
        }
        const uint32_t stop_enc = stop >= (long long)(0xFFFFFFFFu >> prm.tshift) ? 0xFFFFFFFFu
                                                                                 : (((uint32_t)stop + 1u) << prm.tshift) - 1u;
        const bool cand = lane < n && best <= stop_enc;
        if (prm.work_stats) {                     // L <= 2 here (see the launch)
            const int ncand = __popc(__ballot_sync(full, cand));
            const int lane0 = __popc(__ballot_sync(full, is0 && (long long)K <= stop));
            int entries = 0;
            long long visits = 0;
            for (int m = 0; m < L && m < 2; ++m) {
                const uint32_t rkm = m ? rank_b : rank_a;
                int e = (rkm != 0xFFFFFFFFu && (long long)rkm <= stop) ? (m ? span_b : span_a) : 0;
                const int wm = __popc(__ballot_sync(full, rkm != 0xFFFFFFFFu));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(full, e, o);
                entries += e;
                visits += min((long long)wm, stop + 1);
            }
            if (lane == 0) {
                long long *st = prm.work_stats + ((size_t)q * prm.P + b) * 6;
                const bool exhausted = stop_rule > (long long)maxW && (long long)maxW < limit;
                st[0] = exhausted ? (long long)maxW : stop;
                st[1] = visits; st[2] = entries; st[3] = ncand; st[4] = lane0; st[5] = exhausted ? 1 : 0;
            }
        }
        // ---- 5. distances of the promoted points, the partition's top-k by a sort across the lanes
        float bound_d = __int_as_float(0x7F800000), bound_sq = bound_d;
        if (prm.qbound) {
            const uint32_t bb = *reinterpret_cast<volatile uint32_t *>(prm.qbound + ql);
            if (bb < 0x7F7F7F7Fu) {
                bound_d = __uint_as_float(bb);
                const float up = __uint_as_float(bb + 1u);
                bound_sq = __fmul_ru(up, up);
            }
        }
        uint64_t key = kEmptySlot;
        if (cand) {
            const long long gid = lo + lane;
            const float *row = prm.data + (size_t)gid * dim, *qv = prm.query + (size_t)q * dim;
            const float d = prm.vec8 ? dist_sequential_v8(row, qv, dim, bound_sq) : dist_sequential(row, qv, dim, prm.vec4);
            if (d >= 0.0f && d <= bound_d) key = ((uint64_t)__float_as_uint(d) << 32) | (uint32_t)gid;
        }
#pragma unroll
        for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                const uint64_t other = __shfl_xor_sync(full, key, stride);
                const bool up = (lane & size) == 0, low = (lane & stride) == 0;
                key = (low == up) ? min(key, other) : max(key, other);
            }
        }
        uint64_t *out = prm.part_topk + ((size_t)ql * prm.num_parts + b) * prm.kpart;
        if (lane < prm.kpart) out[lane] = key;
        if (prm.qbound && prm.kpart == prm.knn) {
            const uint64_t kth = __shfl_sync(full, key, prm.knn - 1);
            if (lane == 0 && kth != kEmptySlot) atomicMin(prm.qbound + ql, (uint32_t)(kth >> 32));
        }
    }
}

}  // namespace dci
