// Shared device helpers for the DCI kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dci {

constexpr int kMaxIndices = 256;      // upper bound on L*S held in shared memory
constexpr int kMaxTopK = 1024;        // largest k served by the fused top-k path
constexpr uint64_t kEmptySlot = 0xFFFFFFFFFFFFFFFFull;   // (dist bits, id) of an unfilled slot

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Order-preserving map from fp32 to u32 (and back).  -0 is folded into +0 first
// so that keys that compare equal as floats map to the same integer.
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    if (f == 0.0f) f = 0.0f;
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
}

// Exact unsigned division by a runtime-constant divisor d >= 1, branch-free:
// x / d = umulhi(x, magic) + x * unit with magic = floor(2^32 / d) + 1, unit = 0
// for d >= 2 (exact while x * d < 2^32) and magic = 0, unit = 1 for d = 1.
struct FastDiv {
    uint32_t magic, unit;
    __host__ __device__ static FastDiv make(uint32_t d) {
        FastDiv f;
        f.magic = d > 1 ? (uint32_t)(0x100000000ull / d) + 1u : 0u;
        f.unit = d > 1 ? 0u : 1u;
        return f;
    }
    __host__ __device__ static bool exact_for(uint32_t d, uint64_t max_x) {
        return d == 1 || max_x * d < 0x100000000ull;
    }
    __device__ __forceinline__ uint32_t div(uint32_t x) const { return __umulhi(x, magic) + x * unit; }
};

// Exclusive scan, in place, of a[0..n) by the whole CTA; also returns the total
// to every thread.  scratch: 33 shared words.  Ends with a barrier.
template <typename T>
__device__ __forceinline__ uint32_t cta_exclusive_scan(T *a, int n, uint32_t *scratch) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
    const int per = (n + blockDim.x - 1) / blockDim.x;
    const int lo = min(tid * per, n), hi = min(lo + per, n);
    uint32_t sum = 0;
    for (int j = lo; j < hi; ++j) sum += a[j];
    uint32_t inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) scratch[w] = inc;
    __syncthreads();
    if (w == 0) {
        const uint32_t t = lane < nw ? scratch[lane] : 0;
        uint32_t i2 = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t u = __shfl_up_sync(0xFFFFFFFFu, i2, o);
            if (lane >= o) i2 += u;
        }
        scratch[lane] = i2 - t;
        if (lane == 31) scratch[32] = i2;
    }
    __syncthreads();
    uint32_t base = scratch[w] + inc - sum;
    for (int j = lo; j < hi; ++j) { const uint32_t v = a[j]; a[j] = (T)base; base += v; }
    const uint32_t total = scratch[32];
    __syncthreads();
    return total;
}
__device__ __forceinline__ uint32_t cta_exclusive_scan_u32(uint32_t *a, int n, uint32_t *scratch) {
    return cta_exclusive_scan<uint32_t>(a, n, scratch);
}

// Exclusive scan of 16-bit counters in shared memory, eight at a time (128-bit
// accesses).  `a` must be 16-byte aligned and allocated (and zero) up to the
// next multiple of 8 entries beyond n.  Ends with a barrier.
__device__ __forceinline__ void cta_exclusive_scan_u16x8(uint16_t *a, int n, uint32_t *scratch) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
    const int n8 = (n + 7) >> 3;                                   // groups of 8 entries
    const int per = (n8 + blockDim.x - 1) / blockDim.x;            // groups per thread
    const int g0 = min(tid * per, n8), g1 = min(g0 + per, n8);
    uint4 *v = reinterpret_cast<uint4 *>(a);
    uint32_t sum = 0;
    for (int g = g0; g < g1; ++g) {
        const uint4 x = v[g];
        const uint32_t s2 = x.x + x.y + x.z + x.w;     // low and high halves summed side by side: no carry, the total stays below 65 536
        sum += (s2 & 0xFFFFu) + (s2 >> 16);
    }
    uint32_t inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) scratch[w] = inc;
    __syncthreads();
    if (w == 0) {
        const uint32_t t = lane < nw ? scratch[lane] : 0;
        uint32_t i2 = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t u = __shfl_up_sync(0xFFFFFFFFu, i2, o);
            if (lane >= o) i2 += u;
        }
        scratch[lane] = i2 - t;
    }
    __syncthreads();
    uint32_t base = scratch[w] + inc - sum;
    for (int g = g0; g < g1; ++g) {
        const uint4 x = v[g];
        uint4 y;
        // exclusive prefix of the pair (lo, hi) from base: low half base, high half base + lo
        y.x = base * 0x10001u + (x.x << 16); base += (x.x & 0xFFFFu) + (x.x >> 16);
        y.y = base * 0x10001u + (x.y << 16); base += (x.y & 0xFFFFu) + (x.y >> 16);
        y.z = base * 0x10001u + (x.z << 16); base += (x.z & 0xFFFFu) + (x.z >> 16);
        y.w = base * 0x10001u + (x.w << 16); base += (x.w & 0xFFFFu) + (x.w >> 16);
        v[g] = y;
    }
    __syncthreads();
}
__device__ __forceinline__ void cta_scan_counters(uint16_t *a, int n, uint32_t *scratch) {
    cta_exclusive_scan_u16x8(a, n, scratch);
}
__device__ __forceinline__ void cta_scan_counters(uint32_t *a, int n, uint32_t *scratch) {
    cta_exclusive_scan<uint32_t>(a, n, scratch);
}

// Zeroes `bytes` (a multiple of 16) of 16-byte aligned shared memory.  No barrier.
__device__ __forceinline__ void cta_zero16(void *p, size_t bytes) {
    uint4 *v = reinterpret_cast<uint4 *>(p);
    for (size_t i = threadIdx.x; i < (bytes >> 4); i += blockDim.x) v[i] = make_uint4(0u, 0u, 0u, 0u);
}

// Bucket counters are 32-bit, or 16-bit packed two to a word (counts must then
// stay below 65 536, which holds whenever the number of keys does).  arrive()
// adds one to bucket b and returns the previous count.
__device__ __forceinline__ uint32_t bucket_arrive(uint32_t *cnt, int b) { return atomicAdd(&cnt[b], 1u); }
__device__ __forceinline__ uint32_t bucket_arrive(uint16_t *cnt, int b) {
    uint32_t *word = reinterpret_cast<uint32_t *>(cnt) + (b >> 1);
    const int sh = (b & 1) << 4;
    return (atomicAdd(word, 1u << sh) >> sh) & 0xFFFFu;
}

// Stable LSD radix sort of W (u32 key, ValT payload) pairs by one CTA, 8 bits
// per pass over key bits [0, 32).  Buffers may live in shared or global memory.
// Input in (kA, vA); (kB, vB) is the ping-pong buffer.  With RANK_OUT the last
// pass writes rank_out[payload] = final position instead of the sorted pairs;
// otherwise the sorted pairs end in (kA, vA).
// hist: 256 * (blockDim.x / 32) counters in shared memory, laid out [warp][digit]
// so that the lanes of a warp touch different banks; warp_tot: 33 shared words.
// Stability: warp w owns the contiguous slice [w*C, (w+1)*C) of the input and
// walks it in order, 32 keys a round; equal digits inside a round are ranked by
// lane with match.any; offsets are prefix sums in (digit, warp) order.
template <typename ValT, typename CntT, bool RANK_OUT>
__device__ void cta_radix_sort(uint32_t *kA, ValT *vA, uint32_t *kB, ValT *vB, int W,
                               CntT *hist, uint32_t *warp_tot, ValT *rank_out) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
    const int C = (W + nw - 1) / nw;
    const int rounds = (C + 31) >> 5;
    const unsigned lt = lanemask_lt();
    __shared__ uint32_t digit_base[256];
    uint32_t *kin = kA, *kout = kB;
    ValT *vin = vA, *vout = vB;
    CntT *myhist = hist + w * 256;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = pass * 8;
        for (int i = tid; i < 256 * nw; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int r = 0; r < rounds; ++r) {
            const int off = r * 32 + lane;
            const int x = w * C + off;
            const bool valid = off < C && x < W;
            const uint32_t d = valid ? ((kin[x] >> shift) & 255u) : (256u + lane);
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, d);
            if (valid && lane == __ffs(peers) - 1) myhist[d] += (CntT)__popc(peers);
            __syncwarp();
        }
        __syncthreads();
        // hist[w][d] <- number of keys with digit d in warps before w; digit_base[d] <- total of d
        for (int dg = tid; dg < 256; dg += blockDim.x) {     // CTAs may have fewer than 256 threads
            uint32_t run = 0;
            for (int ww = 0; ww < nw; ++ww) {
                const uint32_t c = hist[ww * 256 + dg];
                hist[ww * 256 + dg] = (CntT)run;
                run += c;
            }
            digit_base[dg] = run;
        }
        __syncthreads();
        cta_exclusive_scan_u32(digit_base, 256, warp_tot);
        const bool last = RANK_OUT && pass == 3;
        for (int r = 0; r < rounds; ++r) {
            const int off = r * 32 + lane;
            const int x = w * C + off;
            const bool valid = off < C && x < W;
            uint32_t key = 0;
            ValT val = 0;
            if (valid) { key = kin[x]; val = vin[x]; }
            const uint32_t d = valid ? ((key >> shift) & 255u) : (256u + lane);
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, d);
            uint32_t base = 0;
            if (valid) base = myhist[d];
            __syncwarp();
            if (valid) {
                const uint32_t dest = digit_base[d] + base + __popc(peers & lt);
                if (last) {
                    rank_out[val] = (ValT)dest;
                } else {
                    kout[dest] = key;
                    vout[dest] = val;
                }
                if (lane == __ffs(peers) - 1) myhist[d] = (CntT)(base + __popc(peers));
            }
            __syncwarp();
        }
        __syncthreads();
        uint32_t *tk = kin; kin = kout; kout = tk;
        ValT *tv = vin; vin = vout; vout = tv;
    }
}

constexpr int kMaxBucket = 48;   // largest bucket the counting rank accepts
constexpr int kRankBatch = 4;    // bucket mates compared without a branch

// Bucket of a non-negative fp32 key: equal-width value buckets, a monotone map.  key * scale is
// rounded to an integer by adding 2^23 (the sum's low mantissa bits are then that integer): one
// fused multiply-add and one subtraction instead of a float-to-int conversion, which runs at a
// fraction of the rate.  Needs key * scale < 2^22; the number of buckets is far below that.
__device__ __forceinline__ int bucket_of(uint32_t key_bits, float scale, int last) {
    return min(last, __float_as_int(__fmaf_rn(__uint_as_float(key_bits), scale, 8388608.0f)) - 0x4B000000);
}

// Second half of the counting rank.  Precondition: every key w in [0, W) has
// been dropped into bucket_of(key[w]) with slot[w] = its arrival number there
// and cnt[b] = the size of bucket b (all <= kMaxBucket), cnt[nbuckets] = 0.
// Lists the key indices bucket by bucket in bval, then gives every key its rank
// in ascending (key, tie order): rank = start of its bucket + number of smaller
// keys inside the bucket.  tie_less(a, b) orders two key indices whose keys are
// equal.  rank_out[w] receives the rank.  Ends with a barrier.
// bkey (W words, may be null): when given, the keys are listed bucket by bucket
// too and the ranking walks those lists, so that a warp reads consecutive
// entries, its counter reads fall on the same or neighbouring words and the
// bucket mates it compares with lie next to its own entry; the only scattered
// access left is the store of the rank.  Without it every key looks its bucket
// mates up through bval.
// bucket(k): the bucket of key k, the same monotone map that produced cnt and slot.
template <typename ValT, typename CntT, typename Bucket, typename TieLess, typename Mark>
__device__ __forceinline__ void cta_bucket_place_and_rank(const uint32_t *key, int W, const uint8_t *slot,
                                                          ValT *bval, uint32_t *bkey, CntT *cnt, int nbuckets,
                                                          Bucket bucket, uint32_t *scratch, ValT *rank_out,
                                                          TieLess tie_less, Mark mark) {
    const int tid = threadIdx.x;
    cta_scan_counters(cnt, nbuckets + 1, scratch);           // cnt[b] = start of bucket b, cnt[nbuckets] = W
    mark(8);
    if (bkey) {
        for (int w = tid; w < W; w += blockDim.x) {
            const uint32_t k = key[w];
            const uint32_t dest = (uint32_t)cnt[bucket(k)] + (uint32_t)slot[w];
            bval[dest] = (ValT)w;
            bkey[dest] = k;
        }
        __syncthreads();
        mark(9);
        // The first kRankBatch mates of the bucket are compared without a branch (most buckets hold
        // no more), the rest one by one; equal keys are only counted there and settled by tie_less
        // in a loop of their own, which few entries enter.  A slot beyond the bucket reads as the
        // largest key: never smaller, and equal only to a key that takes the tie loop anyway.
        for (int j = tid; j < W; j += blockDim.x) {
            const uint32_t k = bkey[j];
            const int b = bucket(k);
            const uint32_t lo = cnt[b], hi = cnt[b + 1];
            const uint32_t me = (uint32_t)bval[j];
            uint32_t r = lo, ties = 0;
            uint32_t kk[kRankBatch];
#pragma unroll
            for (int u = 0; u < kRankBatch; ++u) kk[u] = (lo + u < hi) ? bkey[lo + u] : 0xFFFFFFFFu;
#pragma unroll
            for (int u = 0; u < kRankBatch; ++u) { r += (kk[u] < k); ties += (kk[u] == k); }
            for (uint32_t j2 = lo + kRankBatch; j2 < hi; ++j2) {
                const uint32_t k2 = bkey[j2];
                r += (k2 < k);
                ties += (k2 == k);
            }
            if (ties > 1) {                                  // the entry itself is one of them
                for (uint32_t j2 = lo; j2 < hi; ++j2)
                    if (bkey[j2] == k && j2 != (uint32_t)j && tie_less((uint32_t)bval[j2], me)) ++r;
            }
            rank_out[me] = (ValT)r;
        }
        __syncthreads();
        return;
    }
    for (int w = tid; w < W; w += blockDim.x)
        bval[(uint32_t)cnt[bucket(key[w])] + (uint32_t)slot[w]] = (ValT)w;
    __syncthreads();
    mark(9);
    for (int w = tid; w < W; w += blockDim.x) {
        const uint32_t k = key[w];
        const int b = bucket(k);
        const uint32_t lo = cnt[b], hi = cnt[b + 1];
        uint32_t r = lo, ties = 0;
        {                                                // the first four mates without a branch, as above
            uint32_t other[kRankBatch], kj[kRankBatch];
#pragma unroll
            for (int u = 0; u < kRankBatch; ++u) other[u] = lo + u < hi ? (uint32_t)bval[lo + u] : (uint32_t)w;
#pragma unroll
            for (int u = 0; u < kRankBatch; ++u) kj[u] = lo + u < hi ? key[other[u]] : 0xFFFFFFFFu;
#pragma unroll
            for (int u = 0; u < kRankBatch; ++u) { r += (kj[u] < k); ties += (kj[u] == k); }
        }
        for (uint32_t j2 = lo + kRankBatch; j2 < hi; ++j2) {
            const uint32_t k2 = key[bval[j2]];
            r += (k2 < k);
            ties += (k2 == k);
        }
        if (ties > 1) {
            for (uint32_t j2 = lo; j2 < hi; ++j2) {
                const uint32_t o = (uint32_t)bval[j2];
                if (o != (uint32_t)w && key[o] == k && tie_less(o, (uint32_t)w)) ++r;
            }
        }
        rank_out[w] = (ValT)r;
    }
    __syncthreads();
}

// The k1-th and k2-th smallest (1-based) of get(0..cnt), whose values are below
// 2^bits, by radix selection 8 bits at a time.  Requires 1 <= k <= cnt.
// sel: 2 x 256 shared counters; res: 4 shared words.  Results in out[0], out[1].
template <typename Get>
__device__ __forceinline__ void cta_select2(Get get, int cnt, int k1, int k2, int bits,
                                            uint32_t (*sel)[256], uint32_t *res, uint32_t out[2]) {
    const int tid = threadIdx.x, lane = tid & 31;
    int top = ((bits + 7) / 8) * 8 - 8;
    if (top < 0) top = 0;
    if (tid == 0) { res[0] = 0u; res[1] = 0u; res[2] = (uint32_t)k1; res[3] = (uint32_t)k2; }
    for (int shift = top; shift >= 0; shift -= 8) {
        for (int i = tid; i < 512; i += blockDim.x) sel[i >> 8][i & 255] = 0u;
        __syncthreads();
        const uint32_t p0 = res[0], p1 = res[1];
        const bool both = k1 != k2;                       // equal ranks: one histogram serves both
        for (int j = tid; j < cnt; j += blockDim.x) {
            const uint32_t v = get(j), hi = (shift + 8 >= 32) ? 0u : (v >> (shift + 8)), d = (v >> shift) & 255u;
            if (hi == p0) atomicAdd(&sel[0][d], 1u);
            if (both && hi == p1) atomicAdd(&sel[1][d], 1u);
        }
        __syncthreads();
        if (tid < (both ? 64 : 32)) {   // warp 0 resolves the first rank, warp 1 the second
            const int which = tid >> 5;
            const uint32_t want = res[2 + which];
            uint32_t c[8], sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { c[j] = sel[which][lane * 8 + j]; sum += c[j]; }
            uint32_t inc = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o) inc += t;
            }
            const unsigned reach = __ballot_sync(0xFFFFFFFFu, inc >= want);
            const int owner = __ffs(reach) - 1;
            if (lane == owner) {
                uint32_t before = inc - sum;
                int d = 0;
                while (d < 7 && before + c[d] < want) { before += c[d]; ++d; }
                res[which] = (res[which] << 8) | (uint32_t)(lane * 8 + d);
                res[2 + which] = want - before;
            }
        }
        __syncthreads();
    }
    out[0] = res[0];
    out[1] = k1 != k2 ? res[1] : res[0];
    __syncthreads();
}

// In-place ascending bitonic sort of `len` (power of two) u64 keys in shared
// memory by the whole CTA.  Ends with a barrier.
__device__ __forceinline__ void cta_bitonic_sort_u64(uint64_t *a, int len) {
    for (int size = 2; size <= len; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = threadIdx.x; t < (len >> 1); t += blockDim.x) {
                const int lo = ((t / stride) * (stride << 1)) + (t % stride);
                const int hi = lo + stride;
                const bool up = ((lo & size) == 0);
                const uint64_t x = a[lo], y = a[hi];
                if ((x > y) == up) { a[lo] = y; a[hi] = x; }
            }
            __syncthreads();
        }
    }
}

// Appends one element per lane with pred set to a shared list with a single
// atomic per warp; returns the slot (valid where pred).  All lanes must call.
__device__ __forceinline__ int warp_append_slot(bool pred, int *counter) {
    const unsigned m = __ballot_sync(0xFFFFFFFFu, pred);
    int base = 0;
    if ((threadIdx.x & 31) == 0 && m) base = atomicAdd(counter, __popc(m));
    base = __shfl_sync(0xFFFFFFFFu, base, 0);
    return base + __popc(m & lanemask_lt());
}

// Streaming top-k of u64 keys (smaller is better; high word = fp32 distance
// bits, low word = id) by one CTA.
//   bufs   : shared, 2 * cap entries (two halves that swap roles),
//            cap = power of two >= k + blockDim.x
//   shared state: count, thresh, sel[2][256], res[4] supplied by the caller
// Usage: init; every round all threads call offer with at most one key each
// (kEmptySlot for none); finish leaves the k smallest, ascending, in
// result()[0..k) (padded with kEmptySlot).
// When the buffer fills up it is reduced to the k smallest: the k-th smallest
// distance is found by radix selection, the few keys not above it are moved to
// the other half and only those are sorted.
struct CtaTopK {
    uint64_t *buf, *other;
    int *count;
    uint64_t *thresh;   // shared: keys >= *thresh cannot enter the top k
    uint32_t (*sel)[256];
    uint32_t *res;
    int cap, k;

    __device__ __forceinline__ void init(uint64_t *bufs, int *cnt, uint64_t *th, uint32_t (*sel_)[256],
                                         uint32_t *res_, int cap_, int k_) {
        buf = bufs; other = bufs + cap_; count = cnt; thresh = th; sel = sel_; res = res_; cap = cap_; k = k_;
        if (threadIdx.x == 0) { *count = 0; *thresh = kEmptySlot; }
        __syncthreads();
    }
    __device__ __forceinline__ uint64_t *result() { return buf; }
    __device__ __forceinline__ void compact() {   // all threads; keeps the k smallest, sorted
        int c = *count;
        __syncthreads();
        if (c > k && c > 128) {       // a short list is cheaper to sort outright
            uint32_t tau[2];
            const uint64_t *src = buf;
            cta_select2([src](int j) { return (uint32_t)(src[j] >> 32); }, c, k, k, 32, sel, res, tau);
            if (threadIdx.x == 0) *count = 0;
            __syncthreads();
            for (int j0 = 0; j0 < c; j0 += blockDim.x) {
                const int j = j0 + threadIdx.x;
                const uint64_t key = j < c ? buf[j] : kEmptySlot;
                const bool take = j < c && (uint32_t)(key >> 32) <= tau[0];
                const int sl = warp_append_slot(take, count);
                if (take) other[sl] = key;
            }
            __syncthreads();
            c = *count;
            uint64_t *t = buf; buf = other; other = t;
            __syncthreads();
        }
        int len = 2;
        while (len < c) len <<= 1;
        for (int i = c + threadIdx.x; i < len; i += blockDim.x) buf[i] = kEmptySlot;
        __syncthreads();
        cta_bitonic_sort_u64(buf, len);
        if (threadIdx.x == 0) {
            const int nc = c < k ? c : k;
            *count = nc;
            *thresh = nc >= k ? buf[k - 1] : kEmptySlot;
        }
        __syncthreads();
    }
    __device__ __forceinline__ void offer(uint64_t key) {
        const int c = *count;      // read by every thread before any thread of this round appends
        __syncthreads();
        if (c > cap - (int)blockDim.x) compact();
        const bool take = key < *thresh;
        const int sl = warp_append_slot(take, count);
        if (take) buf[sl] = key;
        __syncthreads();
    }
    // offer() for rounds in which at most `producers` threads hold a key (the others pass
    // kEmptySlot): the buffer only has to keep room for that many appends.
    __device__ __forceinline__ void offer_from(uint64_t key, int producers) {
        const int c = *count;
        __syncthreads();
        if (c > cap - producers) compact();
        const bool take = key < *thresh;
        const int sl = warp_append_slot(take, count);
        if (take) buf[sl] = key;
        __syncthreads();
    }
    __device__ __forceinline__ void finish() {
        compact();
        for (int i = *count + threadIdx.x; i < k; i += blockDim.x) buf[i] = kEmptySlot;
        __syncthreads();
    }
};

// State of one streaming top-k kept in shared memory, so that several of them
// can be driven from fully unrolled code without per-object registers.
struct TopKSlot {
    unsigned long long thresh;
    int count;
    int half;       // which half of its buffer pair currently holds the entries
};

__device__ __forceinline__ CtaTopK topk_slot_open(TopKSlot *s, uint64_t *bufs, uint32_t (*sel)[256], uint32_t *res,
                                                  int cap, int k) {
    CtaTopK t;
    t.buf = bufs + (size_t)s->half * cap;
    t.other = bufs + (size_t)(1 - s->half) * cap;
    t.count = &s->count;
    t.thresh = reinterpret_cast<uint64_t *>(&s->thresh);
    t.sel = sel; t.res = res; t.cap = cap; t.k = k;
    return t;
}
__device__ __forceinline__ void topk_slot_close(TopKSlot *s, const CtaTopK &t, const uint64_t *bufs) {
    if (threadIdx.x == 0) s->half = (t.buf == bufs) ? 0 : 1;
    __syncthreads();
}

// Index arrays are partition-major.  First entry of the segment of simple index i for the
// partition whose first point is `lo` and which holds n points (n = ppb except for the last
// partition), I simple indices in all.
__host__ __device__ __forceinline__ size_t segment_start(long long lo, int i, int I, int n) {
    return (size_t)lo * (size_t)I + (size_t)i * (size_t)n;
}

// The inverse permutation (position of each point in its sorted segment) has a layout of its own:
// every segment starts on a multiple of 8 entries, segment (partition b, simple index i) at
// (b * I + i) * pos_stride(ppb), so that the positions of neighbouring points can be read with
// aligned vector loads.  The entries between a segment's n points and the stride are zero.
__host__ __device__ __forceinline__ int pos_stride(int ppb) { return (ppb + 7) & ~7; }
__host__ __device__ __forceinline__ size_t pos_segment_start(long long b, int i, int I, int ppb) {
    return ((size_t)b * (size_t)I + (size_t)i) * (size_t)pos_stride(ppb);
}

}  // namespace dci
