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

// Exact unsigned division by a runtime-constant divisor d >= 1 for x < limit,
// limit = 2^32 / d (see FastDiv::ok).  Falls back to '/' otherwise.
struct FastDiv {
    uint32_t d, magic;
    int fast;
    __host__ __device__ static FastDiv make(uint32_t d, uint64_t max_x) {
        FastDiv f;
        f.d = d;
        f.magic = 0;
        f.fast = 0;
        if (d > 1 && max_x < (0x100000000ull / d)) {
            f.magic = (uint32_t)(0x100000000ull / d) + 1u;
            f.fast = 1;
        }
        return f;
    }
    __device__ __forceinline__ uint32_t div(uint32_t x) const {
        if (d == 1) return x;
        return fast ? __umulhi(x, magic) : x / d;
    }
};

// Exclusive scan, in place, of 8 * blockDim.x counters laid out so that thread
// t owns entries [8t, 8t+8).  warp_tot is a 32-entry shared scratch array.
// Ends with a barrier.
template <typename CntT>
__device__ __forceinline__ void cta_exclusive_scan8(CntT *cnt, uint32_t *warp_tot) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
    CntT *p = cnt + tid * 8;
    uint32_t v[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[j] = p[j]; sum += v[j]; }
    uint32_t inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[w] = inc;
    __syncthreads();
    if (w == 0) {
        uint32_t t = lane < nw ? warp_tot[lane] : 0, i2 = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t u = __shfl_up_sync(0xFFFFFFFFu, i2, o);
            if (lane >= o) i2 += u;
        }
        warp_tot[lane] = i2 - t;
    }
    __syncthreads();
    uint32_t base = warp_tot[w] + inc - sum;
#pragma unroll
    for (int j = 0; j < 8; ++j) { p[j] = (CntT)base; base += v[j]; }
    __syncthreads();
}

// Stable LSD radix sort of W (u32 key, ValT payload) pairs by one CTA, 8 bits
// per pass over key bits [0, 32).  Buffers may live in shared or global memory.
// Input in (kA, vA); (kB, vB) is the ping-pong buffer.  With RANK_OUT the last
// pass writes rank_out[payload] = final position instead of the sorted pairs;
// otherwise the sorted pairs end in (kA, vA).
// hist: 256 * (blockDim.x / 32) counters in shared memory; warp_tot: 32 words.
// Stability: warp w owns the contiguous slice [w*C, (w+1)*C) of the input and
// walks it in order, 32 keys a round; equal digits inside a round are ranked by
// lane with match.any; the scan runs digit-major, warp-minor.
template <typename ValT, typename CntT, bool RANK_OUT>
__device__ void cta_radix_sort(uint32_t *kA, ValT *vA, uint32_t *kB, ValT *vB, int W,
                               CntT *hist, uint32_t *warp_tot, ValT *rank_out) {
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
    const int C = (W + nw - 1) / nw;
    const int rounds = (C + 31) >> 5;
    const unsigned lt = lanemask_lt();
    uint32_t *kin = kA, *kout = kB;
    ValT *vin = vA, *vout = vB;
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
            if (valid && lane == __ffs(peers) - 1) hist[d * nw + w] += (CntT)__popc(peers);
            __syncwarp();
        }
        __syncthreads();
        cta_exclusive_scan8(hist, warp_tot);
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
            if (valid) base = hist[d * nw + w];
            __syncwarp();
            if (valid) {
                const uint32_t dest = base + __popc(peers & lt);
                if (last) {
                    rank_out[val] = (ValT)dest;
                } else {
                    kout[dest] = key;
                    vout[dest] = val;
                }
                if (lane == __ffs(peers) - 1) hist[d * nw + w] = (CntT)(base + __popc(peers));
            }
            __syncwarp();
        }
        __syncthreads();
        uint32_t *tk = kin; kin = kout; kout = tk;
        ValT *tv = vin; vin = vout; vout = tv;
    }
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

// Streaming top-k of u64 keys (smaller is better) by one CTA.
//   buf   : shared, cap entries, cap = power of two >= k + blockDim.x
//   state : shared int[2]: [0] = number of valid entries in buf
// Usage: topk_init; for each round every thread calls topk_offer with at most
// one key (or kEmptySlot for none) -- all threads must call it; topk_finish
// leaves the k smallest, ascending, in buf[0..k) (padded with kEmptySlot).
struct CtaTopK {
    uint64_t *buf;
    int *count;
    uint64_t *thresh;   // shared: keys >= *thresh cannot enter the top k
    int cap, k;

    __device__ __forceinline__ void init(uint64_t *b, int *cnt, uint64_t *th, int cap_, int k_) {
        buf = b; count = cnt; thresh = th; cap = cap_; k = k_;
        if (threadIdx.x == 0) { *count = 0; *thresh = kEmptySlot; }
        __syncthreads();
    }
    __device__ __forceinline__ void compact() {   // all threads; sorts and keeps k
        const int c = *count;
        int len = 2;
        while (len < c) len <<= 1;
        __syncthreads();
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
        if (key < *thresh) {
            const int slot = atomicAdd(count, 1);
            buf[slot] = key;
        }
        __syncthreads();
    }
    __device__ __forceinline__ void finish() {
        compact();
        for (int i = *count + threadIdx.x; i < k; i += blockDim.x) buf[i] = kEmptySlot;
        __syncthreads();
    }
};

}  // namespace dci
