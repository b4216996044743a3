// Tensor-core projection: out[i][p] = <proj[i], x[p]> on the 5th-generation
// tensor cores (tcgen05.mma, accumulator in tensor memory) with fp32 operands
// split into two tf32 terms ("3xTF32": a*b ~= a_lo*b_hi + a_hi*b_lo + a_hi*b_hi).
// An optional replacement for the exact kernel of project.cuh, i.e. for the
// cublasSgemm calls of the reference (src/util_kernel.cu:45-80).  Keys differ
// from the exact path by about 1e-6 * |x| (not bit-identical), so the exact
// path stays the default and the one the parity tests pin.
//
// One CTA of 128 threads computes a tile of 128 points x 32 directions (the
// L*S <= 32 directions are zero padded).  Per 32-wide slice of the coordinate
// axis the threads stage the hi and lo parts of the points (A) and directions
// (B) in shared memory in the K-major no-swizzle canonical layout of the UMMA
// shared-memory descriptor (core matrices of 8 rows x 16 bytes, 128 bytes each;
// the next 16 bytes along K are 128 bytes further, the next 8 rows 1024 bytes
// further), one thread issues 4 x 3 MMAs of shape 128 x 32 x 8 and commits them
// to an mbarrier, and all threads wait for it before restaging.  Several CTAs
// share an SM (40 KB of shared memory and 32 tensor-memory columns each), which
// overlaps one CTA's loads with another's MMAs.  The epilogue reads the 128 x 32
// accumulator with tcgen05.ld (lane = point, column = direction) and writes
// coalesced rows of `out`.  Every wait is bounded; on a time-out the kernel
// raises *error, skips its stores, frees its tensor memory and returns.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace dci {

constexpr int kTcPoints = 128;     // M of the MMA tile (points)
constexpr int kTcDirs = 32;        // N of the MMA tile (directions, zero padded)
constexpr int kTcK = 32;           // coordinates staged per step
constexpr uint32_t kTcWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major, no swizzle: start address, leading (K) byte offset 128, stride (8-row) byte offset 1024,
// descriptor version 1 (bits 46-47), layout type 0.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128u >> 4) << 16) | ((uint64_t)(1024u >> 4) << 32) |
           (1ull << 46);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void split_tf32(float a, float &hi, float &lo) {
    hi = __uint_as_float(__float_as_uint(a) & 0xFFFFE000u);      // the 19 bits a tf32 operand keeps
    lo = __uint_as_float(__float_as_uint(__fsub_rn(a, hi)) & 0xFFFFE000u);
}

__global__ void __launch_bounds__(kTcPoints)
project_tf32x3_kernel(const float *__restrict__ x, long long n, int dim, const float *__restrict__ proj,
                      int num_indices, int i0, float *__restrict__ out, int *error) {
    __shared__ __align__(1024) float a_hi[kTcPoints * kTcK];
    __shared__ __align__(1024) float a_lo[kTcPoints * kTcK];
    __shared__ __align__(1024) float b_hi[kTcDirs * kTcK];
    __shared__ __align__(1024) float b_lo[kTcDirs * kTcK];
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ uint32_t tmem_slot;

    const int tid = threadIdx.x, warp = tid >> 5;
    const long long p0 = (long long)blockIdx.x * kTcPoints;
    const bool vec_ok = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(proj) & 15) == 0);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)kTcDirs));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;

    // instruction descriptor: D = f32, A = B = tf32, both K-major, N = 32, M = 128
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTcDirs >> 3) << 17) |
                           ((uint32_t)(kTcPoints >> 4) << 24);
    uint32_t parity = 0, accumulate = 0;
    int failed = 0;

    for (int k0 = 0; k0 < dim && !failed; k0 += kTcK) {
        // stage A: 128 rows x 8 sixteen-byte pieces; 8 consecutive threads read one row's 128 bytes
        for (int f = tid; f < kTcPoints * (kTcK / 4); f += kTcPoints) {
            const int row = f >> 3, piece = f & 7, col = k0 + piece * 4;
            const long long p = p0 + row;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p < n) {
                const float *src = x + p * dim + col;
                if (vec_ok && col + 3 < dim) {
                    v = __ldg(reinterpret_cast<const float4 *>(src));
                } else {
                    if (col < dim) v.x = __ldg(src);
                    if (col + 1 < dim) v.y = __ldg(src + 1);
                    if (col + 2 < dim) v.z = __ldg(src + 2);
                    if (col + 3 < dim) v.w = __ldg(src + 3);
                }
            }
            float4 h, l;
            split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
            const int off = (row >> 3) * 256 + piece * 32 + (row & 7) * 4;     // in floats
            *reinterpret_cast<float4 *>(a_hi + off) = h;
            *reinterpret_cast<float4 *>(a_lo + off) = l;
        }
        // stage B: 32 rows (directions i0 .. i0+31, zero beyond num_indices) x 8 pieces
        for (int f = tid; f < kTcDirs * (kTcK / 4); f += kTcPoints) {
            const int row = f >> 3, piece = f & 7, col = k0 + piece * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i0 + row < num_indices) {
                const float *src = proj + (size_t)(i0 + row) * dim + col;
                if (vec_ok && col + 3 < dim) {
                    v = __ldg(reinterpret_cast<const float4 *>(src));
                } else {
                    if (col < dim) v.x = __ldg(src);
                    if (col + 1 < dim) v.y = __ldg(src + 1);
                    if (col + 2 < dim) v.z = __ldg(src + 2);
                    if (col + 3 < dim) v.w = __ldg(src + 3);
                }
            }
            float4 h, l;
            split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
            const int off = (row >> 3) * 256 + piece * 32 + (row & 7) * 4;
            *reinterpret_cast<float4 *>(b_hi + off) = h;
            *reinterpret_cast<float4 *>(b_lo + off) = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> tensor-core reads
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t ah = smem_u32(a_hi), al = smem_u32(a_lo), bh = smem_u32(b_hi), bl = smem_u32(b_lo);
#pragma unroll
            for (int kk = 0; kk < kTcK / 8; ++kk) {          // one MMA covers 8 coordinates = 2 pieces = 256 bytes
                const uint32_t step = kk * 256;
                umma_tf32(tmem_d, umma_desc_kmajor(al + step), umma_desc_kmajor(bh + step), idesc, accumulate);
                accumulate = 1;
                umma_tf32(tmem_d, umma_desc_kmajor(ah + step), umma_desc_kmajor(bl + step), idesc, 1u);
                umma_tf32(tmem_d, umma_desc_kmajor(ah + step), umma_desc_kmajor(bh + step), idesc, 1u);
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&mbar))
                         : "memory");
        }
        // wait until the MMAs have read the staged tiles (bounded)
        uint32_t done = 0;
        for (uint32_t spin = 0; spin < kTcWaitLimit && !done; ++spin) {
            asm volatile(
                "{\n\t"
                ".reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.b32 %0, 1, 0, p;\n\t"
                "}\n"
                : "=r"(done)
                : "r"(smem_u32(&mbar)), "r"(parity)
                : "memory");
        }
        parity ^= 1u;
        failed = __syncthreads_or(done ? 0 : 1);
    }

    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!failed) {
        // lane (= point) quarter of this warp, 32 columns (= directions) per thread
        uint32_t r[32];
        const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32"
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const long long p = p0 + tid;
        if (p < n) {
#pragma unroll
            for (int c = 0; c < kTcDirs; ++c)
                if (i0 + c < num_indices) out[(size_t)(i0 + c) * n + p] = __uint_as_float(r[c]);
        }
    } else if (tid == 0) {
        atomicExch(error, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)kTcDirs));
    }
}

// ---------------------------------------------------------------------------
// The same contraction fed by TMA.  Per 32-coordinate slice one thread asks the
// TMA unit for the [128 points x 32] tile of x and the [32 directions x 32] tile
// of proj (128-byte swizzle; directions beyond L*S read as zero) into the next
// stage of a 2-stage ring while the CTA works on the current one: all threads
// split the landed tiles in place into the tf32 "hi" part and a separate "lo"
// tile (an elementwise pass, so the swizzle needs no decoding), then one thread
// issues the 4 x 3 MMAs (K-major, SWIZZLE_128B descriptors, K advanced by 32
// bytes inside the swizzle atom) and commits them to the stage's "empty"
// barrier, which the producer waits on before refilling it.
// Dynamic shared memory: 2 stages x (A raw/hi 16 KB + A lo 16 KB + B raw/hi 4 KB + B lo 4 KB)
// + 1 KB alignment slack.  Requires dim % 4 == 0 and 16-byte aligned x and proj.
constexpr int kTcStages = 2;
constexpr size_t kTcStageBytes = 2 * (kTcPoints * 128) + 2 * (kTcDirs * 128);
constexpr size_t kTcTmaSmem = kTcStages * kTcStageBytes + 1024;

// K-major, 128-byte swizzle: leading offset 1 (unused), stride (8 rows) 1024 bytes, version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024u >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ uint32_t mbar_wait(uint32_t bar, uint32_t parity) {
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < kTcWaitLimit && !done; ++spin) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
    }
    return done;
}

__global__ void __launch_bounds__(kTcPoints)
project_tf32x3_tma_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_p,
                          long long n, int dim, int num_indices, int i0, float *__restrict__ out, int *error) {
    extern __shared__ __align__(16) unsigned char tc_smem[];
    __shared__ __align__(8) unsigned long long full_bar[kTcStages], empty_bar[kTcStages];
    __shared__ uint32_t tmem_slot;

    const int tid = threadIdx.x, warp = tid >> 5;
    const long long p0 = (long long)blockIdx.x * kTcPoints;
    const uint32_t s0 = smem_u32(tc_smem);
    unsigned char *base = tc_smem + (((s0 + 1023u) & ~1023u) - s0);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)kTcDirs));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        for (int s_ = 0; s_ < kTcStages; ++s_) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[s_])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty_bar[s_])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTcDirs >> 3) << 17) |
                           ((uint32_t)(kTcPoints >> 4) << 24);
    const int nchunks = (dim + kTcK - 1) / kTcK;

    auto request = [&](int c) {          // thread 0: TMA loads of slice c into stage c % 2
        const int st = c % kTcStages;
        unsigned char *sb = base + (size_t)st * kTcStageBytes;
        const uint32_t bar = smem_u32(&full_bar[st]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                     "r"((uint32_t)(kTcPoints * 128 + kTcDirs * 128))
                     : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
                "r"(smem_u32(sb)), "l"(&map_x), "r"(c * kTcK), "r"((int)p0), "r"(bar)
            : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
                "r"(smem_u32(sb + 2 * kTcPoints * 128)), "l"(&map_p), "r"(c * kTcK), "r"(i0), "r"(bar)
            : "memory");
    };

    int failed = 0;
    uint32_t accumulate = 0;
    if (tid == 0) request(0);
    for (int c = 0; c < nchunks && !failed; ++c) {
        const int st = c % kTcStages;
        const uint32_t use = (uint32_t)(c / kTcStages);          // how often this stage was used before
        unsigned char *sb = base + (size_t)st * kTcStageBytes;
        // prefetch the next slice into the other stage once its previous MMAs have drained
        if (tid == 0 && c + 1 < nchunks) {
            const int nst = (c + 1) % kTcStages;
            const uint32_t nuse = (uint32_t)((c + 1) / kTcStages);
            uint32_t ok = 1;
            if (nuse > 0) ok = mbar_wait(smem_u32(&empty_bar[nst]), (nuse - 1) & 1u);
            if (ok) request(c + 1); else failed = 1;
        }
        if (!mbar_wait(smem_u32(&full_bar[st]), use & 1u)) failed = 1;
        // split in place: hi stays where the tile landed, lo goes to the tile next to it
        if (!failed) {
            float4 *a_hi = reinterpret_cast<float4 *>(sb), *a_lo = reinterpret_cast<float4 *>(sb + kTcPoints * 128);
            for (int f = tid; f < kTcPoints * 8; f += kTcPoints) {
                const float4 v = a_hi[f];
                float4 h, l;
                split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
                a_hi[f] = h; a_lo[f] = l;
            }
            float4 *b_hi = reinterpret_cast<float4 *>(sb + 2 * kTcPoints * 128);
            float4 *b_lo = reinterpret_cast<float4 *>(sb + 2 * kTcPoints * 128 + kTcDirs * 128);
            for (int f = tid; f < kTcDirs * 8; f += kTcPoints) {
                const float4 v = b_hi[f];
                float4 h, l;
                split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
                b_hi[f] = h; b_lo[f] = l;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        failed = __syncthreads_or(failed);
        if (failed) break;
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t ah = smem_u32(sb), al = ah + kTcPoints * 128, bh = ah + 2 * kTcPoints * 128, bl = bh + kTcDirs * 128;
#pragma unroll
            for (int kk = 0; kk < kTcK / 8; ++kk) {
                const uint32_t step = kk * 32;              // 8 coordinates = 32 bytes inside the 128-byte atom
                umma_tf32(tmem_d, umma_desc_sw128(al + step), umma_desc_sw128(bh + step), idesc, accumulate);
                accumulate = 1;
                umma_tf32(tmem_d, umma_desc_sw128(ah + step), umma_desc_sw128(bl + step), idesc, 1u);
                umma_tf32(tmem_d, umma_desc_sw128(ah + step), umma_desc_sw128(bh + step), idesc, 1u);
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&empty_bar[st]))
                         : "memory");
        }
    }
    // the last slice's MMAs must have finished before the accumulator is read
    if (!failed) {
        const int lc = nchunks - 1;
        if (!mbar_wait(smem_u32(&empty_bar[lc % kTcStages]), (uint32_t)(lc / kTcStages) & 1u)) failed = 1;
    }
    failed = __syncthreads_or(failed);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!failed) {
        uint32_t r[32];
        const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32"
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const long long p = p0 + tid;
        if (p < n) {
#pragma unroll
            for (int cidx = 0; cidx < kTcDirs; ++cidx)
                if (i0 + cidx < num_indices) out[(size_t)(i0 + cidx) * n + p] = __uint_as_float(r[cidx]);
        }
    } else if (tid == 0) {
        atomicExch(error, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)kTcDirs));
    }
}

// ---------------------------------------------------------------------------
// Persistent, warp-specialised form of the TMA-fed kernel.  One CTA per SM loops
// over 128-point tiles.  Roles:
//   warp 0, one lane  : producer -- TMA loads of the next 32-coordinate slice (points + directions)
//                       into a 4-stage ring, as soon as the stage's previous MMAs have drained;
//   warps 2..5        : epilogue -- once a tile's last MMAs are committed, read its accumulator
//                       from tensor memory and store the keys (the accumulator is double buffered,
//                       so the MMAs of the next tile run during these stores, and the converters
//                       never wait for an MMA);
//   warps 6..13       : converters -- split the landed slice into hi / lo tf32 tiles; eight warps
//                       with all their loads issued up front, because a conversion is a chain of
//                       shared-memory round trips and each scheduler only has two of these warps;
//   warp 1, one lane  : MMA issuer -- 4 x 3 tcgen05.mma per converted slice, committed to the
//                       stage's "empty" barrier, and after a tile's last slice to "accumulator full".
// All hand-offs are mbarriers; every wait is bounded and a time-out makes all roles leave.
constexpr int kPsStages = 5;
constexpr int kPsThreads = 448;
constexpr int kPsConverters = 256;
static_assert(kTcDirs * 8 == kPsConverters && (kTcPoints * 8) % kPsConverters == 0, "converter work split");
constexpr size_t kPsSmem = kPsStages * kTcStageBytes + 1024;

constexpr uint32_t kPsTmemCols = 256;   // 2 tiles x 3 accumulators x 32 columns, rounded up to a power of two

// 32 consecutive columns of this warp's 32 tensor-memory lanes -> 32 registers per thread
__device__ __forceinline__ void tmem_ld_32(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(kPsThreads, 1)
project_tf32x3_persistent_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_p,
                                 long long n, int dim, int num_indices, int i0, float *__restrict__ out, int *error) {
    extern __shared__ __align__(16) unsigned char tc_smem[];
    __shared__ __align__(8) unsigned long long full_bar[kPsStages], conv_bar[kPsStages], empty_bar[kPsStages];
    __shared__ __align__(8) unsigned long long acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t s0 = smem_u32(tc_smem);
    unsigned char *base = tc_smem + (((s0 + 1023u) & ~1023u) - s0);

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)kPsTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        abort_flag = 0;
        for (int s_ = 0; s_ < kPsStages; ++s_) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[s_])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&conv_bar[s_])), "r"(kPsConverters));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty_bar[s_])));
        }
        for (int a = 0; a < 2; ++a) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&acc_full[a])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 128;" ::"r"(smem_u32(&acc_empty[a])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    const int nchunks = (dim + kTcK - 1) / kTcK;
    const long long ntiles = (n + kTcPoints - 1) / kTcPoints;
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kTcDirs >> 3) << 17) |
                           ((uint32_t)(kTcPoints >> 4) << 24);

    if (warp == 0 && lane == 0) {
        // ---- producer
        uint32_t q = 0;                                   // slices requested so far
        for (long long tile = blockIdx.x; tile < ntiles && !abort_flag; tile += gridDim.x) {
            for (int c = 0; c < nchunks; ++c, ++q) {
                const int st = (int)(q % kPsStages);
                const uint32_t use = q / kPsStages;
                if (use > 0 && !mbar_wait(smem_u32(&empty_bar[st]), (use - 1) & 1u)) { abort_flag = 1; break; }
                unsigned char *sb = base + (size_t)st * kTcStageBytes;
                const uint32_t bar = smem_u32(&full_bar[st]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                             "r"((uint32_t)(kTcPoints * 128 + kTcDirs * 128))
                             : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
                        "r"(smem_u32(sb)), "l"(&map_x), "r"(c * kTcK), "r"((int)(tile * kTcPoints)), "r"(bar)
                    : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
                        "r"(smem_u32(sb + 2 * kTcPoints * 128)), "l"(&map_p), "r"(c * kTcK), "r"(i0), "r"(bar)
                    : "memory");
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        uint32_t q = 0, t = 0;
        for (long long tile = blockIdx.x; tile < ntiles && !abort_flag; tile += gridDim.x, ++t) {
            const int a = (int)(t & 1u);
            const uint32_t ause = t >> 1;                 // earlier tiles on this accumulator
            if (ause > 0 && !mbar_wait(smem_u32(&acc_empty[a]), (ause - 1) & 1u)) { abort_flag = 1; break; }
            // three accumulators per tile, one per product kind: MMAs into one accumulator run one
            // after the other, MMAs into different ones overlap
            const uint32_t tmem_d = tmem_base + (uint32_t)(a * 3 * kTcDirs);
            for (int c = 0; c < nchunks; ++c, ++q) {
                const int st = (int)(q % kPsStages);
                if (!mbar_wait(smem_u32(&conv_bar[st]), (q / kPsStages) & 1u)) { abort_flag = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t ah = smem_u32(base + (size_t)st * kTcStageBytes), al = ah + kTcPoints * 128,
                               bh = ah + 2 * kTcPoints * 128, bl = bh + kTcDirs * 128;
#pragma unroll
                for (int kk = 0; kk < kTcK / 8; ++kk) {
                    const uint32_t step = kk * 32;
                    const uint32_t acc = (c | kk) ? 1u : 0u;
                    umma_tf32(tmem_d, umma_desc_sw128(al + step), umma_desc_sw128(bh + step), idesc, acc);
                    umma_tf32(tmem_d + kTcDirs, umma_desc_sw128(ah + step), umma_desc_sw128(bl + step), idesc, acc);
                    umma_tf32(tmem_d + 2 * kTcDirs, umma_desc_sw128(ah + step), umma_desc_sw128(bh + step), idesc, acc);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&empty_bar[st]))
                             : "memory");
            }
            if (abort_flag) break;
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&acc_full[a]))
                         : "memory");
        }
    } else if (warp >= 6) {
        // ---- converters
        const int ct = tid - 192;
        constexpr int kA4 = kTcPoints * 8 / kPsConverters;      // float4 of the point tile per thread
        uint32_t q = 0;
        for (long long tile = blockIdx.x; tile < ntiles && !abort_flag; tile += gridDim.x) {
            for (int c = 0; c < nchunks; ++c, ++q) {
                const int st = (int)(q % kPsStages);
                if (!mbar_wait(smem_u32(&full_bar[st]), (q / kPsStages) & 1u)) { abort_flag = 1; break; }
                unsigned char *sb = base + (size_t)st * kTcStageBytes;
                float4 *a_hi = reinterpret_cast<float4 *>(sb), *a_lo = reinterpret_cast<float4 *>(sb + kTcPoints * 128);
                float4 *b_hi = reinterpret_cast<float4 *>(sb + 2 * kTcPoints * 128);
                float4 *b_lo = reinterpret_cast<float4 *>(sb + 2 * kTcPoints * 128 + kTcDirs * 128);
                float4 v[kA4 + 1];
#pragma unroll
                for (int u = 0; u < kA4; ++u) v[u] = a_hi[ct + u * kPsConverters];
                v[kA4] = b_hi[ct];                               // kTcDirs * 8 == kPsConverters
#pragma unroll
                for (int u = 0; u <= kA4; ++u) {
                    float4 h, l;
                    split_tf32(v[u].x, h.x, l.x); split_tf32(v[u].y, h.y, l.y);
                    split_tf32(v[u].z, h.z, l.z); split_tf32(v[u].w, h.w, l.w);
                    if (u < kA4) { a_hi[ct + u * kPsConverters] = h; a_lo[ct + u * kPsConverters] = l; }
                    else { b_hi[ct] = h; b_lo[ct] = l; }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(smem_u32(&conv_bar[st]));
            }
            if (abort_flag) break;
        }
    } else if (warp >= 2) {
        // ---- epilogue: 128 threads; warp w reads the tensor-memory lanes 32 * (w % 4) .. + 31
        uint32_t t = 0;
        for (long long tile = blockIdx.x; tile < ntiles && !abort_flag; tile += gridDim.x, ++t) {
            // epilogue of this tile
            const int a = (int)(t & 1u);
            if (!mbar_wait(smem_u32(&acc_full[a]), (t >> 1) & 1u)) { abort_flag = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[32], r1[32], r2[32];
            const uint32_t taddr = tmem_base + (uint32_t)(a * 3 * kTcDirs) + ((uint32_t)((warp & 3) * 32) << 16);
            tmem_ld_32(r, taddr);                    // lo x hi
            tmem_ld_32(r1, taddr + kTcDirs);         // hi x lo
            tmem_ld_32(r2, taddr + 2 * kTcDirs);     // hi x hi
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(smem_u32(&acc_empty[a]));
            const long long p = tile * kTcPoints + (warp & 3) * 32 + lane;     // TMEM lane = point of the tile
            if (p < n) {
#pragma unroll
                for (int cidx = 0; cidx < kTcDirs; ++cidx)
                    if (i0 + cidx < num_indices)     // small terms first
                        out[(size_t)(i0 + cidx) * n + p] =
                            (__uint_as_float(r[cidx]) + __uint_as_float(r1[cidx])) + __uint_as_float(r2[cidx]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && abort_flag) atomicExch(error, 1);
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kPsTmemCols));
    }
}

}  // namespace dci
