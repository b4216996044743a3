// Exact fp32 projection: out[i][p] = sum_k proj[i][k] * x[p][k], one fused
// multiply-add per term, k ascending, accumulator starting at +0.  This fixed
// order is the library's definition of a projected key; it replaces the
// cublasSgemm calls of the reference (src/util_kernel.cu:45-80, called from
// src/dci_cuda_kernel.cu:167-169 for data and :802-803 for queries).
// HBM-bound: reads 4*dim bytes and writes 4*L*S bytes per point.
#pragma once
#include "common.cuh"

namespace dci {

constexpr int kProjThreads = 128;  // threads per CTA
constexpr int kProjPerThread = 2;  // points per thread: a direction value read from shared memory feeds both
constexpr int kProjPoints = kProjThreads * kProjPerThread;   // points per CTA tile
constexpr int kProjK = 32;         // k-chunk staged through shared memory
constexpr int kProjPad = 36;       // row stride of the staged x tile: 16-byte aligned, conflict-free float4 reads

// Two fused multiply-adds in one instruction (sm_100 packed fp32): each half is an ordinary IEEE
// fma, so results do not change.
__device__ __forceinline__ void fma2(float2 &acc, const float2 a, const float2 b) {
    unsigned long long c = *reinterpret_cast<unsigned long long *>(&acc);
    asm("fma.rn.f32x2 %0, %1, %2, %0;"
        : "+l"(c)
        : "l"(*reinterpret_cast<const unsigned long long *>(&a)), "l"(*reinterpret_cast<const unsigned long long *>(&b)));
    acc = *reinterpret_cast<float2 *>(&c);
}

// Each thread owns two points (tid and tid + 128 of the tile) and DIRS accumulators for each,
// kept as pairs of neighbouring directions.  The directions are staged coordinate-major, so one
// 128-bit shared-memory load brings one coordinate of four directions: two packed operands that
// feed two packed multiply-adds per point with the point's coordinate in both halves.  A
// coordinate is finished for every direction before the next one starts, so every accumulator
// still adds its terms in ascending coordinate order and the result is unchanged; coordinates
// beyond the end of a row are zero in both operands and add nothing (an accumulator that starts
// at +0 is never -0).  DIRS is a multiple of 4.
template <int DIRS>
__global__ void __launch_bounds__(kProjThreads)
project_exact_kernel(const float *__restrict__ x, long long n, int dim,
                     const float *__restrict__ proj, int num_indices, float *__restrict__ out) {
    static_assert(DIRS % 4 == 0, "directions are handled four at a time");
    __shared__ __align__(16) float xs[kProjPoints][kProjPad];
    __shared__ __align__(16) float ps[kProjK][DIRS];
    const int tid = threadIdx.x;
    const long long p0 = (long long)blockIdx.x * kProjPoints;
    const bool vec_ok = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    for (int i0 = 0; i0 < num_indices; i0 += DIRS) {
        float2 acc[kProjPerThread][DIRS / 2];
#pragma unroll
        for (int u = 0; u < kProjPerThread; ++u)
#pragma unroll
            for (int d = 0; d < DIRS / 2; ++d) acc[u][d] = make_float2(0.0f, 0.0f);
        for (int k0 = 0; k0 < dim; k0 += kProjK) {
            const int kn = min(kProjK, dim - k0);
            // stage the x tile: 256 rows x 32 columns, 8 threads (float4 each) per row; columns
            // beyond the row's end are zero
            if (vec_ok) {
                const int c4 = (tid & 7) * 4;
                for (int r = tid >> 3; r < kProjPoints; r += kProjThreads / 8) {
                    const long long p = p0 + r;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p < n && c4 < kn)
                        v = __ldg(reinterpret_cast<const float4 *>(x + p * dim + k0 + c4));
                    *reinterpret_cast<float4 *>(&xs[r][c4]) = v;
                }
            } else {
                const int c = tid & 31;
                for (int r = tid >> 5; r < kProjPoints; r += kProjThreads / 32) {
                    const long long p = p0 + r;
                    xs[r][c] = (p < n && c < kn) ? __ldg(x + p * dim + k0 + c) : 0.0f;
                }
            }
            for (int e = tid; e < DIRS * kProjK; e += kProjThreads) {
                const int d = e / kProjK, c = e % kProjK;          // coalesced reads of the directions' rows
                ps[c][d] = (i0 + d < num_indices && c < kn) ? __ldg(proj + (size_t)(i0 + d) * dim + k0 + c) : 0.0f;
            }
            __syncthreads();
            const int kn4 = (kn + 3) & ~3;
            for (int c = 0; c < kn4; c += 4) {
                float4 xv[kProjPerThread];
#pragma unroll
                for (int u = 0; u < kProjPerThread; ++u)
                    xv[u] = *reinterpret_cast<const float4 *>(&xs[tid + u * kProjThreads][c]);
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    float2 xb[kProjPerThread];
#pragma unroll
                    for (int u = 0; u < kProjPerThread; ++u) {
                        const float v = cc == 0 ? xv[u].x : (cc == 1 ? xv[u].y : (cc == 2 ? xv[u].z : xv[u].w));
                        xb[u] = make_float2(v, v);
                    }
#pragma unroll
                    for (int d4 = 0; d4 < DIRS / 4; ++d4) {
                        const float4 pv = *reinterpret_cast<const float4 *>(&ps[c + cc][4 * d4]);
#pragma unroll
                        for (int u = 0; u < kProjPerThread; ++u) {
                            fma2(acc[u][2 * d4], make_float2(pv.x, pv.y), xb[u]);
                            fma2(acc[u][2 * d4 + 1], make_float2(pv.z, pv.w), xb[u]);
                        }
                    }
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int u = 0; u < kProjPerThread; ++u) {
            const long long p = p0 + tid + u * kProjThreads;
            if (p < n) {
#pragma unroll
                for (int d = 0; d < DIRS / 2; ++d) {
                    if (i0 + 2 * d < num_indices) out[(size_t)(i0 + 2 * d) * n + p] = acc[u][d].x;
                    if (i0 + 2 * d + 1 < num_indices) out[(size_t)(i0 + 2 * d + 1) * n + p] = acc[u][d].y;
                }
            }
        }
    }
}

}  // namespace dci
