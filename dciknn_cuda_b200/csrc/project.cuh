// Exact fp32 projection: out[i][p] = sum_k proj[i][k] * x[p][k], one fused
// multiply-add per term, k ascending, accumulator starting at +0.  This fixed
// order is the library's definition of a projected key; it replaces the
// cublasSgemm calls of the reference (src/util_kernel.cu:45-80, called from
// src/dci_cuda_kernel.cu:167-169 for data and :802-803 for queries).
// HBM-bound: reads 4*dim bytes and writes 4*L*S bytes per point.
#pragma once
#include "common.cuh"

namespace dci {

constexpr int kProjPoints = 128;   // points per CTA tile (one per thread)
constexpr int kProjK = 32;         // k-chunk staged through shared memory
constexpr int kProjPad = 36;       // row stride of the staged x tile: 16-byte aligned, conflict-free float4 reads

// Each thread owns one point and DIRS accumulators.  Both operands are read from
// shared memory four coordinates at a time (one 128-bit load of the point's
// row, one broadcast 128-bit load per direction), so a load feeds four
// multiply-adds and the kernel is limited by HBM / the FMA pipe, not by shared
// memory issue.  The four products of a load are still added in ascending
// coordinate order, so the result is unchanged.
template <int DIRS>
__global__ void __launch_bounds__(kProjPoints)
project_exact_kernel(const float *__restrict__ x, long long n, int dim,
                     const float *__restrict__ proj, int num_indices, float *__restrict__ out) {
    __shared__ __align__(16) float xs[kProjPoints][kProjPad];
    __shared__ __align__(16) float ps[DIRS][kProjK];
    const int tid = threadIdx.x;
    const long long p0 = (long long)blockIdx.x * kProjPoints;
    const bool vec_ok = (dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    for (int i0 = 0; i0 < num_indices; i0 += DIRS) {
        float acc[DIRS];
#pragma unroll
        for (int d = 0; d < DIRS; ++d) acc[d] = 0.0f;
        for (int k0 = 0; k0 < dim; k0 += kProjK) {
            const int kn = min(kProjK, dim - k0);
            // stage the x tile: 128 rows x 32 columns, 8 threads (float4 each) per row; columns
            // beyond the row's end are zero (a zero product leaves the sum unchanged)
            if (vec_ok) {
                const int c4 = (tid & 7) * 4;
                for (int r = tid >> 3; r < kProjPoints; r += kProjPoints / 8) {
                    const long long p = p0 + r;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p < n && c4 < kn)
                        v = __ldg(reinterpret_cast<const float4 *>(x + p * dim + k0 + c4));
                    *reinterpret_cast<float4 *>(&xs[r][c4]) = v;
                }
            } else {
                const int c = tid & 31;
                for (int r = tid >> 5; r < kProjPoints; r += kProjPoints / 32) {
                    const long long p = p0 + r;
                    xs[r][c] = (p < n && c < kn) ? __ldg(x + p * dim + k0 + c) : 0.0f;
                }
            }
            for (int e = tid; e < DIRS * kProjK; e += kProjPoints) {
                const int d = e / kProjK, c = e % kProjK;
                ps[d][c] = (i0 + d < num_indices && c < kn) ? __ldg(proj + (size_t)(i0 + d) * dim + k0 + c) : 0.0f;
            }
            __syncthreads();
            const int kn4 = (kn + 3) & ~3;
            for (int c = 0; c < kn4; c += 4) {
                const float4 xv = *reinterpret_cast<const float4 *>(&xs[tid][c]);
#pragma unroll
                for (int d = 0; d < DIRS; ++d) {
                    const float4 pv = *reinterpret_cast<const float4 *>(&ps[d][c]);
                    float a = acc[d];
                    a = __fmaf_rn(pv.x, xv.x, a);
                    if (c + 1 < kn) a = __fmaf_rn(pv.y, xv.y, a);
                    if (c + 2 < kn) a = __fmaf_rn(pv.z, xv.z, a);
                    if (c + 3 < kn) a = __fmaf_rn(pv.w, xv.w, a);
                    acc[d] = a;
                }
            }
            __syncthreads();
        }
        const long long p = p0 + tid;
        if (p < n) {
#pragma unroll
            for (int d = 0; d < DIRS; ++d)
                if (i0 + d < num_indices) out[(size_t)(i0 + d) * n + p] = acc[d];
        }
    }
}

}  // namespace dci
