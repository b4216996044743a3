// Projection directions: L*S rows of `dim` i.i.d. standard normals, each row
// scaled to unit length.  Replaces dci_gen_proj_vec / normalize_proj_vecs
// (reference src/dci_cuda_kernel.cu:52-90) and the cuRAND XORWOW fill
// (src/util_kernel.cu:82-101, 119-137) with a counter-based generator, so a row
// depends only on (seed, row, column).
#pragma once
#include "common.cuh"

namespace dci {

// Philox-4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy
// as 1, 2, 3", SC'11), written from the published description.
__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
        const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += W0; k1 += W1;
    }
}

// One CTA per direction row.
__global__ void gen_directions_kernel(float *proj, int dim, unsigned long long seed) {
    const int row = blockIdx.x;
    float *out = proj + (size_t)row * dim;
    __shared__ float red[32];
    float sq = 0.0f;
    for (int q4 = threadIdx.x; q4 * 4 < dim; q4 += blockDim.x) {
        uint32_t c[4] = {(uint32_t)q4, (uint32_t)row, 0x44434931u, 0u};
        philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
        float z[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {   // Box-Muller on two uniforms in (0, 1]
            const float u1 = ((float)(c[2 * h] >> 8) + 1.0f) * (1.0f / 16777216.0f);
            const float u2 = ((float)(c[2 * h + 1] >> 8) + 0.5f) * (1.0f / 16777216.0f);
            const float rad = sqrtf(-2.0f * logf(u1));
            float sn, cs;
            sincospif(2.0f * u2, &sn, &cs);
            z[2 * h] = rad * cs;
            z[2 * h + 1] = rad * sn;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = q4 * 4 + j;
            if (col < dim) { out[col] = z[j]; sq += z[j] * z[j]; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (threadIdx.x == 0) red[0] = sqrtf(v);
    }
    __syncthreads();
    const float norm = red[0];
    for (int col = threadIdx.x; col < dim; col += blockDim.x) out[col] = out[col] / norm;
}

}  // namespace dci
