// Exact fp32 projection fed by TMA: the same arithmetic as project_exact_kernel (one fused
// multiply-add per term, coordinates ascending, accumulators from +0, hence bit-identical keys), with
// the rows streamed through a ring of shared-memory stages by bulk tensor copies instead of being
// staged by the computing threads.  Replaces the cublasSgemm calls of the reference
// (src/util_kernel.cu:45-80, called from src/dci_cuda_kernel.cu:167-169 and :802-803).
//
// One CTA = 4 computing warps + 1 producer warp, persistent over tiles of 512 points (256 when more
// than 20 directions leave registers for two points per thread only); a thread owns four points, so
// that one 128-bit read of four directions from shared memory feeds eight packed multiply-adds.  A
// stage holds the tile's rows x 16 coordinates as TMA boxes of 256 rows (64-byte rows with the 64-byte
// swizzle, so that the threads' 16-byte reads of different rows fall on different banks).  The
// producer's elected lane waits for a free stage and issues the copies of a (tile, 16-coordinate
// slice); the computing warps wait for the slice, add it to their accumulators and release the stage
// (one arrival per warp).  The directions are kept in shared memory for the whole launch,
// coordinate-major.  4*dim bytes in and 4*L*S bytes out per point, nothing read twice; measured with
// 20 directions the copies alone run at 0.87 of the HBM copy rate, the arithmetic alone (2 warps per
// scheduler, fp32 pipe 57-62 % busy) at 0.75, both together at 0.68.
//
// Every wait is bounded: a wait that runs out sets *error, and the CTA stops issuing copies, waits
// (bounded again) for the copies it has in flight and leaves.
#pragma once
#include "project.cuh"
#include "project_tf32.cuh"

namespace dci {

constexpr int kPxBoxRows = 256;                    // rows of a TMA box
constexpr int kPxCols = 16;                        // coordinates per stage (64-byte rows)
constexpr int kPxComputeWarps = 4;
constexpr int kPxThreads = (kPxComputeWarps + 1) * 32;
constexpr int kPxMaxStages = 8;
// points per thread: four while the accumulators fit the registers of two CTAs per SM, else two
__host__ __device__ constexpr int px_per_thread(int dirs) { return dirs <= 20 ? 4 : 2; }
__host__ __device__ constexpr int px_rows(int dirs) { return px_per_thread(dirs) * kPxComputeWarps * 32; }   // points per tile
__host__ __device__ constexpr int px_stage_bytes(int dirs) { return px_rows(dirs) * kPxCols * 4; }           // 32 or 16 KB

__host__ __device__ inline size_t px_dirs_bytes(int dim, int dirs) {
    return (size_t)((dim + kPxCols - 1) / kPxCols * kPxCols) * dirs * sizeof(float);
}
__host__ __device__ inline size_t px_smem_bytes(int dim, int dirs, int stages) {
    return 1024 + (size_t)stages * px_stage_bytes(dirs) + px_dirs_bytes(dim, dirs);
}

template <int DIRS>
__global__ void __launch_bounds__(kPxThreads, DIRS <= 32 ? 2 : 1)
project_exact_tma_kernel(const __grid_constant__ CUtensorMap map_x, long long n, int dim,
                         const float *__restrict__ proj, int num_indices, int stages, float *__restrict__ out,
                         int *error) {
    static_assert(DIRS % 4 == 0, "directions are handled four at a time");
    constexpr int kPxPerThread = px_per_thread(DIRS), kPxRows = px_rows(DIRS), kPxStageBytes = px_stage_bytes(DIRS);
    constexpr int kPxBoxes = kPxRows / kPxBoxRows;
    extern __shared__ __align__(16) unsigned char px_smem[];
    __shared__ __align__(8) unsigned long long full_bar[kPxMaxStages], empty_bar[kPxMaxStages];
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t s0 = smem_u32(px_smem);
    unsigned char *base = px_smem + (((s0 + 1023u) & ~1023u) - s0);          // stages start on a 1024-byte boundary
    float *ps = reinterpret_cast<float *>(base + (size_t)stages * kPxStageBytes);   // [dim rounded up to 16][DIRS]
    const int nchunks = (dim + kPxCols - 1) / kPxCols;
    const long long ntiles = (n + kPxRows - 1) / kPxRows;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&empty_bar[s])), "r"(kPxComputeWarps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
    }
    // directions, coordinate-major; coordinates beyond dim and directions beyond num_indices are zero
    for (int e = tid; e < DIRS * nchunks * kPxCols; e += kPxThreads) {
        const int d = e / (nchunks * kPxCols), c = e - d * (nchunks * kPxCols);          // coalesced reads of a direction's row
        ps[(size_t)c * DIRS + d] = (d < num_indices && c < dim) ? __ldg(proj + (size_t)d * dim + c) : 0.0f;
    }
    __syncthreads();

    if (warp == kPxComputeWarps) {
        // ---- producer
        if (lane == 0) {
            uint32_t it = 0;
            int issued_ok = 1;
            for (long long tile = blockIdx.x; tile < ntiles && issued_ok; tile += gridDim.x) {
                for (int c = 0; c < nchunks; ++c, ++it) {
                    const int s = (int)(it % (uint32_t)stages);
                    const uint32_t use = it / (uint32_t)stages;
                    if (use > 0 && !mbar_wait(smem_u32(&empty_bar[s]), (use - 1u) & 1u)) { issued_ok = 0; break; }
                    if (*reinterpret_cast<volatile int *>(&s_abort)) { issued_ok = 0; break; }
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                                 "r"((uint32_t)kPxStageBytes)
                                 : "memory");
#pragma unroll
                    for (int bx = 0; bx < kPxBoxes; ++bx)
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
                                "r"(smem_u32(base + (size_t)s * kPxStageBytes + (size_t)bx * kPxBoxRows * kPxCols * 4)), "l"(&map_x),
                            "r"(c * kPxCols), "r"((int)(tile * kPxRows + bx * kPxBoxRows)), "r"(bar)
                            : "memory");
                }
            }
            if (!issued_ok) {
                atomicExch(error, 1);
                *reinterpret_cast<volatile int *>(&s_abort) = 1;
            }
        }
    } else {
        // ---- computing warps: thread t owns rows t, t + (number of computing threads), ... of every tile
        const uint32_t sw = (uint32_t)(tid >> 1) & 3u;                // 64-byte swizzle term of all its rows (their distance is 0 mod 8)
        uint32_t it = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            float2 acc[kPxPerThread][DIRS / 2];
#pragma unroll
            for (int u = 0; u < kPxPerThread; ++u)
#pragma unroll
                for (int d = 0; d < DIRS / 2; ++d) acc[u][d] = make_float2(0.0f, 0.0f);
            for (int c = 0; c < nchunks; ++c, ++it) {
                const int s = (int)(it % (uint32_t)stages);
                if (!mbar_wait(smem_u32(&full_bar[s]), (it / (uint32_t)stages) & 1u)) { ok = false; break; }
                const unsigned char *row0 = base + (size_t)s * kPxStageBytes + (size_t)tid * (kPxCols * 4);
                const float *pc = ps + (size_t)c * kPxCols * DIRS;
#pragma unroll 2
                for (int j = 0; j < kPxCols / 4; ++j) {               // 16-byte pieces of the 64-byte row slice
                    const uint32_t off = ((uint32_t)j ^ sw) << 4;
                    float4 xv[kPxPerThread];
#pragma unroll
                    for (int u = 0; u < kPxPerThread; ++u)
                        xv[u] = *reinterpret_cast<const float4 *>(row0 + (size_t)u * (kPxComputeWarps * 32) * (kPxCols * 4) + off);
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        float2 xb[kPxPerThread];
#pragma unroll
                        for (int u = 0; u < kPxPerThread; ++u) {
                            const float v = cc == 0 ? xv[u].x : (cc == 1 ? xv[u].y : (cc == 2 ? xv[u].z : xv[u].w));
                            xb[u] = make_float2(v, v);
                        }
                        const float *pd = pc + (size_t)(4 * j + cc) * DIRS;
#pragma unroll
                        for (int d4 = 0; d4 < DIRS / 4; ++d4) {
                            const float4 pv = *reinterpret_cast<const float4 *>(pd + 4 * d4);
#pragma unroll
                            for (int u = 0; u < kPxPerThread; ++u) {
                                fma2(acc[u][2 * d4], make_float2(pv.x, pv.y), xb[u]);
                                fma2(acc[u][2 * d4 + 1], make_float2(pv.z, pv.w), xb[u]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
            }
            if (!ok) break;
#pragma unroll
            for (int u = 0; u < kPxPerThread; ++u) {
                const long long p = tile * kPxRows + tid + u * (kPxComputeWarps * 32);
                if (p < n) {
#pragma unroll
                    for (int d = 0; d < DIRS / 2; ++d) {
                        if (2 * d < num_indices) out[(size_t)(2 * d) * n + p] = acc[u][d].x;
                        if (2 * d + 1 < num_indices) out[(size_t)(2 * d + 1) * n + p] = acc[u][d].y;
                    }
                }
            }
        }
        if (!ok) {
            atomicExch(error, 1);
            *reinterpret_cast<volatile int *>(&s_abort) = 1;
        }
    }
    // Nobody leaves while a copy may still be on its way into this CTA's shared memory: after a
    // failed wait the copies already issued are given one more bounded wait each.
    __syncthreads();
    if (*reinterpret_cast<volatile int *>(&s_abort) && tid == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_wait(smem_u32(&full_bar[s]), 0u);
            mbar_wait(smem_u32(&full_bar[s]), 1u);
        }
    }
}

}  // namespace dci
