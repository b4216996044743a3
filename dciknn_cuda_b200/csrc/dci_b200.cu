// C ABI and host orchestration of the B200-native Prioritized DCI engine.
// The declarations and their relation to the reference's API are in
// include/dci_b200.h.  Replaces the host side of the reference:
// dci_init/dci_add/dci_query/dci_clear/dci_reset/dci_free
// (src/dci_cuda_kernel.cu:93-110, 149-187, 777-899) and the Torch shim
// (src/dci_cuda.cpp:54-173).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <new>

#include "../../include/dci_b200.h"
#include "build_index.cuh"
#include "common.cuh"
#include "directions.cuh"
#include "project.cuh"
#include "project_tf32.cuh"
#include "project_exact_tma.cuh"
#include "traverse.cuh"

namespace {

thread_local char g_err[1024] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define DCI_CUDA(call)                                                                     \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess)                                                             \
            return fail(DCI_B200_ERR_CUDA, "%s failed at %s:%d: %s", #call, __FILE__,      \
                        __LINE__, cudaGetErrorString(e_));                                 \
    } while (0)

// every cudaMalloc / cudaFree this library issues goes through these two (dci_b200_device_alloc_calls)
std::atomic<long long> g_alloc_calls{0};
cudaError_t counted_malloc(void **p, size_t bytes) { ++g_alloc_calls; return cudaMalloc(p, bytes); }
cudaError_t counted_free(void *p) { ++g_alloc_calls; return cudaFree(p); }

struct Buf {
    void *p = nullptr;
    size_t cap = 0;
    cudaError_t ensure(size_t bytes) {
        if (bytes <= cap) return cudaSuccess;
        if (p) { counted_free(p); p = nullptr; cap = 0; }
        cudaError_t e = counted_malloc(&p, bytes);
        if (e == cudaSuccess) cap = bytes;
        return e;
    }
    void release() { if (p) counted_free(p); p = nullptr; cap = 0; }
};

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) return;
        ok = (prev == dev) || cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

int next_pow2(int x) { int p = 1; while (p < x) p <<= 1; return p; }

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Tensor map over a row-major fp32 matrix [rows][dim] with boxes of [box_rows][box_cols = 32 or 16] and
// the swizzle of that row width; out-of-range elements read as zero.
bool make_tensor_map_2d(CUtensorMap *map, const float *ptr, long long rows, int dim, int box_rows, int box_cols = 32) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn || dim % 4 != 0 || ((uintptr_t)ptr & 15) != 0 || box_rows < 1 || box_rows > 256 || rows < 1) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)dim, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)dim * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    // the swizzle spans a box row: 128 bytes for 32 columns, 64 bytes for 16
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)ptr, dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

struct dci_b200 {
    int dim = 0, L = 0, S = 0, device = 0;
    int num_points = 0, P = 0, T = 0, ppb = 0, num_parts = 0;
    const float *d_data = nullptr;       // borrowed
    float *d_proj = nullptr;             // [L*S][dim]
    int *d_copyflag = nullptr;           // set (and left set) by a TMA-fed kernel whose bounded wait ran out
    int exact_tma = 1;                   // 0: never use the TMA-fed exact projection
    Buf keys, ids, pos, keysT;           // sorted index, inverse positions, stride-T keys: L*S*N entries each, partition-major (segment_start)
    int max_ctas = 0;                    // > 0: cap on the traversal grid (dci_b200_set_max_ctas)
    Buf tmp_keys, qproj, part_topk, scratch, merge_scratch, stats, phases, hq, hids, hdists, qbound;
    int distance_bound = 1;              // 1: share a per-query distance bound between partitions
    int stats_on = 0, stats_nq = 0, phases_valid = 0;
    int timing_on = 0;
    int last_qbatch = 1;                 // queries per CTA pass of the last traversal launch
    int last_projection_tma = 0;
    int projection_mode = 0;             // 0: exact fp32 FMA order, 1: tensor cores, 3xTF32
    Buf errflag;
    cudaEvent_t ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t pev[2] = {nullptr, nullptr};   // around the kernels of the last projection (timing mode)
    int pev_valid = 0;
    float t_project = 0.f, t_traverse = 0.f, t_merge = 0.f;
    int t_traverse_launches = 0;
    long long launches = 0;
    int sm_count = 0;
    size_t smem_optin = 0, smem_per_sm = 0;
};

namespace {

int launch_directions(dci_b200 *h, unsigned long long seed, cudaStream_t st) {
    dci::gen_directions_kernel<<<h->L * h->S, 128, 0, st>>>(h->d_proj, h->dim, seed);
    h->launches++;
    DCI_CUDA(cudaGetLastError());
    return 0;
}

// flag_word: device word for the tensor-core kernels' bounded-wait flag; nullptr = the handle's own
// (allocated on first use).  allow_timing = false keeps the timing events (created on first use) out.
int launch_project(dci_b200 *h, const float *d_x, long long n, float *d_out, cudaStream_t st,
                   int *flag_word = nullptr, bool allow_timing = true) {
    if (n <= 0) return 0;
    const int I = h->L * h->S;
    struct KernelTimer {       // timing mode: events right around the kernel launches, after the host-side set-up
        dci_b200 *h; cudaStream_t st; bool on; bool allow;
        void start() {
            on = h->timing_on != 0 && allow;
            h->pev_valid = 0;
            if (!on) return;
            for (auto &e : h->pev) if (!e && cudaEventCreate(&e) != cudaSuccess) { on = false; return; }
            cudaEventRecord(h->pev[0], st);
        }
        void stop() { if (on && cudaEventRecord(h->pev[1], st) == cudaSuccess) h->pev_valid = 1; }
    } timer{h, st, false, allow_timing};
    if (h->projection_mode != 0) {
        if (!flag_word) {
            DCI_CUDA(h->errflag.ensure(sizeof(int)));
            flag_word = (int *)h->errflag.p;
        }
        DCI_CUDA(cudaMemsetAsync(flag_word, 0, sizeof(int), st));
        const unsigned tgrid = (unsigned)((n + dci::kTcPoints - 1) / dci::kTcPoints);
        CUtensorMap map_x, map_p;
        const bool tma = h->projection_mode != 2 && make_tensor_map_2d(&map_x, d_x, n, h->dim, dci::kTcPoints) &&
                         make_tensor_map_2d(&map_p, h->d_proj, I, h->dim, dci::kTcDirs);
        const bool persistent = tma && h->projection_mode == 1;
        if (persistent)
            DCI_CUDA(cudaFuncSetAttribute(dci::project_tf32x3_persistent_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dci::kPsSmem));
        else if (tma)
            DCI_CUDA(cudaFuncSetAttribute(dci::project_tf32x3_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)dci::kTcTmaSmem));
        h->last_projection_tma = tma ? 1 : 0;
        timer.start();
        for (int i0 = 0; i0 < I; i0 += dci::kTcDirs) {
            if (persistent)
                dci::project_tf32x3_persistent_kernel<<<std::min<unsigned>(tgrid, (unsigned)h->sm_count), dci::kPsThreads,
                                                        dci::kPsSmem, st>>>(map_x, map_p, n, h->dim, I, i0, d_out,
                                                                            flag_word);
            else if (tma)
                dci::project_tf32x3_tma_kernel<<<tgrid, dci::kTcPoints, dci::kTcTmaSmem, st>>>(
                    map_x, map_p, n, h->dim, I, i0, d_out, flag_word);
            else
                dci::project_tf32x3_kernel<<<tgrid, dci::kTcPoints, 0, st>>>(d_x, n, h->dim, h->d_proj, I, i0, d_out,
                                                                           flag_word);
            h->launches++;
            DCI_CUDA(cudaGetLastError());
        }
        timer.stop();
        int flag = 0;      // this mode checks its bounded waits before going on
        DCI_CUDA(cudaMemcpyAsync(&flag, flag_word, sizeof(int), cudaMemcpyDeviceToHost, st));
        DCI_CUDA(cudaStreamSynchronize(st));
        if (flag) return fail(DCI_B200_ERR_CUDA, "tensor-core projection: a wait on the MMA barrier timed out");
        return 0;
    }
    // Large inputs take the TMA-fed kernel when the rows can be described by a tensor map (dim a multiple
    // of 4, 16-byte aligned base), one pass covers all directions and they fit in shared memory beside at
    // least two stages; everything else takes the kernel that stages the rows itself.  Same arithmetic.
    if (h->exact_tma && I <= 40 && n >= 1024) {
        const int dirs = I <= 8 ? 8 : (I <= 12 ? 12 : (I <= 20 ? 20 : (I <= 32 ? 32 : 40)));
        const size_t dbytes = dci::px_dirs_bytes(h->dim, dirs);
        const long long stage = dci::px_stage_bytes(dirs);
        const long long per_cta2 = (long long)h->smem_per_sm / 2 - 1024 - 1024 - 512 - (long long)dbytes;   // two CTAs per SM
        const long long per_cta1 = (long long)h->smem_optin - 1024 - 512 - (long long)dbytes;
        int stages = 0, per_sm = 0;
        if (per_cta2 >= 3 * stage) { stages = (int)std::min<long long>(4, per_cta2 / stage); per_sm = 2; }
        else if (per_cta1 >= 2 * stage) { stages = (int)std::min<long long>(dci::kPxMaxStages, per_cta1 / stage); per_sm = 1; }
        CUtensorMap map_x;
        if (stages && make_tensor_map_2d(&map_x, d_x, n, h->dim, dci::kPxBoxRows, dci::kPxCols)) {
            const size_t dyn = dci::px_smem_bytes(h->dim, dirs, stages);
            const long long ntiles = (n + dci::px_rows(dirs) - 1) / dci::px_rows(dirs);
            const unsigned pgrid = (unsigned)std::min<long long>(ntiles, (long long)h->sm_count * per_sm);
            auto go = [&](auto kern) -> int {
                DCI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
                timer.start();
                kern<<<pgrid, dci::kPxThreads, dyn, st>>>(map_x, n, h->dim, h->d_proj, I, stages, d_out, h->d_copyflag);
                timer.stop();
                h->launches++;
                DCI_CUDA(cudaGetLastError());
                h->last_projection_tma = 1;
                return 0;
            };
            switch (dirs) {
                case 8: return go(dci::project_exact_tma_kernel<8>);
                case 12: return go(dci::project_exact_tma_kernel<12>);
                case 20: return go(dci::project_exact_tma_kernel<20>);
                case 32: return go(dci::project_exact_tma_kernel<32>);
                default: return go(dci::project_exact_tma_kernel<40>);
            }
        }
    }
    h->last_projection_tma = 0;
    const unsigned grid = (unsigned)((n + dci::kProjPoints - 1) / dci::kProjPoints);
    timer.start();
    // fewest passes over the points, then the smallest accumulator count that achieves it
    if (I <= 8)
        dci::project_exact_kernel<8><<<grid, dci::kProjThreads, 0, st>>>(d_x, n, h->dim, h->d_proj, I, d_out);
    else if (I <= 12)
        dci::project_exact_kernel<12><<<grid, dci::kProjThreads, 0, st>>>(d_x, n, h->dim, h->d_proj, I, d_out);
    else if (I <= 20)
        dci::project_exact_kernel<20><<<grid, dci::kProjThreads, 0, st>>>(d_x, n, h->dim, h->d_proj, I, d_out);
    else if (I <= 32)
        dci::project_exact_kernel<32><<<grid, dci::kProjThreads, 0, st>>>(d_x, n, h->dim, h->d_proj, I, d_out);
    else
        dci::project_exact_kernel<40><<<grid, dci::kProjThreads, 0, st>>>(d_x, n, h->dim, h->d_proj, I, d_out);
    timer.stop();
    h->launches++;
    DCI_CUDA(cudaGetLastError());
    return 0;
}

template <typename ValT>
int launch_build(dci_b200 *h, const float *d_unsorted, cudaStream_t st) {
    const int I = h->L * h->S;
    const int nthreads = h->ppb >= 4096 ? 1024 : (h->ppb >= 1024 ? 512 : 256);
    const long long nseg = (long long)I * h->num_parts;
    cudaFuncAttributes fa;
    DCI_CUDA(cudaFuncGetAttributes(&fa, dci::build_segments_kernel<ValT, true>));
    // the opt-in limit covers static + dynamic shared memory, and the driver reserves 1 KB per CTA
    const size_t static_smem = fa.sharedSizeBytes + 1024;
    // buckets of the counting rank: two per key, one per key, or none (radix sort only), whichever fits
    int nbuckets = 0;
    auto lay = dci::BuildLayout<ValT>::make(nthreads, h->ppb, 0);
    for (int nb : {2 * h->ppb, h->ppb}) {
        if (nb < 64 || sizeof(ValT) != 2 || nb > 65535 * 2) continue;      // 16-bit packed counters only
        const auto l2 = dci::BuildLayout<ValT>::make(nthreads, h->ppb, nb);
        if (l2.hist_bytes + l2.slot_bytes + l2.buf_bytes + static_smem <= h->smem_optin) { nbuckets = nb; lay = l2; break; }
    }
    const bool smem = lay.hist_bytes + lay.slot_bytes + lay.buf_bytes + static_smem <= h->smem_optin;
    if (smem) {
        auto kern = dci::build_segments_kernel<ValT, true>;
        const size_t dyn = lay.hist_bytes + lay.slot_bytes + lay.buf_bytes;
        DCI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
        int per_sm = (int)std::max<size_t>(1, std::min<size_t>(h->smem_per_sm / (dyn + 1024), 2048 / nthreads));
        const unsigned grid = (unsigned)std::min<long long>(nseg, (long long)h->sm_count * per_sm);
        kern<<<grid, nthreads, dyn, st>>>(d_unsorted, h->num_points, I, h->ppb, h->num_parts,
                                          (float *)h->keys.p, (int *)h->ids.p, (ValT *)h->pos.p, (float *)h->keysT.p, h->T,
                                          nullptr, 0, nbuckets);
    } else {
        auto kern = dci::build_segments_kernel<ValT, false>;
        const unsigned grid = (unsigned)std::min<long long>(nseg, (long long)h->sm_count * (2048 / nthreads));
        DCI_CUDA(h->scratch.ensure(lay.buf_bytes * grid));
        kern<<<grid, nthreads, lay.hist_bytes, st>>>(d_unsorted, h->num_points, I, h->ppb, h->num_parts,
                                                     (float *)h->keys.p, (int *)h->ids.p, (ValT *)h->pos.p,
                                                     (float *)h->keysT.p, h->T,
                                                     (unsigned char *)h->scratch.p, lay.buf_bytes, 0);
    }
    h->launches++;
    DCI_CUDA(cudaGetLastError());
    return 0;
}

// Number of value buckets for the window ordering: as many as twice the windows
// of a composite index (so that most buckets hold at most one window) while the
// whole work item still fits shared memory, else fewer.
template <typename ValT>
int pick_buckets(dci_b200 *h, dci::TraverseParams &prm, int nthreads, size_t static_smem) {
    // first choice: twice as many buckets as windows and a bucket-ordered copy of the keys
    const int choices[4] = {2 * prm.wcap, 2 * prm.wcap, prm.wcap, prm.wcap / 2};
    for (int c = 0; c < 4; ++c) {
        const int nb = std::min(std::max(choices[c], 64), 1 << 20);
        const auto lay = dci::TraverseLayout<ValT>::make(nthreads, prm.dim, prm.topk_global ? 0 : prm.topk_cap, prm.L,
                                                         prm.wcap, prm.ppb, nb, prm.vec4 && !prm.vec8, c == 0);
        if (lay.fixed_bytes + lay.big_bytes + static_smem <= h->smem_optin) { prm.bkey = c == 0 ? 1 : 0; return nb; }
    }
    prm.bkey = 1;      // the work arrays live in the CTA's global slab: room is no concern, sequential access matters more
    return std::min(std::max(prm.wcap / 2, 64), 16384);
}

template <typename ValT, typename PosT>
int launch_traverse(dci_b200 *h, dci::TraverseParams prm, int nthreads, cudaStream_t st) {
    cudaFuncAttributes fa;
    DCI_CUDA(cudaFuncGetAttributes(&fa, dci::traverse_kernel<ValT, PosT, true, true>));
    const size_t static_smem = fa.sharedSizeBytes;
    prm.nbuckets = pick_buckets<ValT>(h, prm, nthreads, static_smem);
    const int cap_smem = prm.topk_global ? 0 : prm.topk_cap;
    auto lay = dci::TraverseLayout<ValT>::make(nthreads, prm.dim, cap_smem, prm.L, prm.wcap, prm.ppb, prm.nbuckets,
                                               prm.vec4 && !prm.vec8, prm.bkey != 0);
    if (lay.fixed_bytes + static_smem > h->smem_optin)
        return fail(DCI_B200_ERR_UNSUPPORTED, "dim=%d with k=%d needs %zu bytes of shared memory per CTA, more than the device offers",
                    prm.dim, prm.knn, lay.fixed_bytes + static_smem);
    const bool smem = lay.fixed_bytes + lay.big_bytes + static_smem <= h->smem_optin;
    if (!smem) lay = dci::TraverseLayout<ValT>::make(nthreads, prm.dim, cap_smem, prm.L, prm.wcap, prm.ppb, prm.nbuckets, false, prm.bkey != 0);
    const size_t dyn = smem ? lay.fixed_bytes + lay.big_bytes : lay.fixed_bytes;
    // queries per CTA pass: the dense distance pass needs, per query, a pair of selection buffers
    // and the query vector inside the shared "big" region
    // ... and pays off when work items are exhaustive: lane 0 of a partition sees about ppb / T
    // promotions, so a quota well above that (with an iteration cap beyond the last window) is never met
    prm.qbatch = 1;
    const bool likely_exhaustive = (long long)prm.max_cand * prm.T * 2 > 3ll * prm.ppb && prm.outer_s >= prm.wcap;
    if (smem && prm.vec8 && !prm.topk_global && !prm.blind && likely_exhaustive) {
        prm.dense_cap = next_pow2(prm.kpart + nthreads / 4);
        // per query a pair of selection buffers; for the group the query vectors, always kMaxQBatch slots
        // per coordinate
        const size_t per_q = (size_t)prm.dense_cap * 16 + 16, dq_bytes = (size_t)prm.dim * 4 * dci::kMaxQBatch;
        prm.qbatch = lay.big_bytes > dq_bytes
                         ? (int)std::max<size_t>(1, std::min<size_t>(dci::kMaxQBatch, (lay.big_bytes - dq_bytes) / per_q))
                         : 1;
    }
    prm.topk_global_off = lay.fallback_bytes + (smem ? 0 : lay.big_bytes);
    const size_t per_cta = prm.topk_global_off + (prm.topk_global ? (size_t)prm.topk_cap * 16 : 0);
    const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(h->smem_per_sm / (dyn + static_smem + 1024), 2048 / nthreads));
    h->last_qbatch = prm.qbatch;
    const long long nwork = (long long)((prm.nq + prm.qbatch - 1) / prm.qbatch) * prm.num_parts;
    unsigned grid = (unsigned)std::min<long long>(nwork, (long long)h->sm_count * per_sm);
    if (h->max_ctas > 0) grid = std::min(grid, (unsigned)h->max_ctas);
    DCI_CUDA(h->scratch.ensure(per_cta * grid));
    prm.gscratch = (unsigned char *)h->scratch.p;
    prm.gscratch_per_cta = per_cta;
    // the common case has kernel instances of its own, without the code of the rarer paths
    const bool lean = !prm.blind && !prm.topk_global && prm.vec8 && !prm.work_stats && !prm.phase_cycles && prm.T > 1;
    auto go = [&](auto kern) -> int {
        DCI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
        kern<<<grid, nthreads, dyn, st>>>(prm);
        return 0;
    };
    if (smem && prm.qbatch > 1) {
        if (int rc = lean ? go(dci::traverse_kernel<ValT, PosT, true, true, true>) : go(dci::traverse_kernel<ValT, PosT, true, true>)) return rc;
    } else if (smem) {
        if (int rc = lean ? go(dci::traverse_kernel<ValT, PosT, true, false, true>) : go(dci::traverse_kernel<ValT, PosT, true, false>)) return rc;
    } else {
        if (int rc = lean ? go(dci::traverse_kernel<ValT, PosT, false, false, true>) : go(dci::traverse_kernel<ValT, PosT, false, false>)) return rc;
    }
    h->launches++;
    DCI_CUDA(cudaGetLastError());
    return 0;
}

int check_handle(dci_b200 *h) {
    if (!h) return fail(DCI_B200_ERR_ARG, "null handle");
    return 0;
}

}  // namespace

extern "C" {

const char *dci_b200_last_error(void) { return g_err; }

int dci_b200_abi_version(void) { return 1; }

int dci_b200_create(dci_b200_t **out, int dim, int num_comp_indices, int num_simp_indices,
                    int device, unsigned long long seed) {
    if (!out) return fail(DCI_B200_ERR_ARG, "out is null");
    *out = nullptr;
    if (dim <= 0) return fail(DCI_B200_ERR_ARG, "dim must be positive, got %d", dim);
    if (num_comp_indices <= 0 || num_simp_indices <= 0)
        return fail(DCI_B200_ERR_ARG, "num_comp_indices and num_simp_indices must be positive, got %d and %d",
                    num_comp_indices, num_simp_indices);
    if ((long long)num_comp_indices * num_simp_indices > dci::kMaxIndices || num_comp_indices > 64)
        return fail(DCI_B200_ERR_UNSUPPORTED, "at most %d simple indices in total and 64 composite indices are supported",
                    dci::kMaxIndices);
    int ndev = 0;
    DCI_CUDA(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return fail(DCI_B200_ERR_ARG, "device %d out of range (%d devices)", device, ndev);
    DeviceGuard g(device);
    if (!g.ok) return fail(DCI_B200_ERR_CUDA, "cannot select device %d", device);
    dci_b200 *h = new (std::nothrow) dci_b200();
    if (!h) return fail(DCI_B200_ERR_CUDA, "host allocation failed");
    h->dim = dim; h->L = num_comp_indices; h->S = num_simp_indices; h->device = device;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { delete h; return fail(DCI_B200_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e)); }
    h->sm_count = prop.multiProcessorCount;
    h->smem_optin = prop.sharedMemPerBlockOptin;
    h->smem_per_sm = prop.sharedMemPerMultiprocessor;
    // the word in which the TMA-fed exact projection reports a wait that ran out sits behind the directions
    const size_t proj_bytes = (sizeof(float) * (size_t)dim * h->L * h->S + 255) & ~(size_t)255;
    e = counted_malloc((void **)&h->d_proj, proj_bytes + 256);
    if (e != cudaSuccess) { delete h; return fail(DCI_B200_ERR_CUDA, "cudaMalloc(directions): %s", cudaGetErrorString(e)); }
    h->d_copyflag = (int *)((unsigned char *)h->d_proj + proj_bytes);
    e = cudaMemset(h->d_copyflag, 0, 256);
    if (e != cudaSuccess) { counted_free(h->d_proj); delete h; return fail(DCI_B200_ERR_CUDA, "cudaMemset: %s", cudaGetErrorString(e)); }
    int rc = launch_directions(h, seed, 0);
    if (rc == 0 && (e = cudaDeviceSynchronize()) != cudaSuccess)
        rc = fail(DCI_B200_ERR_CUDA, "direction generation: %s", cudaGetErrorString(e));
    if (rc) { counted_free(h->d_proj); delete h; return rc; }
    *out = h;
    return 0;
}

int dci_b200_destroy(dci_b200_t *h) {
    if (!h) return 0;
    DeviceGuard g(h->device);
    cudaDeviceSynchronize();
    Buf *bufs[] = {&h->keys, &h->ids, &h->pos, &h->keysT, &h->tmp_keys, &h->qproj, &h->part_topk, &h->scratch, &h->merge_scratch, &h->stats, &h->phases, &h->errflag, &h->qbound,
                   &h->hq, &h->hids, &h->hdists};
    for (Buf *b : bufs) b->release();
    if (h->d_proj) counted_free(h->d_proj);
    for (auto &e : h->ev) if (e) cudaEventDestroy(e);
    for (auto &e : h->pev) if (e) cudaEventDestroy(e);
    delete h;
    return 0;
}

int dci_b200_get_proj(dci_b200_t *h, float *h_out) {
    if (int rc = check_handle(h)) return rc;
    if (!h_out) return fail(DCI_B200_ERR_ARG, "h_out is null");
    DeviceGuard g(h->device);
    DCI_CUDA(cudaDeviceSynchronize());
    DCI_CUDA(cudaMemcpy(h_out, h->d_proj, sizeof(float) * (size_t)h->dim * h->L * h->S, cudaMemcpyDeviceToHost));
    return 0;
}

int dci_b200_set_proj(dci_b200_t *h, const float *h_in) {
    if (int rc = check_handle(h)) return rc;
    if (!h_in) return fail(DCI_B200_ERR_ARG, "h_in is null");
    if (h->num_points > 0) return fail(DCI_B200_ERR_STATE, "directions cannot change while the index holds points; clear first");
    DeviceGuard g(h->device);
    DCI_CUDA(cudaDeviceSynchronize());
    DCI_CUDA(cudaMemcpy(h->d_proj, h_in, sizeof(float) * (size_t)h->dim * h->L * h->S, cudaMemcpyHostToDevice));
    return 0;
}

// Limits shared by add and append: the encoded promotion (rank << tshift | lane) must fit 32 bits.
static int check_partition_limits(dci_b200 *h, int ppb, int thread_size) {
    int tshift = 0;
    while ((1 << tshift) < thread_size) ++tshift;
    const unsigned long long wcap = (unsigned long long)h->S * ((ppb + thread_size - 1) / thread_size + 2);
    if ((wcap << tshift) >= 0xFFFFFFFFull ||
        !dci::FastDiv::exact_for((uint32_t)thread_size, (uint64_t)ppb + 2ull * thread_size))
        return fail(DCI_B200_ERR_UNSUPPORTED, "partition of %d points with %d simple indices and thread_size %d is too large",
                    ppb, h->S, thread_size);
    return 0;
}

// Positions within a partition are kept in 16 bits while a position plus the offset of the window grid
// (below thread_size) still fits; the traversal relies on this bound.
static inline bool pos16(int ppb, int thread_size) { return (long long)ppb + thread_size <= 65536; }

// bytes of the position array: every (partition, simple index) segment padded to pos_stride(ppb)
static size_t pos_bytes(int I, int num_parts, int ppb, int thread_size) {
    return (size_t)I * num_parts * dci::pos_stride(ppb) * (pos16(ppb, thread_size) ? sizeof(uint16_t) : sizeof(uint32_t));
}

static int ensure_index_buffers(dci_b200 *h, size_t n_entries, int ppb, int num_parts, int thread_size) {
    DCI_CUDA(h->keys.ensure(n_entries * sizeof(float)));
    DCI_CUDA(h->ids.ensure(n_entries * sizeof(int)));
    DCI_CUDA(h->keysT.ensure(n_entries * sizeof(float)));
    DCI_CUDA(h->pos.ensure(pos_bytes(h->L * h->S, num_parts, ppb, thread_size)));
    return 0;
}

int dci_b200_add(dci_b200_t *h, const float *d_data, int num_points, int block_size, int thread_size, void *stream) {
    if (int rc = check_handle(h)) return rc;
    if (h->num_points > 0)
        return fail(DCI_B200_ERR_STATE, "the index already holds %d points; it does not support insertion of more than one array (clear first)", h->num_points);
    if (!d_data) return fail(DCI_B200_ERR_ARG, "d_data is null");
    if (num_points <= 0) return fail(DCI_B200_ERR_ARG, "num_points must be positive, got %d", num_points);
    if (block_size <= 0 || thread_size <= 0)
        return fail(DCI_B200_ERR_ARG, "block_size and thread_size must be positive, got %d and %d", block_size, thread_size);
    if (thread_size > 65536) return fail(DCI_B200_ERR_UNSUPPORTED, "thread_size above 65536 is not supported");
    DeviceGuard g(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int I = h->L * h->S;
    const int ppb = (num_points + block_size - 1) / block_size;
    const int num_parts = (num_points + ppb - 1) / ppb;
    if (int rc = check_partition_limits(h, ppb, thread_size)) return rc;
    const size_t n_entries = (size_t)I * num_points;
    if (int rc = ensure_index_buffers(h, n_entries, ppb, num_parts, thread_size)) return rc;
    DCI_CUDA(h->tmp_keys.ensure(n_entries * sizeof(float)));
    h->num_points = num_points; h->P = block_size; h->T = thread_size; h->ppb = ppb; h->num_parts = num_parts;
    h->d_data = d_data;
    int rc = launch_project(h, d_data, num_points, (float *)h->tmp_keys.p, st);
    if (!rc) rc = pos16(ppb, thread_size) ? launch_build<uint16_t>(h, (const float *)h->tmp_keys.p, st)
                                 : launch_build<uint32_t>(h, (const float *)h->tmp_keys.p, st);
    if (rc) { h->num_points = 0; h->d_data = nullptr; }
    return rc;
}

int dci_b200_append(dci_b200_t *h, const float *d_all_data, int num_points_total, void *stream) {
    if (int rc = check_handle(h)) return rc;
    if (h->num_points <= 0) return fail(DCI_B200_ERR_STATE, "append needs an index that already holds points (add first)");
    if (!d_all_data) return fail(DCI_B200_ERR_ARG, "d_all_data is null");
    if (num_points_total <= h->num_points)
        return fail(DCI_B200_ERR_ARG, "num_points_total (%d) must exceed the %d points already indexed", num_points_total,
                    h->num_points);
    DeviceGuard g(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int I = h->L * h->S, n_old = h->num_points, n_new = num_points_total, n_add = n_new - n_old;
    const int ppb = (n_new + h->P - 1) / h->P;
    const int num_parts = (n_new + ppb - 1) / ppb;
    if (int rc = check_partition_limits(h, ppb, h->T)) return rc;
    // 1. the old rows' keys, back in id order, at the new row stride
    DCI_CUDA(h->tmp_keys.ensure((size_t)I * n_new * sizeof(float)));
    {
        const unsigned grid = (unsigned)std::min<long long>((long long)I * h->num_parts, (long long)h->sm_count * 8);
        dci::unsort_keys_kernel<<<grid, 256, 0, st>>>((const float *)h->keys.p, (const int *)h->ids.p, n_old, I, h->ppb,
                                                      h->num_parts, (float *)h->tmp_keys.p, n_new);
        h->launches++;
        DCI_CUDA(cudaGetLastError());
    }
    // 2. keys of the new rows only (staged in the stride-T buffer, which step 3 rewrites anyway).
    // From here on the old index is gone (its stride-T keys are overwritten), so every failure
    // leaves the handle empty rather than claiming an index it no longer has.
    auto invalidate = [h](int rc) { h->num_points = 0; h->d_data = nullptr; return rc; };
#define DCI_CUDA_OR_EMPTY(call)                                                                     \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess)                                                                      \
            return invalidate(fail(DCI_B200_ERR_CUDA, "%s failed at %s:%d: %s", #call, __FILE__,    \
                                   __LINE__, cudaGetErrorString(e_)));                              \
    } while (0)
    DCI_CUDA_OR_EMPTY(cudaStreamSynchronize(st));       // growing a buffer frees it: nothing may still read it
    DCI_CUDA_OR_EMPTY(h->keysT.ensure((size_t)I * n_new * sizeof(float)));
    if (int rc = launch_project(h, d_all_data + (size_t)n_old * h->dim, n_add, (float *)h->keysT.p, st)) return invalidate(rc);
    DCI_CUDA_OR_EMPTY(cudaMemcpy2DAsync((float *)h->tmp_keys.p + n_old, (size_t)n_new * sizeof(float), h->keysT.p,
                                        (size_t)n_add * sizeof(float), (size_t)n_add * sizeof(float), (size_t)I,
                                        cudaMemcpyDeviceToDevice, st));
    DCI_CUDA_OR_EMPTY(cudaStreamSynchronize(st));
#undef DCI_CUDA_OR_EMPTY
    // 3. every segment again, for the partition bounds of the new point count
    if (int rc = ensure_index_buffers(h, (size_t)I * n_new, ppb, num_parts, h->T)) { h->num_points = 0; h->d_data = nullptr; return rc; }
    h->num_points = n_new; h->ppb = ppb; h->num_parts = num_parts; h->d_data = d_all_data;
    int rc = pos16(ppb, h->T) ? launch_build<uint16_t>(h, (const float *)h->tmp_keys.p, st)
                            : launch_build<uint32_t>(h, (const float *)h->tmp_keys.p, st);
    if (rc) { h->num_points = 0; h->d_data = nullptr; }
    return rc;
}

int dci_b200_set_index(dci_b200_t *h, const float *d_data, int num_points, int block_size, int thread_size,
                       const float *h_keys, const int *h_ids, void *stream) {
    if (int rc = check_handle(h)) return rc;
    if (h->num_points > 0)
        return fail(DCI_B200_ERR_STATE, "the index already holds %d points (clear first)", h->num_points);
    if (!d_data || !h_keys || !h_ids) return fail(DCI_B200_ERR_ARG, "null pointer passed to set_index");
    if (num_points <= 0 || block_size <= 0 || thread_size <= 0 || thread_size > 65536)
        return fail(DCI_B200_ERR_ARG, "num_points, block_size and thread_size must be positive");
    DeviceGuard g(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int I = h->L * h->S;
    const int ppb = (num_points + block_size - 1) / block_size;
    const int num_parts = (num_points + ppb - 1) / ppb;
    {
        int tshift = 0;
        while ((1 << tshift) < thread_size) ++tshift;
        const unsigned long long wcap = (unsigned long long)h->S * ((ppb + thread_size - 1) / thread_size + 2);
        if ((wcap << tshift) >= 0xFFFFFFFFull ||
            !dci::FastDiv::exact_for((uint32_t)thread_size, (uint64_t)ppb + 2ull * thread_size))
            return fail(DCI_B200_ERR_UNSUPPORTED, "partition of %d points is too large for thread_size %d", ppb, thread_size);
    }
    const size_t n_entries = (size_t)I * num_points;
    DCI_CUDA(h->keys.ensure(n_entries * sizeof(float)));
    DCI_CUDA(h->ids.ensure(n_entries * sizeof(int)));
    DCI_CUDA(h->keysT.ensure(n_entries * sizeof(float)));
    DCI_CUDA(h->pos.ensure(pos_bytes(I, num_parts, ppb, thread_size)));
    DCI_CUDA(h->errflag.ensure(sizeof(int)));
    DCI_CUDA(cudaMemsetAsync(h->errflag.p, 0, sizeof(int), st));
    // the caller's arrays are [I][N]; the kernel checks them and writes the partition-major index
    DCI_CUDA(h->tmp_keys.ensure(n_entries * sizeof(float)));
    DCI_CUDA(h->scratch.ensure(n_entries * sizeof(int)));
    DCI_CUDA(cudaMemcpyAsync(h->tmp_keys.p, h_keys, n_entries * sizeof(float), cudaMemcpyHostToDevice, st));
    DCI_CUDA(cudaMemcpyAsync(h->scratch.p, h_ids, n_entries * sizeof(int), cudaMemcpyHostToDevice, st));
    const unsigned grid = (unsigned)std::min<long long>((long long)I * num_parts, (long long)h->sm_count * 8);
    // positions start as a sentinel (all ones, beyond any partition) so that the second kernel sees
    // every point that no entry of its segment names
    DCI_CUDA(cudaMemsetAsync(h->pos.p, 0xFF, pos_bytes(I, num_parts, ppb, thread_size), st));
    if (pos16(ppb, thread_size)) {
        dci::derive_index_kernel<uint16_t><<<grid, 256, 0, st>>>(
            (const float *)h->tmp_keys.p, (const int *)h->scratch.p, num_points, I, ppb, num_parts, thread_size,
            (float *)h->keys.p, (int *)h->ids.p, (uint16_t *)h->pos.p, (float *)h->keysT.p, (int *)h->errflag.p);
        dci::check_index_kernel<uint16_t><<<grid, 256, 0, st>>>((const int *)h->ids.p, (uint16_t *)h->pos.p,
                                                               num_points, I, ppb, num_parts, (int *)h->errflag.p);
    } else {
        dci::derive_index_kernel<uint32_t><<<grid, 256, 0, st>>>(
            (const float *)h->tmp_keys.p, (const int *)h->scratch.p, num_points, I, ppb, num_parts, thread_size,
            (float *)h->keys.p, (int *)h->ids.p, (uint32_t *)h->pos.p, (float *)h->keysT.p, (int *)h->errflag.p);
        dci::check_index_kernel<uint32_t><<<grid, 256, 0, st>>>((const int *)h->ids.p, (uint32_t *)h->pos.p,
                                                               num_points, I, ppb, num_parts, (int *)h->errflag.p);
    }
    h->launches += 2;
    DCI_CUDA(cudaGetLastError());
    int flag = 0;
    DCI_CUDA(cudaMemcpyAsync(&flag, h->errflag.p, sizeof(int), cudaMemcpyDeviceToHost, st));
    DCI_CUDA(cudaStreamSynchronize(st));
    if (flag) return fail(DCI_B200_ERR_ARG, "the index is not valid: a segment is not ascending, holds an id outside its partition, or names a point twice");
    h->num_points = num_points; h->P = block_size; h->T = thread_size; h->ppb = ppb; h->num_parts = num_parts;
    h->d_data = d_data;
    return 0;
}

// out_width: entries per query in the outputs (num_neighbours, or the candidate list length of a blind query)
// d_packed: when not null the merged keys (distance bits << 32 | id) go there and d_ids / d_dists are unused
static int query_impl(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                      int num_outer_iterations, int max_num_candidates, int blind, int out_width, int block_size,
                      int thread_size, int *d_ids, float *d_dists, void *stream,
                      unsigned long long *d_packed = nullptr) {
    if (int rc = check_handle(h)) return rc;
    if (h->num_points <= 0) return fail(DCI_B200_ERR_STATE, "the index is empty; add data first");
    if (num_queries < 0) return fail(DCI_B200_ERR_ARG, "num_queries must not be negative");
    if (num_queries == 0) return 0;
    if (!d_query || (!d_packed && (!d_ids || (!d_dists && !blind)))) return fail(DCI_B200_ERR_ARG, "null query or output pointer");
    if (num_neighbours <= 0) return fail(DCI_B200_ERR_ARG, "num_neighbours must be positive, got %d", num_neighbours);
    if (num_neighbours > h->num_points)
        return fail(DCI_B200_ERR_ARG, "num_neighbours (%d) exceeds the number of indexed points (%d)", num_neighbours, h->num_points);
    if (block_size != h->P || thread_size != h->T)
        return fail(DCI_B200_ERR_ARG, "block_size/thread_size (%d, %d) differ from the values the index was built with (%d, %d)",
                    block_size, thread_size, h->P, h->T);
    DeviceGuard g(h->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int I = h->L * h->S;
    DCI_CUDA(h->qproj.ensure(sizeof(float) * (size_t)I * num_queries));
    const bool timing = h->timing_on != 0;
    if (timing) {
        for (auto &e : h->ev) if (!e) DCI_CUDA(cudaEventCreate(&e));
        h->t_project = h->t_traverse = h->t_merge = 0.f;
        h->t_traverse_launches = 0;
        DCI_CUDA(cudaEventRecord(h->ev[0], st));
    }
    if (int rc = launch_project(h, d_query, num_queries, (float *)h->qproj.p, st)) return rc;
    if (timing) DCI_CUDA(cudaEventRecord(h->ev[1], st));

    dci::TraverseParams prm;
    memset(&prm, 0, sizeof(prm));
    prm.skeys = (const float *)h->keys.p; prm.skeysT = (const float *)h->keysT.p; prm.sids = (const int *)h->ids.p;
    prm.spos = h->pos.p; prm.data = h->d_data;
    prm.qproj = (const float *)h->qproj.p; prm.query = d_query;
    prm.N = h->num_points; prm.dim = h->dim; prm.L = h->L; prm.S = h->S; prm.P = h->P; prm.T = h->T;
    prm.ppb = h->ppb; prm.num_parts = h->num_parts; prm.nq_total = num_queries;
    prm.knn = num_neighbours; prm.max_cand = max_num_candidates;
    prm.outer_s = (long long)num_outer_iterations * h->S;
    prm.wcap = h->S * ((h->ppb + h->T - 1) / h->T + 2);
    prm.tshift = 0;
    while ((1 << prm.tshift) < h->T) ++prm.tshift;
    prm.divT = dci::FastDiv::make((uint32_t)h->T);
    prm.vec4 = (h->dim % 4 == 0) && (((uintptr_t)h->d_data & 15) == 0) && (((uintptr_t)d_query & 15) == 0);
    prm.vec8 = (h->dim % 8 == 0) && (((uintptr_t)h->d_data & 31) == 0);
    const int nthreads = prm.wcap >= 4096 ? 1024 : (prm.wcap >= 1024 ? 512 : (prm.wcap >= 256 ? 256 : 64));
    prm.blind = blind ? 1 : 0;
    prm.kpart = std::min(out_width, h->ppb);
    prm.topk_cap = next_pow2(prm.kpart + nthreads);
    // larger selection buffers do not fit shared memory; a blind query reads the promotion records
    // while it selects, and the shared buffers would overlay them
    prm.topk_global = (prm.topk_cap > 2048 || blind) ? 1 : 0;
    const int merge_threads = 256;
    const int merge_cap = next_pow2(out_width + merge_threads);
    const bool merge_global = merge_cap > 2048;

    if (h->stats_on & 2) {
        DCI_CUDA(h->phases.ensure(sizeof(long long) * 16));
        DCI_CUDA(cudaMemsetAsync(h->phases.p, 0, sizeof(long long) * 16, st));
        prm.phase_cycles = (long long *)h->phases.p;
        h->phases_valid = 1;
    }
    if (h->stats_on & 1) {
        const size_t bytes = sizeof(long long) * 6 * (size_t)num_queries * h->P;
        DCI_CUDA(h->stats.ensure(bytes));
        DCI_CUDA(cudaMemsetAsync(h->stats.p, 0, bytes, st));
        prm.work_stats = (long long *)h->stats.p;
        h->stats_nq = num_queries;
    }
    const size_t per_query = sizeof(uint64_t) * (size_t)h->num_parts * prm.kpart;
    const int batch = (int)std::max<size_t>(1, std::min<size_t>((size_t)num_queries, ((size_t)1 << 30) / per_query));
    DCI_CUDA(h->part_topk.ensure(per_query * batch));
    prm.part_topk = (uint64_t *)h->part_topk.p;
    const int merge_grid_cap = merge_global ? 2 * h->sm_count : (1 << 30);
    if (merge_global) DCI_CUDA(h->merge_scratch.ensure((size_t)merge_grid_cap * 2 * merge_cap * sizeof(uint64_t)));
    if (h->distance_bound && !blind) DCI_CUDA(h->qbound.ensure(sizeof(uint32_t) * (size_t)batch));
    for (int q0 = 0; q0 < num_queries; q0 += batch) {
        prm.q0 = q0;
        prm.nq = std::min(batch, num_queries - q0);
        if (h->distance_bound && !blind) {
            prm.qbound = (uint32_t *)h->qbound.p;
            DCI_CUDA(cudaMemsetAsync(prm.qbound, 0x7F, sizeof(uint32_t) * (size_t)prm.nq, st));   // 0x7F7F7F7F: a huge finite float
        }
        if (timing) DCI_CUDA(cudaEventRecord(h->ev[2], st));
        int rc;
        // partitions of at most 32 points with at most 32 windows per composite index: one warp per
        // (query, partition) pair instead of one CTA (per-phase cycle counters exist only in the CTA
        // kernel, and the warp kernel keeps statistics for at most two composite indices)
        const bool small = h->ppb <= 32 && prm.wcap <= 32 && h->S <= 32 && pos16(h->ppb, h->T) && !blind && !prm.topk_global &&
                           !(h->stats_on & 2) && (!(h->stats_on & 1) || h->L <= 2);
        if (small) {
            const long long nwork = (long long)prm.nq * prm.num_parts;
            unsigned grid = (unsigned)std::min<long long>((nwork + dci::kSmallWarps - 1) / dci::kSmallWarps,
                                                          (long long)h->sm_count * 8);
            if (h->max_ctas > 0) grid = std::min(grid, (unsigned)h->max_ctas);
            dci::traverse_small_kernel<<<grid, dci::kSmallWarps * 32, 0, st>>>(prm);
            h->launches++;
            h->last_qbatch = 1;
            DCI_CUDA(cudaGetLastError());
            rc = 0;
        } else if (pos16(prm.ppb, h->T))
            rc = (prm.wcap <= 65535) ? launch_traverse<uint16_t, uint16_t>(h, prm, nthreads, st)
                                     : launch_traverse<uint32_t, uint16_t>(h, prm, nthreads, st);
        else
            rc = launch_traverse<uint32_t, uint32_t>(h, prm, nthreads, st);
        if (rc) return rc;
        if (timing) DCI_CUDA(cudaEventRecord(h->ev[3], st));
        dci::merge_partitions_kernel<<<std::min(prm.nq, merge_grid_cap), merge_threads,
                                       merge_global ? 0 : (size_t)merge_cap * 16, st>>>(
            prm.part_topk, h->num_parts, prm.kpart, out_width, merge_cap, q0, prm.nq,
            merge_global ? (uint64_t *)h->merge_scratch.p : nullptr, d_ids, d_dists, prm.blind,
            reinterpret_cast<uint64_t *>(d_packed));
        h->launches++;
        DCI_CUDA(cudaGetLastError());
        if (timing) {   // timing mode synchronises after every batch; it is off by default
            float ms = 0.f;
            DCI_CUDA(cudaEventRecord(h->ev[4], st));
            DCI_CUDA(cudaEventSynchronize(h->ev[4]));
            if (q0 == 0) { DCI_CUDA(cudaEventElapsedTime(&ms, h->ev[0], h->ev[1])); h->t_project = ms; }
            DCI_CUDA(cudaEventElapsedTime(&ms, h->ev[2], h->ev[3])); h->t_traverse += ms;
            DCI_CUDA(cudaEventElapsedTime(&ms, h->ev[3], h->ev[4])); h->t_merge += ms;
            h->t_traverse_launches++;
        }
    }
    return 0;
}

int dci_b200_query(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                   int num_outer_iterations, int max_num_candidates, int blind, int block_size,
                   int thread_size, int *d_ids, float *d_dists, void *stream) {
    if (blind)
        return fail(DCI_B200_ERR_UNSUPPORTED, "blind querying returns lists of another length: use dci_b200_query_blind");
    return query_impl(h, d_query, num_queries, num_neighbours, num_outer_iterations, max_num_candidates, 0,
                      num_neighbours, block_size, thread_size, d_ids, d_dists, stream);
}

int dci_b200_query_packed(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                          int num_outer_iterations, int max_num_candidates, int block_size, int thread_size,
                          unsigned long long *d_packed, void *stream) {
    if (!d_packed) return fail(DCI_B200_ERR_ARG, "null output pointer");
    return query_impl(h, d_query, num_queries, num_neighbours, num_outer_iterations, max_num_candidates, 0,
                      num_neighbours, block_size, thread_size, nullptr, nullptr, stream, d_packed);
}

int dci_b200_blind_width(int num_outer_iterations, int max_num_candidates) {
    return std::max(0, std::min(num_outer_iterations, max_num_candidates));
}

int dci_b200_query_blind(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                         int num_outer_iterations, int max_num_candidates, int block_size, int thread_size,
                         int *d_ids, int *d_iterations, void *stream) {
    const int width = dci_b200_blind_width(num_outer_iterations, max_num_candidates);
    if (width <= 0) return fail(DCI_B200_ERR_ARG, "num_outer_iterations and max_num_candidates must be positive");
    return query_impl(h, d_query, num_queries, num_neighbours, num_outer_iterations, max_num_candidates, 1, width,
                      block_size, thread_size, d_ids, reinterpret_cast<float *>(d_iterations), stream);
}

int dci_b200_query_host(dci_b200_t *h, const float *h_query, int num_queries, int num_neighbours,
                        int num_outer_iterations, int max_num_candidates, int blind, int block_size,
                        int thread_size, int *h_ids, float *h_dists) {
    if (int rc = check_handle(h)) return rc;
    if (num_queries < 0) return fail(DCI_B200_ERR_ARG, "num_queries must not be negative");
    if (num_queries == 0) return 0;
    if (!h_query || !h_ids || !h_dists) return fail(DCI_B200_ERR_ARG, "null query or output pointer");
    if (num_neighbours <= 0) return fail(DCI_B200_ERR_ARG, "num_neighbours must be positive, got %d", num_neighbours);
    DeviceGuard g(h->device);
    const size_t qbytes = sizeof(float) * (size_t)num_queries * h->dim;
    const size_t obytes = sizeof(int) * (size_t)num_queries * num_neighbours;
    DCI_CUDA(h->hq.ensure(qbytes));
    DCI_CUDA(h->hids.ensure(obytes));
    DCI_CUDA(h->hdists.ensure(obytes));
    DCI_CUDA(cudaMemcpyAsync(h->hq.p, h_query, qbytes, cudaMemcpyHostToDevice, 0));
    int rc = dci_b200_query(h, (const float *)h->hq.p, num_queries, num_neighbours, num_outer_iterations,
                            max_num_candidates, blind, block_size, thread_size, (int *)h->hids.p,
                            (float *)h->hdists.p, nullptr);
    if (rc) return rc;
    DCI_CUDA(cudaMemcpyAsync(h_ids, h->hids.p, obytes, cudaMemcpyDeviceToHost, 0));
    DCI_CUDA(cudaMemcpyAsync(h_dists, h->hdists.p, obytes, cudaMemcpyDeviceToHost, 0));
    int copy_flag = 0;
    DCI_CUDA(cudaMemcpyAsync(&copy_flag, h->d_copyflag, sizeof(int), cudaMemcpyDeviceToHost, 0));
    DCI_CUDA(cudaStreamSynchronize(0));
    if (copy_flag) {      // reported once; the projection that set it (data or queries) has to be repeated
        cudaMemsetAsync(h->d_copyflag, 0, sizeof(int), 0);
        return fail(DCI_B200_ERR_CUDA, "exact projection: a wait on a TMA copy ran out; keys may be incomplete");
    }
    return 0;
}

int dci_b200_clear(dci_b200_t *h) {
    if (int rc = check_handle(h)) return rc;
    DeviceGuard g(h->device);
    DCI_CUDA(cudaDeviceSynchronize());
    // the index buffers are kept for the next add (add / query / clear cycles are the
    // reference's typical use, example.py:75-82); destroy returns them
    h->num_points = 0; h->d_data = nullptr; h->P = h->T = h->ppb = h->num_parts = 0;
    return 0;
}

int dci_b200_reset(dci_b200_t *h, unsigned long long seed) {
    if (int rc = dci_b200_clear(h)) return rc;
    DeviceGuard g(h->device);
    if (int rc = launch_directions(h, seed, 0)) return rc;
    DCI_CUDA(cudaDeviceSynchronize());
    return 0;
}

int dci_b200_num_points(dci_b200_t *h) { return h ? h->num_points : 0; }

int dci_b200_get_index(dci_b200_t *h, float *h_keys, int *h_ids) {
    if (int rc = check_handle(h)) return rc;
    if (!h_keys || !h_ids) return fail(DCI_B200_ERR_ARG, "null output pointer");
    if (h->num_points <= 0) return fail(DCI_B200_ERR_STATE, "the index is empty");
    DeviceGuard g(h->device);
    DCI_CUDA(cudaDeviceSynchronize());
    // the index is partition-major on the device; callers see [I][N]
    const int I = h->L * h->S;
    const size_t n = (size_t)I * h->num_points;
    DCI_CUDA(h->tmp_keys.ensure(n * sizeof(float)));
    DCI_CUDA(h->scratch.ensure(n * sizeof(int)));
    const unsigned grid = (unsigned)std::min<long long>((long long)I * h->num_parts, (long long)h->sm_count * 8);
    dci::export_index_kernel<<<grid, 256>>>((const float *)h->keys.p, (const int *)h->ids.p, h->num_points, I, h->ppb,
                                            h->num_parts, (float *)h->tmp_keys.p, (int *)h->scratch.p);
    h->launches++;
    DCI_CUDA(cudaGetLastError());
    DCI_CUDA(cudaMemcpy(h_keys, h->tmp_keys.p, n * sizeof(float), cudaMemcpyDeviceToHost));
    DCI_CUDA(cudaMemcpy(h_ids, h->scratch.p, n * sizeof(int), cudaMemcpyDeviceToHost));
    return 0;
}

int dci_b200_project(dci_b200_t *h, const float *d_x, int n, float *d_out, void *stream) {
    if (int rc = check_handle(h)) return rc;
    if (!d_x || !d_out || n < 0) return fail(DCI_B200_ERR_ARG, "bad argument to project");
    DeviceGuard g(h->device);
    return launch_project(h, d_x, n, d_out, (cudaStream_t)stream);
}

int dci_b200_enable_work_stats(dci_b200_t *h, int on) {
    if (int rc = check_handle(h)) return rc;
    h->stats_on = on & 3;
    if (!(on & 1)) h->stats_nq = 0;
    if (!(on & 2)) h->phases_valid = 0;
    return 0;
}

int dci_b200_get_work_stats(dci_b200_t *h, long long *h_out, long long capacity_records) {
    if (int rc = check_handle(h)) return rc;
    if (!h_out) return fail(DCI_B200_ERR_ARG, "h_out is null");
    const long long records = (long long)h->stats_nq * h->P;
    if (records <= 0) return fail(DCI_B200_ERR_STATE, "no work statistics recorded; enable them before the query");
    if (capacity_records < records) return fail(DCI_B200_ERR_ARG, "capacity %lld below the %lld records available", capacity_records, records);
    DeviceGuard g(h->device);
    DCI_CUDA(cudaDeviceSynchronize());
    DCI_CUDA(cudaMemcpy(h_out, h->stats.p, sizeof(long long) * 6 * (size_t)records, cudaMemcpyDeviceToHost));
    return 0;
}

int dci_b200_get_phase_cycles(dci_b200_t *h, long long *h_out) {
    if (int rc = check_handle(h)) return rc;
    if (!h_out) return fail(DCI_B200_ERR_ARG, "h_out is null");
    if (!h->phases.p || !h->phases_valid) return fail(DCI_B200_ERR_STATE, "no work statistics recorded; enable them before the query");
    DeviceGuard g(h->device);
    DCI_CUDA(cudaDeviceSynchronize());
    DCI_CUDA(cudaMemcpy(h_out, h->phases.p, sizeof(long long) * 16, cudaMemcpyDeviceToHost));
    h_out[11] = h->last_qbatch;
    h_out[13] = h->last_projection_tma;
    return 0;
}

long long dci_b200_launch_count(dci_b200_t *h) { return h ? h->launches : 0; }

long long dci_b200_device_alloc_calls(void) { return g_alloc_calls.load(); }

int dci_b200_set_max_ctas(dci_b200_t *h, int max_ctas) {
    if (int rc = check_handle(h)) return rc;
    if (max_ctas < 0) return fail(DCI_B200_ERR_ARG, "max_ctas must not be negative");
    h->max_ctas = max_ctas;
    return 0;
}

int dci_b200_set_projection(dci_b200_t *h, int mode) {
    if (int rc = check_handle(h)) return rc;
    if (mode < 0 || mode > 4)
        return fail(DCI_B200_ERR_ARG, "projection mode must be 0 (exact), 1 (tensor cores, persistent TMA pipeline), "
                                      "2 (tensor cores, plain loads), 3 (tensor cores, one TMA-fed tile per CTA) or "
                                      "4 (exact, rows staged by the computing threads only)");
    if (h->num_points > 0) return fail(DCI_B200_ERR_STATE, "the projection mode cannot change while the index holds points; clear first");
    h->projection_mode = mode == 4 ? 0 : mode;      // modes 0 and 4 give the same keys, bit for bit
    h->exact_tma = mode == 4 ? 0 : 1;
    return 0;
}

int dci_b200_enable_timing(dci_b200_t *h, int on) {
    if (int rc = check_handle(h)) return rc;
    h->timing_on = on ? 1 : 0;
    return 0;
}

int dci_b200_get_timing(dci_b200_t *h, float *h_ms) {
    if (int rc = check_handle(h)) return rc;
    if (!h_ms) return fail(DCI_B200_ERR_ARG, "h_ms is null");
    h_ms[0] = h->t_project; h_ms[1] = h->t_traverse; h_ms[2] = h->t_merge;
    h_ms[3] = (float)h->t_traverse_launches;
    return 0;
}

int dci_b200_last_projection_ms(dci_b200_t *h, float *h_ms) {
    if (int rc = check_handle(h)) return rc;
    if (!h_ms) return fail(DCI_B200_ERR_ARG, "h_ms is null");
    if (!h->pev_valid) return fail(DCI_B200_ERR_STATE, "no projection has run in timing mode yet");
    DeviceGuard g(h->device);
    DCI_CUDA(cudaEventSynchronize(h->pev[1]));
    DCI_CUDA(cudaEventElapsedTime(h_ms, h->pev[0], h->pev[1]));
    return 0;
}

int dci_b200_merge_shards(const int *d_ids_in, const float *d_dists_in, int num_shards, int num_queries,
                          int k, const long long *id_offsets, long long *d_ids_out, float *d_dists_out,
                          int device, void *stream) {
    if (!d_ids_in || !d_dists_in || !id_offsets || !d_ids_out || !d_dists_out)
        return fail(DCI_B200_ERR_ARG, "null pointer passed to merge_shards");
    if (num_shards <= 0 || num_shards > 64 || num_queries < 0 || k <= 0)
        return fail(DCI_B200_ERR_ARG, "merge_shards needs 1..64 shards, num_queries >= 0 and k > 0");
    if (num_queries == 0) return 0;
    for (int s = 0; s < num_shards; ++s)
        if (id_offsets[s] < 0 || id_offsets[s] > 0x7FFFFFFFll)
            return fail(DCI_B200_ERR_UNSUPPORTED, "id offsets must lie in [0, 2^31)");
    DeviceGuard g(device);
    if (!g.ok) return fail(DCI_B200_ERR_CUDA, "cannot select device %d", device);
    cudaStream_t st = (cudaStream_t)stream;
    dci::ShardOffsets off;
    memset(&off, 0, sizeof(off));
    for (int s = 0; s < num_shards; ++s) off.v[s] = id_offsets[s];
    const int threads = 256, cap = next_pow2(k + threads);
    if (k > dci::kMaxTopK)      // lists too long for the selection buffers: merge by rank (sorted input)
        dci::merge_shards_sorted_kernel<<<num_queries, threads, 0, st>>>(d_ids_in, d_dists_in, num_shards, num_queries, k,
                                                                        off, d_ids_out, d_dists_out);
    else
        dci::merge_shards_kernel<<<num_queries, threads, (size_t)cap * 16, st>>>(
            d_ids_in, d_dists_in, num_shards, num_queries, k, cap, off, d_ids_out, d_dists_out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DCI_B200_ERR_CUDA, "merge_shards launch: %s", cudaGetErrorString(e));
    return 0;
}

int dci_b200_merge_shards_packed(const unsigned long long *d_packed_in, int num_shards, int num_queries, int k,
                                 const long long *id_offsets, long long *d_ids_out, float *d_dists_out,
                                 int device, void *stream) {
    if (!d_packed_in || !id_offsets || !d_ids_out || !d_dists_out)
        return fail(DCI_B200_ERR_ARG, "null pointer passed to merge_shards_packed");
    if (num_shards <= 0 || num_shards > 64 || num_queries < 0 || k <= 0)
        return fail(DCI_B200_ERR_ARG, "merge_shards_packed needs 1..64 shards, num_queries >= 0 and k > 0");
    if (k > dci::kMaxTopK)
        return fail(DCI_B200_ERR_UNSUPPORTED, "merge_shards_packed serves k up to %d; use dci_b200_merge_shards above that", dci::kMaxTopK);
    if (num_queries == 0) return 0;
    for (int s = 0; s < num_shards; ++s)
        if (id_offsets[s] < 0 || id_offsets[s] > 0x7FFFFFFFll)
            return fail(DCI_B200_ERR_UNSUPPORTED, "id offsets must lie in [0, 2^31)");
    DeviceGuard g(device);
    if (!g.ok) return fail(DCI_B200_ERR_CUDA, "cannot select device %d", device);
    dci::ShardOffsets off;
    memset(&off, 0, sizeof(off));
    for (int s = 0; s < num_shards; ++s) off.v[s] = id_offsets[s];
    const int threads = 256, cap = next_pow2(k + threads);
    dci::merge_shards_packed_kernel<<<num_queries, threads, (size_t)cap * 16, (cudaStream_t)stream>>>(
        reinterpret_cast<const uint64_t *>(d_packed_in), num_shards, num_queries, k, cap, off, d_ids_out, d_dists_out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DCI_B200_ERR_CUDA, "merge_shards_packed launch: %s", cudaGetErrorString(e));
    return 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// MDCI below Python: the reference shards one point set over several devices and runs the
// per-device queries from host threads (dciknn_cuda/core.py:110-157, src/dci_cuda.cpp:120-134).
// Here one host thread drives every device: all calls of this library are asynchronous, so the D
// shards are projected, sorted and queried side by side on their own streams; the queries reach the
// other devices and the packed lists come back to devices[0] as peer copies over NVLink, ordered
// with events, and devices[0] merges.
struct dci_b200_mdci {
    int D = 0, dim = 0, P = 0, T = 0;
    long long num_points = 0, dpd = 0;
    int dev[64];
    dci_b200 *shard[64];
    cudaStream_t st[64];
    cudaEvent_t ev[64];
    cudaEvent_t ev_query = nullptr;
    Buf data[64], query[64], lists[64], tmp[64];   // per device: owned shard rows, query copy, packed lists, short lists
    Buf gathered, q0, ids0, dists0;                 // on dev[0]
};

namespace {

int mdci_check(dci_b200_mdci *m) {
    if (!m) return fail(DCI_B200_ERR_ARG, "null MDCI handle");
    return 0;
}

}  // namespace

extern "C" {

int dci_b200_mdci_create(dci_b200_mdci_t **out, int dim, int num_comp_indices, int num_simp_indices,
                         const int *devices, int num_devices, const unsigned long long *seeds) {
    if (!out) return fail(DCI_B200_ERR_ARG, "out is null");
    *out = nullptr;
    if (!devices || num_devices < 1 || num_devices > 64)
        return fail(DCI_B200_ERR_ARG, "MDCI needs 1 to 64 devices, got %d", num_devices);
    dci_b200_mdci *m = new (std::nothrow) dci_b200_mdci();
    if (!m) return fail(DCI_B200_ERR_CUDA, "host allocation failed");
    m->dim = dim;
    for (int i = 0; i < 64; ++i) { m->shard[i] = nullptr; m->st[i] = nullptr; m->ev[i] = nullptr; m->dev[i] = 0; }
    int rc = 0;
    for (int i = 0; i < num_devices && !rc; ++i) {
        m->dev[i] = devices[i];
        // every shard has its own directions, as in the reference (one _dci_new per device, core.py:117)
        rc = dci_b200_create(&m->shard[i], dim, num_comp_indices, num_simp_indices, devices[i],
                             seeds ? seeds[i] : 0x9E3779B97F4A7C15ull * (unsigned long long)(i + 1));
        if (rc) break;
        m->D = i + 1;
        DeviceGuard g(devices[i]);
        if (cudaStreamCreateWithFlags(&m->st[i], cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&m->ev[i], cudaEventDisableTiming) != cudaSuccess)
            rc = fail(DCI_B200_ERR_CUDA, "cannot create a stream or an event on device %d", devices[i]);
        for (int j = 0; j < i && !rc; ++j) {          // direct copies between the devices where the box allows them
            if (devices[j] == devices[i]) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, devices[i], devices[j]) == cudaSuccess && can) {
                cudaDeviceEnablePeerAccess(devices[j], 0);
                DeviceGuard g2(devices[j]);
                cudaDeviceEnablePeerAccess(devices[i], 0);
            }
            cudaGetLastError();                        // "already enabled" is not an error here
        }
    }
    if (!rc) {
        DeviceGuard g(m->dev[0]);
        if (cudaEventCreateWithFlags(&m->ev_query, cudaEventDisableTiming) != cudaSuccess)
            rc = fail(DCI_B200_ERR_CUDA, "cannot create an event on device %d", m->dev[0]);
    }
    if (rc) {
        char keep[sizeof(g_err)];
        memcpy(keep, g_err, sizeof(keep));
        dci_b200_mdci_destroy(m);
        memcpy(g_err, keep, sizeof(keep));
        return rc;
    }
    *out = m;
    return 0;
}

int dci_b200_mdci_destroy(dci_b200_mdci_t *m) {
    if (!m) return 0;
    for (int i = 0; i < 64; ++i) {
        if (!m->shard[i] && !m->st[i] && !m->ev[i]) continue;
        DeviceGuard g(m->dev[i]);
        if (m->st[i]) { cudaStreamSynchronize(m->st[i]); cudaStreamDestroy(m->st[i]); }
        if (m->ev[i]) cudaEventDestroy(m->ev[i]);
        if (m->shard[i]) dci_b200_destroy(m->shard[i]);
        m->data[i].release(); m->query[i].release(); m->lists[i].release(); m->tmp[i].release();
    }
    {
        DeviceGuard g(m->dev[0]);
        if (m->ev_query) cudaEventDestroy(m->ev_query);
        m->gathered.release(); m->q0.release(); m->ids0.release(); m->dists0.release();
    }
    delete m;
    return 0;
}

int dci_b200_mdci_num_devices(dci_b200_mdci_t *m) { return m ? m->D : 0; }

dci_b200_t *dci_b200_mdci_shard(dci_b200_mdci_t *m, int i) { return (m && i >= 0 && i < m->D) ? m->shard[i] : nullptr; }

long long dci_b200_mdci_data_per_device(dci_b200_mdci_t *m) { return m ? m->dpd : 0; }

int dci_b200_mdci_add(dci_b200_mdci_t *m, const float *h_data, long long num_points, int block_size, int thread_size) {
    if (int rc = mdci_check(m)) return rc;
    if (m->num_points > 0)
        return fail(DCI_B200_ERR_STATE, "the index already holds %lld points; it does not support insertion of more than one array (clear first)", m->num_points);
    if (!h_data || num_points <= 0) return fail(DCI_B200_ERR_ARG, "null data or no points");
    const long long dpd = num_points / m->D + 1;                    // the reference's rule, core.py:122
    if (dpd > 0x7FFFFFFFll) return fail(DCI_B200_ERR_UNSUPPORTED, "a shard of %lld points is too large", dpd);
    for (int i = 0; i < m->D; ++i) {                                  // everything below is enqueued, device by device
        const long long lo = std::min(num_points, dpd * i), hi = std::min(num_points, dpd * (i + 1));
        if (hi <= lo) continue;                                       // a trailing shard without rows stays empty
        DeviceGuard g(m->dev[i]);
        const size_t bytes = sizeof(float) * (size_t)(hi - lo) * m->dim;
        DCI_CUDA(m->data[i].ensure(bytes));
        DCI_CUDA(cudaMemcpyAsync(m->data[i].p, h_data + (size_t)lo * m->dim, bytes, cudaMemcpyHostToDevice, m->st[i]));
        if (int rc = dci_b200_add(m->shard[i], (const float *)m->data[i].p, (int)(hi - lo), block_size, thread_size, m->st[i])) {
            for (int j = 0; j <= i; ++j) dci_b200_clear(m->shard[j]);
            return rc;
        }
    }
    for (int i = 0; i < m->D; ++i) {
        DeviceGuard g(m->dev[i]);
        DCI_CUDA(cudaStreamSynchronize(m->st[i]));
    }
    m->num_points = num_points; m->dpd = dpd; m->P = block_size; m->T = thread_size;
    return 0;
}

int dci_b200_mdci_clear(dci_b200_mdci_t *m) {
    if (int rc = mdci_check(m)) return rc;
    for (int i = 0; i < m->D; ++i)
        if (int rc = dci_b200_clear(m->shard[i])) return rc;
    m->num_points = 0; m->dpd = 0;
    return 0;
}

int dci_b200_mdci_query(dci_b200_mdci_t *m, const float *d_query, int num_queries, int num_neighbours,
                        int num_outer_iterations, int max_num_candidates, long long *d_ids, float *d_dists,
                        void *stream) {
    if (int rc = mdci_check(m)) return rc;
    if (m->num_points <= 0) return fail(DCI_B200_ERR_STATE, "the index is empty; add data first");
    if (num_neighbours <= 0) return fail(DCI_B200_ERR_ARG, "num_neighbours must be positive");   // core.py:131-132
    if (num_neighbours > dci::kMaxTopK)
        return fail(DCI_B200_ERR_UNSUPPORTED, "dci_b200_mdci_query serves num_neighbours up to %d", dci::kMaxTopK);
    if (num_queries < 0) return fail(DCI_B200_ERR_ARG, "num_queries must not be negative");
    if (num_queries == 0) return 0;
    if (!d_query || !d_ids || !d_dists) return fail(DCI_B200_ERR_ARG, "null query or output pointer");
    const int k = num_neighbours, nq = num_queries;
    const size_t qbytes = sizeof(float) * (size_t)nq * m->dim, lbytes = sizeof(uint64_t) * (size_t)nq * k;
    cudaStream_t st0 = (cudaStream_t)stream;
    long long offsets[64];
    {
        DeviceGuard g(m->dev[0]);
        DCI_CUDA(m->gathered.ensure(lbytes * m->D));
        for (int i = 0; i < m->D; ++i)                                // a shard without rows: every slot empty
            if (dci_b200_num_points(m->shard[i]) <= 0)
                DCI_CUDA(cudaMemsetAsync((unsigned long long *)m->gathered.p + (size_t)i * nq * k, 0xFF, lbytes, st0));
        DCI_CUDA(cudaEventRecord(m->ev_query, st0));                  // the queries are ready from here on
    }
    for (int i = 0; i < m->D; ++i) {
        offsets[i] = m->dpd * i;                                      // core.py:149
        DeviceGuard g(m->dev[i]);
        cudaStream_t st = m->st[i];
        unsigned long long *dst = (unsigned long long *)m->gathered.p + (size_t)i * nq * k;
        const int n_i = dci_b200_num_points(m->shard[i]);
        DCI_CUDA(cudaStreamWaitEvent(st, m->ev_query, 0));
        if (n_i > 0) {
            const float *q = d_query;
            if (m->dev[i] != m->dev[0]) {                             // the reference copies the queries to every device, core.py:143
                DCI_CUDA(m->query[i].ensure(qbytes));
                DCI_CUDA(cudaMemcpyPeerAsync(m->query[i].p, m->dev[i], d_query, m->dev[0], qbytes, st));
                q = (const float *)m->query[i].p;
            }
            DCI_CUDA(m->lists[i].ensure(lbytes));
            const int k_i = std::min(k, n_i);                         // a shard shorter than k answers with what it has
            if (k_i == k) {
                if (int rc = dci_b200_query_packed(m->shard[i], q, nq, k, num_outer_iterations, max_num_candidates, m->P, m->T,
                                                   (unsigned long long *)m->lists[i].p, st)) return rc;
            } else {
                DCI_CUDA(m->tmp[i].ensure(sizeof(uint64_t) * (size_t)nq * k_i));
                if (int rc = dci_b200_query_packed(m->shard[i], q, nq, k_i, num_outer_iterations, max_num_candidates, m->P, m->T,
                                                   (unsigned long long *)m->tmp[i].p, st)) return rc;
                DCI_CUDA(cudaMemsetAsync(m->lists[i].p, 0xFF, lbytes, st));
                DCI_CUDA(cudaMemcpy2DAsync(m->lists[i].p, sizeof(uint64_t) * (size_t)k, m->tmp[i].p, sizeof(uint64_t) * (size_t)k_i,
                                           sizeof(uint64_t) * (size_t)k_i, (size_t)nq, cudaMemcpyDeviceToDevice, st));
            }
            DCI_CUDA(cudaMemcpyPeerAsync(dst, m->dev[0], m->lists[i].p, m->dev[i], lbytes, st));
        }
        DCI_CUDA(cudaEventRecord(m->ev[i], st));
    }
    DeviceGuard g(m->dev[0]);
    for (int i = 0; i < m->D; ++i) DCI_CUDA(cudaStreamWaitEvent(st0, m->ev[i], 0));
    return dci_b200_merge_shards_packed((const unsigned long long *)m->gathered.p, m->D, nq, k, offsets, d_ids, d_dists,
                                        m->dev[0], st0);
}

int dci_b200_mdci_query_host(dci_b200_mdci_t *m, const float *h_query, int num_queries, int num_neighbours,
                             int num_outer_iterations, int max_num_candidates, long long *h_ids, float *h_dists) {
    if (int rc = mdci_check(m)) return rc;
    if (num_queries < 0) return fail(DCI_B200_ERR_ARG, "num_queries must not be negative");
    if (num_queries == 0) return 0;
    if (!h_query || !h_ids || !h_dists) return fail(DCI_B200_ERR_ARG, "null query or output pointer");
    if (num_neighbours <= 0) return fail(DCI_B200_ERR_ARG, "num_neighbours must be positive");
    DeviceGuard g(m->dev[0]);
    const size_t qbytes = sizeof(float) * (size_t)num_queries * m->dim;
    const size_t n_out = (size_t)num_queries * num_neighbours;
    DCI_CUDA(m->q0.ensure(qbytes));
    DCI_CUDA(m->ids0.ensure(n_out * sizeof(long long)));
    DCI_CUDA(m->dists0.ensure(n_out * sizeof(float)));
    cudaStream_t st0 = m->st[0];
    DCI_CUDA(cudaMemcpyAsync(m->q0.p, h_query, qbytes, cudaMemcpyHostToDevice, st0));
    if (int rc = dci_b200_mdci_query(m, (const float *)m->q0.p, num_queries, num_neighbours, num_outer_iterations,
                                     max_num_candidates, (long long *)m->ids0.p, (float *)m->dists0.p, st0)) return rc;
    DCI_CUDA(cudaMemcpyAsync(h_ids, m->ids0.p, n_out * sizeof(long long), cudaMemcpyDeviceToHost, st0));
    DCI_CUDA(cudaMemcpyAsync(h_dists, m->dists0.p, n_out * sizeof(float), cudaMemcpyDeviceToHost, st0));
    DCI_CUDA(cudaStreamSynchronize(st0));
    return 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Query without any allocation (see include/dci_b200.h, dci_b200_query_noalloc).
// Its working memory is this fixed array, which every GPU that loads the
// library holds until the process exits.  In host code the symbol below is only
// a stand-in: the device address is obtained per device with
// cudaGetSymbolAddress and cached.
#define DCI_B200_NOALLOC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_noalloc_scratch[DCI_B200_NOALLOC_SCRATCH_BYTES];

namespace {

std::mutex g_noalloc_mutex;
unsigned char *g_noalloc_addr[64] = {nullptr};

// Device address of g_noalloc_scratch on `device`, which must be current.
int noalloc_scratch_address(int device, unsigned char **out) {
    if (device < 0 || device >= 64) return fail(DCI_B200_ERR_UNSUPPORTED, "device index %d out of range for the built-in scratch", device);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_addr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return fail(DCI_B200_ERR_CUDA, "cudaGetSymbolAddress(built-in scratch) failed on device %d: %s", device,
                        cudaGetErrorString(e));
        g_noalloc_addr[device] = (unsigned char *)p;
    }
    *out = g_noalloc_addr[device];
    return 0;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

template <typename ValT, typename PosT>
int query_noalloc_impl(dci_b200 *h, dci::TraverseParams prm, int nthreads, unsigned char *scratch, size_t avail,
                       int num_queries, int *d_ids, float *d_dists, cudaStream_t st) {
    cudaFuncAttributes fa;
    DCI_CUDA(cudaFuncGetAttributes(&fa, dci::traverse_kernel<ValT, PosT, true, true>));
    const size_t static_smem = fa.sharedSizeBytes;
    prm.nbuckets = pick_buckets<ValT>(h, prm, nthreads, static_smem);
    auto lay = dci::TraverseLayout<ValT>::make(nthreads, prm.dim, prm.topk_cap, prm.L, prm.wcap, prm.ppb, prm.nbuckets,
                                               prm.vec4 && !prm.vec8, prm.bkey != 0);
    if (lay.fixed_bytes + static_smem > h->smem_optin)
        return fail(DCI_B200_ERR_UNSUPPORTED, "dim=%d needs more shared memory per CTA than the device offers", prm.dim);
    const bool smem = lay.fixed_bytes + lay.big_bytes + static_smem <= h->smem_optin;
    if (!smem) lay = dci::TraverseLayout<ValT>::make(nthreads, prm.dim, prm.topk_cap, prm.L, prm.wcap, prm.ppb, prm.nbuckets, false, prm.bkey != 0);
    const size_t dyn = smem ? lay.fixed_bytes + lay.big_bytes : lay.fixed_bytes;
    const size_t per_cta = align256(lay.fallback_bytes + (smem ? 0 : lay.big_bytes));
    const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(h->smem_per_sm / (dyn + static_smem + 1024), 2048 / nthreads));
    const long long max_grid = std::min<long long>((long long)num_queries * prm.num_parts, (long long)h->sm_count * per_sm);
    const size_t slabs = per_cta * (size_t)max_grid;
    // per query of a pass: its per-partition result lists and its word of the shared distance bound
    const size_t per_query = sizeof(uint64_t) * (size_t)prm.num_parts * prm.kpart + sizeof(uint32_t);
    if (slabs + per_query + 256 > avail)
        return fail(DCI_B200_ERR_UNSUPPORTED,
                    "this index and k need %zu bytes of working memory, the built-in scratch of the allocation-free query holds %u",
                    slabs + per_query + 256 + ((size_t)DCI_B200_NOALLOC_SCRATCH_BYTES - avail), (unsigned)DCI_B200_NOALLOC_SCRATCH_BYTES);
    const int batch = (int)std::min<size_t>((size_t)num_queries, (avail - slabs - 256) / per_query);
    prm.gscratch = scratch;
    prm.gscratch_per_cta = per_cta;
    prm.part_topk = (uint64_t *)(scratch + slabs);
    uint32_t *qbound = h->distance_bound
                           ? (uint32_t *)(scratch + slabs + align256(sizeof(uint64_t) * (size_t)prm.num_parts * prm.kpart * batch))
                           : nullptr;
    const int merge_threads = 256;
    const int merge_cap = next_pow2(prm.knn + merge_threads);
    // the same kernel instances as the regular query
    const bool lean = !prm.blind && !prm.topk_global && prm.vec8 && !prm.work_stats && !prm.phase_cycles && prm.T > 1;
    void (*kern)(const dci::TraverseParams) =
        smem ? (lean ? dci::traverse_kernel<ValT, PosT, true, false, true> : dci::traverse_kernel<ValT, PosT, true, false, false>)
             : (lean ? dci::traverse_kernel<ValT, PosT, false, false, true> : dci::traverse_kernel<ValT, PosT, false, false, false>);
    DCI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    for (int q0 = 0; q0 < num_queries; q0 += batch) {
        prm.q0 = q0;
        prm.nq = std::min(batch, num_queries - q0);
        if (qbound) {      // the bound words must start as "no bound yet": the array keeps the last call's contents
            prm.qbound = qbound;
            DCI_CUDA(cudaMemsetAsync(qbound, 0x7F, sizeof(uint32_t) * (size_t)prm.nq, st));
        }
        const unsigned grid = (unsigned)std::min<long long>((long long)prm.nq * prm.num_parts, max_grid);
        kern<<<grid, nthreads, dyn, st>>>(prm);
        h->launches++;
        DCI_CUDA(cudaGetLastError());
        dci::merge_partitions_kernel<<<prm.nq, merge_threads, (size_t)merge_cap * 16, st>>>(
            prm.part_topk, prm.num_parts, prm.kpart, prm.knn, merge_cap, q0, prm.nq, nullptr, d_ids, d_dists, 0);
        h->launches++;
        DCI_CUDA(cudaGetLastError());
    }
    return 0;
}

}  // namespace

extern "C" int dci_b200_query_noalloc(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                                      int num_outer_iterations, int max_num_candidates, int block_size,
                                      int thread_size, int *d_ids, float *d_dists, void *stream) {
    if (int rc = check_handle(h)) return rc;
    if (h->num_points <= 0) return fail(DCI_B200_ERR_STATE, "the index is empty; add data first");
    if (num_queries < 0) return fail(DCI_B200_ERR_ARG, "num_queries must not be negative");
    if (num_queries == 0) return 0;
    if (!d_query || !d_ids || !d_dists) return fail(DCI_B200_ERR_ARG, "null query or output pointer");
    if (num_neighbours <= 0) return fail(DCI_B200_ERR_ARG, "num_neighbours must be positive, got %d", num_neighbours);
    if (num_neighbours > h->num_points)
        return fail(DCI_B200_ERR_ARG, "num_neighbours (%d) exceeds the number of indexed points (%d)", num_neighbours, h->num_points);
    if (num_neighbours > dci::kMaxTopK)
        return fail(DCI_B200_ERR_UNSUPPORTED, "num_neighbours above %d is not supported by the allocation-free query", dci::kMaxTopK);
    if (block_size != h->P || thread_size != h->T)
        return fail(DCI_B200_ERR_ARG, "block_size/thread_size (%d, %d) differ from the values the index was built with (%d, %d)",
                    block_size, thread_size, h->P, h->T);
    DeviceGuard g(h->device);
    if (!g.ok) return fail(DCI_B200_ERR_CUDA, "cannot select device %d", h->device);
    unsigned char *scratch = nullptr;
    if (int rc = noalloc_scratch_address(h->device, &scratch)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int I = h->L * h->S;
    // layout of the array: [flag word of the tensor-core projection, 256 B][projected queries][slabs][lists][bounds]
    const size_t qproj_bytes = align256(sizeof(float) * (size_t)I * num_queries);
    if (qproj_bytes + 256 >= (size_t)DCI_B200_NOALLOC_SCRATCH_BYTES)
        return fail(DCI_B200_ERR_UNSUPPORTED, "%d queries need %zu bytes for their projections alone, the built-in scratch holds %u",
                    num_queries, qproj_bytes, (unsigned)DCI_B200_NOALLOC_SCRATCH_BYTES);
    float *qproj = (float *)(scratch + 256);
    // the handle's own flag word and timing events are created on first use, so neither is used here
    if (int rc = launch_project(h, d_query, num_queries, qproj, st, (int *)scratch, false)) return rc;

    dci::TraverseParams prm;
    memset(&prm, 0, sizeof(prm));
    prm.skeys = (const float *)h->keys.p; prm.skeysT = (const float *)h->keysT.p; prm.sids = (const int *)h->ids.p;
    prm.spos = h->pos.p; prm.data = h->d_data;
    prm.qproj = qproj; prm.query = d_query;
    prm.N = h->num_points; prm.dim = h->dim; prm.L = h->L; prm.S = h->S; prm.P = h->P; prm.T = h->T;
    prm.ppb = h->ppb; prm.num_parts = h->num_parts; prm.nq_total = num_queries;
    prm.knn = num_neighbours; prm.max_cand = max_num_candidates;
    prm.outer_s = (long long)num_outer_iterations * h->S;
    prm.wcap = h->S * ((h->ppb + h->T - 1) / h->T + 2);
    prm.tshift = 0;
    while ((1 << prm.tshift) < h->T) ++prm.tshift;
    prm.divT = dci::FastDiv::make((uint32_t)h->T);
    prm.vec4 = (h->dim % 4 == 0) && (((uintptr_t)h->d_data & 15) == 0) && (((uintptr_t)d_query & 15) == 0);
    prm.vec8 = (h->dim % 8 == 0) && (((uintptr_t)h->d_data & 31) == 0);
    const int nthreads = prm.wcap >= 4096 ? 1024 : (prm.wcap >= 1024 ? 512 : (prm.wcap >= 256 ? 256 : 64));
    prm.kpart = std::min(num_neighbours, h->ppb);
    prm.topk_cap = next_pow2(prm.kpart + nthreads);
    unsigned char *rest = scratch + 256 + qproj_bytes;
    const size_t avail = (size_t)DCI_B200_NOALLOC_SCRATCH_BYTES - 256 - qproj_bytes;
    if (pos16(prm.ppb, h->T))
        return (prm.wcap <= 65535)
                   ? query_noalloc_impl<uint16_t, uint16_t>(h, prm, nthreads, rest, avail, num_queries, d_ids, d_dists, st)
                   : query_noalloc_impl<uint32_t, uint16_t>(h, prm, nthreads, rest, avail, num_queries, d_ids, d_dists, st);
    return query_noalloc_impl<uint32_t, uint32_t>(h, prm, nthreads, rest, avail, num_queries, d_ids, d_dists, st);
}
