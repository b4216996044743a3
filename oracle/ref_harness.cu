/*
 * ref_harness.cu -- TEST INFRASTRUCTURE ONLY.
 *
 * A C-ABI wrapper that is compiled TOGETHER WITH the reference project's own,
 * unmodified CUDA sources (src/dci_cuda_kernel.cu, src/util_kernel.cu; see
 * oracle/build_ref.py) so that tests and the benchmark's reference arm can
 * drive the reference's C API (include/dci.h:58-84) without its PyTorch shim:
 * create an instance, read or overwrite its projection directions, add data,
 * read the built index back, and query.  None of the reference's code is
 * reproduced here; this file only calls it.
 */
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "dci.h"
#include "util.h"

#define REF_CHECK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    snprintf(g_err, sizeof(g_err), "%s:%d %s", __FILE__, __LINE__, cudaGetErrorString(e_)); return -1; } } while (0)

static char g_err[512] = "";

extern "C" const char *ref_last_error(void) { return g_err; }

/* The reference sorts with a recursive device quicksort (dci_cuda_kernel.cu:
 * 206-247); with the default 1 KiB device stack that is only safe for the small
 * partitions of its example.  The harness raises the per-thread stack limit of
 * its own context before any reference kernel runs. */
extern "C" int ref_dci_create(void **out, int dim, int L, int S, int device) {
    REF_CHECK(cudaSetDevice(device));
    REF_CHECK(cudaDeviceSetLimit(cudaLimitStackSize, 32 * 1024));
    dci *inst = NULL;
    REF_CHECK(cudaMallocManaged((void **)&inst, sizeof(dci)));
    memset(inst, 0, sizeof(dci));
    dci_init(inst, dim, L, S, device);
    REF_CHECK(cudaDeviceSynchronize());
    REF_CHECK(cudaGetLastError());
    *out = inst;
    return 0;
}

extern "C" int ref_dci_get_proj(void *h, float *host_out) {
    dci *inst = (dci *)h;
    REF_CHECK(cudaDeviceSynchronize());
    size_t n = (size_t)inst->dim * inst->num_comp_indices * inst->num_simp_indices;
    REF_CHECK(cudaMemcpy(host_out, inst->proj_vec, n * sizeof(float), cudaMemcpyDefault));
    return 0;
}

extern "C" int ref_dci_set_proj(void *h, const float *host_in) {
    dci *inst = (dci *)h;
    REF_CHECK(cudaDeviceSynchronize());
    size_t n = (size_t)inst->dim * inst->num_comp_indices * inst->num_simp_indices;
    REF_CHECK(cudaMemcpy(inst->proj_vec, host_in, n * sizeof(float), cudaMemcpyDefault));
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

extern "C" int ref_dci_add(void *h, int num_points, float *d_data, int block_size, int thread_size) {
    dci *inst = (dci *)h;
    dci_add(inst, inst->dim, num_points, d_data, block_size, thread_size);
    REF_CHECK(cudaDeviceSynchronize());
    REF_CHECK(cudaGetLastError());
    return 0;
}

/* Copies the built index out as SoA: keys[I][N], ids[I][N]. */
extern "C" int ref_dci_get_index(void *h, float *host_keys, int *host_ids) {
    dci *inst = (dci *)h;
    REF_CHECK(cudaDeviceSynchronize());
    size_t n = (size_t)inst->num_points * inst->num_comp_indices * inst->num_simp_indices;
    idx_elem *tmp = (idx_elem *)malloc(n * sizeof(idx_elem));
    if (!tmp) { snprintf(g_err, sizeof(g_err), "host alloc failed"); return -1; }
    cudaError_t e = cudaMemcpy(tmp, inst->indices, n * sizeof(idx_elem), cudaMemcpyDefault);
    if (e != cudaSuccess) { free(tmp); REF_CHECK(e); }
    for (size_t x = 0; x < n; ++x) { host_keys[x] = tmp[x].key; host_ids[x] = tmp[x].value; }
    free(tmp);
    return 0;
}

/* Projects queries exactly as dci_query does (dci_cuda_kernel.cu:802-803): the
 * same cuBLAS call with the same shapes; out is [nq][I] on the host. */
extern "C" int ref_dci_project_queries(void *h, int nq, const float *d_query, float *host_out) {
    dci *inst = (dci *)h;
    int I = inst->num_comp_indices * inst->num_simp_indices;
    float *qp = NULL;
    int dev = 0;
    REF_CHECK(cudaMallocManaged((void **)&qp, sizeof(float) * (size_t)I * nq));
    matmul_device(CUBLAS_OP_N, CUBLAS_OP_T, nq, I, inst->dim, d_query, inst->proj_vec, qp, dev);
    REF_CHECK(cudaDeviceSynchronize());
    REF_CHECK(cudaMemcpy(host_out, qp, sizeof(float) * (size_t)I * nq, cudaMemcpyDefault));
    REF_CHECK(cudaFree(qp));
    return 0;
}

extern "C" int ref_dci_query(void *h, int nq, const float *d_query, int k, int num_outer_iterations,
                             int max_num_candidates, int block_size, int thread_size,
                             int *d_ids, float *d_dists) {
    dci *inst = (dci *)h;
    dci_query_config cfg;
    cfg.blind = false;
    cfg.num_outer_iterations = num_outer_iterations;
    cfg.max_num_candidates = max_num_candidates;
    dci_query(inst, inst->dim, nq, d_query, k, cfg, d_ids, d_dists, block_size, thread_size);
    REF_CHECK(cudaDeviceSynchronize());
    REF_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int ref_dci_clear(void *h) {
    dci_clear((dci *)h);
    REF_CHECK(cudaDeviceSynchronize());
    return 0;
}

extern "C" int ref_dci_destroy(void *h) {
    dci *inst = (dci *)h;
    dci_free(inst);
    REF_CHECK(cudaFree(inst));
    return 0;
}
