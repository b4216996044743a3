// Index build: one stable radix sort per (simple index, partition) segment.
// Replaces copy_to_indices + sort_indices (+ the recursive device quicksort)
// of the reference (src/dci_cuda_kernel.cu:113-146, 190-247).  The result is
// kept as flat arrays keys / ids (SoA) instead of the reference's array of
// {key, id} structs (include/dci.h:27-30), plus the inverse permutation pos:
// the position of point p inside its partition's sorted segment of simple
// index i (16-bit when partitions hold fewer than 65 536 points), which lets a
// query look a point's window up directly instead of scattering over index
// entries.  All four arrays are PARTITION-MAJOR: the I segments of a partition
// lie next to each other (segment_start), so that a work item of the traversal
// -- one query against one partition -- touches one contiguous range of each
// array instead of I ranges that are N entries apart.  A third copy of the keys,
// keysT, holds every segment "stride-T transposed": the key at sorted position
// y = j*T + r sits at r*(n/T) + min(r, n%T) + j, so that the keys at positions
// r, r+T, r+2T, ... -- the window starts of one query -- are contiguous.
// Equal keys are ordered by id (the input order), which the reference leaves
// unspecified.
#pragma once
#include "common.cuh"

namespace dci {

template <typename ValT>
struct BuildLayout {
    size_t hist_bytes, buf_bytes;
    __host__ __device__ static size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }
    __host__ __device__ static BuildLayout make(int nthreads, int cap) {
        BuildLayout l;
        l.hist_bytes = align16((size_t)256 * (nthreads / 32) * sizeof(ValT));
        l.buf_bytes = align16((size_t)cap * 4) * 2 + align16((size_t)cap * sizeof(ValT)) * 2;
        return l;
    }
};

// Persistent CTAs; CTA c sorts segments c, c + gridDim.x, ...
// SMEM: the ping-pong buffers live in dynamic shared memory; otherwise in the
// CTA's slab of `gscratch`.
template <typename ValT, bool SMEM>
__global__ void __launch_bounds__(1024)
build_segments_kernel(const float *__restrict__ keys_unsorted, int N, int num_indices, int ppb,
                      int num_parts, float *__restrict__ skeys, int *__restrict__ sids,
                      ValT *__restrict__ spos, float *__restrict__ skeysT, int T,
                      unsigned char *gscratch, size_t gscratch_per_cta) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ uint32_t warp_tot[40];
    const BuildLayout<ValT> lay = BuildLayout<ValT>::make(blockDim.x, ppb);
    ValT *hist = reinterpret_cast<ValT *>(dyn_smem);
    unsigned char *big = SMEM ? dyn_smem + lay.hist_bytes : gscratch + (size_t)blockIdx.x * gscratch_per_cta;
    const size_t kbytes = BuildLayout<ValT>::align16((size_t)ppb * 4);
    const size_t vbytes = BuildLayout<ValT>::align16((size_t)ppb * sizeof(ValT));
    uint32_t *kA = reinterpret_cast<uint32_t *>(big);
    uint32_t *kB = reinterpret_cast<uint32_t *>(big + kbytes);
    ValT *vA = reinterpret_cast<ValT *>(big + 2 * kbytes);
    ValT *vB = reinterpret_cast<ValT *>(big + 2 * kbytes + vbytes);
    const long long nseg = (long long)num_indices * num_parts;
    for (long long seg = blockIdx.x; seg < nseg; seg += gridDim.x) {
        const int i = (int)(seg / num_parts), b = (int)(seg % num_parts);
        const long long lo = (long long)b * ppb;
        const int n = (int)min((long long)ppb, (long long)N - lo);
        const size_t row = segment_start(lo, i, num_indices, n);
        const size_t urow = (size_t)i * N + lo;               // the projection writes [I][N]
        const size_t prow = pos_segment_start(b, i, num_indices, ppb);
        for (int x = threadIdx.x; x < n; x += blockDim.x) {
            kA[x] = float_to_ordered(keys_unsorted[urow + x]);
            vA[x] = (ValT)x;
        }
        __syncthreads();
        cta_radix_sort<ValT, ValT, false>(kA, vA, kB, vB, n, hist, warp_tot, (ValT *)nullptr);
        const int qn = n / T, rem = n % T;
        for (int x = threadIdx.x; x < n; x += blockDim.x) {
            const int r = x % T, j = x / T;
            skeysT[row + r * qn + min(r, rem) + j] = ordered_to_float(kA[x]);
            skeys[row + x] = ordered_to_float(kA[x]);
            sids[row + x] = (int)(lo + vA[x]);
            spos[prow + vA[x]] = (ValT)x;
        }
        for (int x = n + threadIdx.x; x < pos_stride(ppb); x += blockDim.x) spos[prow + x] = (ValT)0;
        __syncthreads();
    }
}

// Installs a sorted index that was produced elsewhere (a saved index, or the reference's own
// `indices` array, include/dci.h:44): in_keys / in_ids are [I][N] with every partition's segment
// sorted; the kernel checks them and writes the partition-major keys, ids, inverse positions and
// stride-T keys.  One CTA per (simple index, partition) segment, looping.
template <typename PosT>
__global__ void derive_index_kernel(const float *__restrict__ in_keys, const int *__restrict__ in_ids, int N,
                                    int num_indices, int ppb, int num_parts, int T, float *__restrict__ skeys,
                                    int *__restrict__ sids, PosT *__restrict__ spos, float *__restrict__ skeysT,
                                    int *bad) {
    const long long nseg = (long long)num_indices * num_parts;
    for (long long seg = blockIdx.x; seg < nseg; seg += gridDim.x) {
        const int i = (int)(seg / num_parts), b = (int)(seg % num_parts);
        const long long lo = (long long)b * ppb;
        const int n = (int)min((long long)ppb, (long long)N - lo);
        const size_t row = segment_start(lo, i, num_indices, n);
        const size_t urow = (size_t)i * N + lo;
        const size_t prow = pos_segment_start(b, i, num_indices, ppb);
        const int qn = n / T, rem = n % T;
        for (int x = threadIdx.x; x < n; x += blockDim.x) {
            const long long p = (long long)in_ids[urow + x] - lo;
            const float key = in_keys[urow + x];
            if (p < 0 || p >= n || (x > 0 && key < in_keys[urow + x - 1])) {
                atomicExch(bad, 1);        // id outside its partition or keys not ascending
                continue;
            }
            skeys[row + x] = key;
            sids[row + x] = in_ids[urow + x];
            spos[prow + p] = (PosT)x;
            const int r = x % T, j = x / T;
            skeysT[row + r * qn + min(r, rem) + j] = key;
        }
    }
}

// Second half of the validation of an installed index: every point of a partition must occur exactly
// once in each of its segments.  The caller fills spos with 0xFF bytes before derive_index_kernel, so
// a point that no entry named still holds the sentinel (>= n), and a point named twice leaves another
// one unnamed.  Sets *bad otherwise, and zeroes the padding behind each segment's positions.  Same
// segment loop as derive_index_kernel.
template <typename PosT>
__global__ void check_index_kernel(const int *__restrict__ sids, PosT *__restrict__ spos, int N,
                                   int num_indices, int ppb, int num_parts, int *bad) {
    const long long nseg = (long long)num_indices * num_parts;
    for (long long seg = blockIdx.x; seg < nseg; seg += gridDim.x) {
        const int i = (int)(seg / num_parts), b = (int)(seg % num_parts);
        const long long lo = (long long)b * ppb;
        const int n = (int)min((long long)ppb, (long long)N - lo);
        const size_t row = segment_start(lo, i, num_indices, n);
        const size_t prow = pos_segment_start(b, i, num_indices, ppb);
        for (int p = threadIdx.x; p < n; p += blockDim.x) {
            const long long x = (long long)spos[prow + p];
            if (x >= n || (long long)sids[row + x] != lo + p) atomicExch(bad, 1);
        }
        for (int p = n + threadIdx.x; p < pos_stride(ppb); p += blockDim.x) spos[prow + p] = (PosT)0;
    }
}

// Sorted index back to [I][N] arrays: out_keys / out_ids (either may be null) receive the sorted
// segments in the layout callers see (dci_b200_get_index).
__global__ void export_index_kernel(const float *__restrict__ skeys, const int *__restrict__ sids, int N,
                                    int num_indices, int ppb, int num_parts, float *__restrict__ out_keys,
                                    int *__restrict__ out_ids) {
    const long long nseg = (long long)num_indices * num_parts;
    for (long long seg = blockIdx.x; seg < nseg; seg += gridDim.x) {
        const int i = (int)(seg / num_parts), b = (int)(seg % num_parts);
        const long long lo = (long long)b * ppb;
        const int n = (int)min((long long)ppb, (long long)N - lo);
        const size_t row = segment_start(lo, i, num_indices, n);
        const size_t urow = (size_t)i * N + lo;
        for (int x = threadIdx.x; x < n; x += blockDim.x) {
            if (out_keys) out_keys[urow + x] = skeys[row + x];
            if (out_ids) out_ids[urow + x] = sids[row + x];
        }
    }
}

// Inverse of the build's sort, for appending rows: writes the key of every indexed point back to
// out[i][id], `out` having rows of `out_stride` floats.
__global__ void unsort_keys_kernel(const float *__restrict__ skeys, const int *__restrict__ sids, int N,
                                   int num_indices, int ppb, int num_parts, float *__restrict__ out,
                                   int out_stride) {
    const long long nseg = (long long)num_indices * num_parts;
    for (long long seg = blockIdx.x; seg < nseg; seg += gridDim.x) {
        const int i = (int)(seg / num_parts), b = (int)(seg % num_parts);
        const long long lo = (long long)b * ppb;
        const int n = (int)min((long long)ppb, (long long)N - lo);
        const size_t row = segment_start(lo, i, num_indices, n);
        for (int x = threadIdx.x; x < n; x += blockDim.x)
            out[(size_t)i * out_stride + sids[row + x]] = skeys[row + x];
    }
}

}  // namespace dci
