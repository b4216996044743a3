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

// nbuckets > 0: room for the counting rank (bucket counters over the radix histogram's place, one
// arrival byte per key); 0: radix sort only.
template <typename ValT>
struct BuildLayout {
    size_t hist_bytes, slot_bytes, buf_bytes;
    __host__ __device__ static size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }
    __host__ __device__ static BuildLayout make(int nthreads, int cap, int nbuckets) {
        BuildLayout l;
        const size_t radix = (size_t)256 * (nthreads / 32) * sizeof(ValT);
        const size_t counters = nbuckets > 0 ? (size_t)(nbuckets + 16) * sizeof(ValT) : 0;
        l.hist_bytes = align16(radix > counters ? radix : counters);
        l.slot_bytes = nbuckets > 0 ? align16((size_t)cap) : 0;
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
                      unsigned char *gscratch, size_t gscratch_per_cta, int nbuckets) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    __shared__ uint32_t warp_tot[40];
    __shared__ uint32_t s_lohi[2];
    const BuildLayout<ValT> lay = BuildLayout<ValT>::make(blockDim.x, ppb, SMEM ? nbuckets : 0);
    ValT *hist = reinterpret_cast<ValT *>(dyn_smem);
    uint8_t *slot = reinterpret_cast<uint8_t *>(dyn_smem + lay.hist_bytes);
    unsigned char *big = SMEM ? dyn_smem + lay.hist_bytes + lay.slot_bytes : gscratch + (size_t)blockIdx.x * gscratch_per_cta;
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
        uint32_t kmin = 0xFFFFFFFFu, kmax = 0u;
        for (int x = threadIdx.x; x < n; x += blockDim.x) {
            const uint32_t k = float_to_ordered(keys_unsorted[urow + x]);
            kA[x] = k;
            kmin = min(kmin, k); kmax = max(kmax, k);
        }
        const uint32_t *ks = kA;          // the sorted keys and the points they belong to, once sorted
        const ValT *vs = vA;
        bool ranked = false;
        if (SMEM && nbuckets > 0) {
            // Counting rank: the keys are dropped into equal-width value buckets between the segment's
            // smallest and largest key (about two buckets per key), a scan gives the bucket starts, and a
            // key's place is its bucket's start plus the number of smaller keys (ties by point id) among
            // its few bucket mates.  One pass over the keys each instead of the radix sort's eight.
            if (threadIdx.x == 0) { s_lohi[0] = 0xFFFFFFFFu; s_lohi[1] = 0u; }
            cta_zero16(hist, lay.hist_bytes);
            __syncthreads();
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                kmin = min(kmin, __shfl_xor_sync(0xFFFFFFFFu, kmin, o));
                kmax = max(kmax, __shfl_xor_sync(0xFFFFFFFFu, kmax, o));
            }
            if ((threadIdx.x & 31) == 0) { atomicMin(&s_lohi[0], kmin); atomicMax(&s_lohi[1], kmax); }
            __syncthreads();
            const float fmin_ = ordered_to_float(s_lohi[0]), range = ordered_to_float(s_lohi[1]) - fmin_;
            const bool usable = range > 0.0f && range < 3.0e38f;
            const float scale = usable ? (float)nbuckets / range : 0.0f;
            const int last = nbuckets - 1;
            auto bucket = [fmin_, scale, last](uint32_t k) {
                return bucket_of(__float_as_uint(ordered_to_float(k) - fmin_), scale, last);
            };
            int over = usable ? 0 : 1;
            if (usable)
                for (int x = threadIdx.x; x < n; x += blockDim.x) {
                    const uint32_t arrival = bucket_arrive(hist, bucket(kA[x]));
                    over |= (arrival >= (uint32_t)kMaxBucket);      // the arrival that makes a bucket too large reports it
                    slot[x] = (uint8_t)min(arrival, 255u);
                }
            over = __syncthreads_or(over);
            if (!over) {
                cta_bucket_place_and_rank<ValT, ValT>(kA, n, slot, vA, kB, hist, nbuckets, bucket, warp_tot, vB,
                                                      [](uint32_t a, uint32_t b2) { return a < b2; }, [](int) {});
                for (int x = threadIdx.x; x < n; x += blockDim.x) {       // vB[x] = place of point x
                    const uint32_t r = vB[x];
                    kB[r] = kA[x];
                    vA[r] = (ValT)x;
                }
                __syncthreads();
                ks = kB;
                ranked = true;
            }
        }
        if (!ranked) {                     // many equal keys (or no shared memory for the counters): radix sort
            for (int x = threadIdx.x; x < n; x += blockDim.x) vA[x] = (ValT)x;
            __syncthreads();
            cta_radix_sort<ValT, ValT, false>(kA, vA, kB, vB, n, hist, warp_tot, (ValT *)nullptr);
        }
        const int qn = n / T, rem = n % T;
        // every output array is written in its own order, so that the stores of a warp are contiguous:
        // the stride-T keys residue class by residue class (while T is small enough for that to keep
        // the threads busy), the positions from the ranks, which are indexed by point
        for (int x = threadIdx.x; x < n; x += blockDim.x) {
            skeys[row + x] = ordered_to_float(ks[x]);
            sids[row + x] = (int)(lo + vs[x]);
            if (ranked) spos[prow + x] = vB[x];
            else spos[prow + vs[x]] = (ValT)x;
        }
        if (T <= 64) {
            for (int r = 0; r < T; ++r) {
                const size_t base = row + (size_t)r * qn + min(r, rem);
                const int cnt = qn + (r < rem ? 1 : 0);
                for (int j = threadIdx.x; j < cnt; j += blockDim.x) skeysT[base + j] = ordered_to_float(ks[j * T + r]);
            }
        } else {
            for (int x = threadIdx.x; x < n; x += blockDim.x) {
                const int r = x % T, j = x / T;
                skeysT[row + r * qn + min(r, rem) + j] = ordered_to_float(ks[x]);
            }
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
