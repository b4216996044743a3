/*
 * dci_b200.h -- C ABI of the B200-native Prioritized DCI k-NN engine.
 *
 * This is the boundary a host binding loads (ctypes, cgo, JNI, a PyTorch
 * extension ...).  It replaces, function for function, the C API of the
 * reference project (include/dci.h:58-84) and the pybind entry points built on
 * it (src/dci_cuda.cpp:175-183).  Differences from that API, all deliberate:
 *   - extern "C", opaque handle, every call returns a status (0 = ok) and
 *     dci_b200_last_error() describes the last failure of the calling thread
 *     (the reference returns void and checks no CUDA error);
 *   - the caller allocates the outputs (the reference cudaMallocs them and
 *     never frees them, src/dci_cuda.cpp:100-101);
 *   - work is enqueued on the stream the caller passes (the reference uses the
 *     legacy default stream and synchronises the device after every kernel);
 *   - projection directions can be read and written, and the generator takes
 *     an explicit seed (the reference seeds cuRAND from the process-global
 *     rand(), src/util_kernel.cu:124-127).
 *
 * All pointers named d_* are device pointers on the handle's device; h_* are
 * host pointers.  `stream` is a cudaStream_t passed as void* (NULL = default
 * stream).  Unless stated otherwise calls are asynchronous with respect to the
 * host: results are complete when the stream reaches the end of the enqueued
 * work.
 *
 * Concurrency: a handle owns one set of work buffers (projected queries,
 * per-partition lists, slabs, statistics) that grow on demand and are reused by
 * every call.  At most one call per handle may be in flight: use one stream per
 * handle (or order the streams yourself), and do not call a handle from two
 * threads at once.  Growing a buffer frees the old one, so a call that needs
 * more room than any before it must not overlap earlier work of the same
 * handle on another stream.  dci_b200_query_host uses the legacy default
 * stream and synchronises it; that stream does not order against non-blocking
 * streams.  Different handles are independent.
 */
#ifndef DCI_B200_H
#define DCI_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dci_b200 dci_b200_t;
typedef struct dci_b200_mdci dci_b200_mdci_t;   /* one index sharded over several devices, see the end of this file */

enum {
    DCI_B200_OK = 0,
    DCI_B200_ERR_ARG = 1,        /* bad argument (message says which)          */
    DCI_B200_ERR_STATE = 2,      /* e.g. add() on a non-empty index            */
    DCI_B200_ERR_CUDA = 3,       /* a CUDA call failed                         */
    DCI_B200_ERR_UNSUPPORTED = 4 /* e.g. a partition beyond the size limits    */
};

/* Message for the last non-zero status returned to this thread. */
const char *dci_b200_last_error(void);

/* Version of this ABI (increases when a signature changes). */
int dci_b200_abi_version(void);

/* Replaces dci_init (include/dci.h:61-62, src/dci_cuda_kernel.cu:93-110) and
 * _dci_new (src/dci_cuda.cpp:54-66): creates an empty index for `dim`-
 * dimensional points with L = num_comp_indices composite indices of
 * S = num_simp_indices simple indices each, on CUDA device `device`, and
 * generates L*S Gaussian unit directions from `seed` on the device
 * (replaces dci_gen_proj_vec, src/dci_cuda_kernel.cu:77-90).  Synchronous. */
int dci_b200_create(dci_b200_t **out, int dim, int num_comp_indices, int num_simp_indices,
                    int device, unsigned long long seed);

/* Replaces dci_free (include/dci.h:82) and _dci_free.  Synchronous. */
int dci_b200_destroy(dci_b200_t *h);

/* Directions, row-major [L*S][dim], row i = h + m*S for simple index h of
 * composite index m (same layout as the reference's proj_vec, include/dci.h:45).
 * The reference has no such accessors; parity tests need them.  Synchronous.
 * set_proj is rejected while the index holds points. */
int dci_b200_get_proj(dci_b200_t *h, float *h_out);
int dci_b200_set_proj(dci_b200_t *h, const float *h_in);

/* Replaces dci_add (include/dci.h:68-69, src/dci_cuda_kernel.cu:149-187) and
 * _dci_add: projects the num_points rows of d_data ([num_points][dim] fp32,
 * row-major) on every direction and sorts each (simple index, partition)
 * segment by (key, id).  block_size = number of partitions P (each partition
 * is the id range [b*ppb, (b+1)*ppb), ppb = ceil(num_points / P));
 * thread_size = the window width T used by queries.  Both are semantic
 * parameters in the reference (src/dci_cuda_kernel.cu:178, :424-427, :487).
 * As in the reference the index BORROWS d_data: it must stay valid and
 * unchanged until clear/reset/destroy.  A second add without clear fails with
 * DCI_B200_ERR_STATE (dciknn_cuda/core.py:70-71). */
int dci_b200_add(dci_b200_t *h, const float *d_data, int num_points, int block_size,
                 int thread_size, void *stream);

/* No counterpart in the reference, whose dci_add refuses a second array
 * (src/dci_cuda_kernel.cu:157, dciknn_cuda/core.py:70-71): grows an index that
 * already holds N0 points to num_points_total > N0 points.  d_all_data is
 * [num_points_total][dim]; its first N0 rows must be the rows already indexed,
 * unchanged (the caller appends in place or copies them).  Only the new rows
 * are projected; the old rows' keys are recovered from the sorted index; every
 * segment is then sorted again for the partition bounds of the new count
 * (ppb = ceil(num_points_total / P), with the P and T of the first add).  The
 * result is the index dci_b200_add would build from d_all_data, bit for bit.
 * The index borrows d_all_data from then on.  Synchronises the stream. */
int dci_b200_append(dci_b200_t *h, const float *d_all_data, int num_points_total, void *stream);

/* Replaces dci_query (include/dci.h:71-75, src/dci_cuda_kernel.cu:777-875) and
 * _dci_query: for each of the num_queries rows of d_query returns the
 * num_neighbours candidates nearest in Euclidean distance among the points the
 * prioritized traversal promotes, rows ascending by (distance, id).
 * num_outer_iterations / max_num_candidates are the fields of
 * dci_query_config (include/dci.h:52-56) and stop each partition's traversal
 * exactly as the reference does (src/dci_cuda_kernel.cu:598-607).
 * block_size / thread_size must equal the values given to add (the reference
 * passes them on every call).  blind != 0 returns DCI_B200_ERR_UNSUPPORTED:
 * blind results have another length, see dci_b200_query_blind.
 * d_ids: [num_queries][num_neighbours] int32, d_dists: same shape fp32.  Slots
 * beyond the number of promoted points hold id -1 and distance +inf.
 * Any 1 <= num_neighbours <= num_points is accepted; above 1024 the selection
 * buffers move from shared to global memory and the query is slower. */
int dci_b200_query(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                   int num_outer_iterations, int max_num_candidates, int blind,
                   int block_size, int thread_size, int *d_ids, float *d_dists, void *stream);

/* dci_b200_query with the result in the form MDCI ships between GPUs (replaces the two float
 * tensors that dciknn_cuda/core.py:146-151 moves per device): d_packed is
 * [num_queries][num_neighbours] 64-bit keys, (fp32 bits of the distance << 32) | id, rows
 * ascending, all ones in slots beyond the number of promoted points.  Input of
 * dci_b200_merge_shards_packed. */
int dci_b200_query_packed(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                          int num_outer_iterations, int max_num_candidates, int block_size,
                          int thread_size, unsigned long long *d_packed, void *stream);

/* A working form of the reference's blind querying, which its comments specify
 * (src/dci_cuda_kernel.cu:398-399, :775-776: no distance is computed, no
 * indexed vector is read, the result is the candidates "in the order of
 * retrieval", max_possible_num_candidates = min(max_num_candidates,
 * num_outer_iterations) per query, :784-785) but whose code cannot run
 * (unsynchronised candidate counter :498-505, host reads of device memory
 * :770-772, output sized for k ids by src/dci_cuda.cpp:99-100).  The traversal
 * and its stop rule are those of dci_b200_query with the same arguments.
 * Partitions are traversed side by side, so "order of retrieval" is defined
 * as ascending (iteration of the partition's loop at which the point was
 * promoted, point id).  d_ids: [num_queries][width] int32 with width =
 * dci_b200_blind_width(num_outer_iterations, max_num_candidates), -1 in unused
 * slots; d_iterations: the same shape, the promotion iterations (-1 in unused
 * slots), or NULL.  dci_b200_query itself refuses blind != 0 because its
 * outputs have another length. */
int dci_b200_blind_width(int num_outer_iterations, int max_num_candidates);
int dci_b200_query_blind(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                         int num_outer_iterations, int max_num_candidates, int block_size,
                         int thread_size, int *d_ids, int *d_iterations, void *stream);

/* Same query with HOST buffers: copies the queries to the device, runs the
 * query and copies ids and distances back.  Synchronous. */
int dci_b200_query_host(dci_b200_t *h, const float *h_query, int num_queries, int num_neighbours,
                        int num_outer_iterations, int max_num_candidates, int blind,
                        int block_size, int thread_size, int *h_ids, float *h_dists);

/* Replace dci_clear / dci_reset (include/dci.h:77-80, src/dci_cuda_kernel.cu:
 * 878-891): clear drops the indexed points and keeps the directions; reset also
 * draws new directions from `seed`.  Synchronous.  The device buffers of the
 * index are kept for the next add and returned by dci_b200_destroy. */
int dci_b200_clear(dci_b200_t *h);
int dci_b200_reset(dci_b200_t *h, unsigned long long seed);

/* Number of points currently indexed. */
int dci_b200_num_points(dci_b200_t *h);

/* Copies the built index to the host as keys[L*S][N] and ids[L*S][N] (each
 * partition's segment ascending by (key, id)); the counterpart of reading the
 * reference's `indices` array (include/dci.h:44).  For tests.  Synchronous. */
int dci_b200_get_index(dci_b200_t *h, float *h_keys, int *h_ids);

/* Installs an index that was built elsewhere -- one saved with get_index, or the
 * reference's own sorted `indices` array -- instead of projecting and sorting:
 * h_keys / h_ids are host arrays [L*S][num_points] in get_index's layout, built
 * for the same directions, block_size and thread_size.  The derived arrays are
 * rebuilt on the device; a segment that is not ascending, or an id outside its
 * partition, is rejected with DCI_B200_ERR_ARG.  d_data is borrowed as in add.
 * (The reference cannot save or load an index.)  Synchronous. */
int dci_b200_set_index(dci_b200_t *h, const float *d_data, int num_points, int block_size, int thread_size,
                       const float *h_keys, const int *h_ids, void *stream);

/* Projects n rows of d_x on the handle's directions with the library's exact
 * fp32 path: d_out[i][p] = <proj[i], x[p]>, layout [L*S][n].  For tests. */
int dci_b200_project(dci_b200_t *h, const float *d_x, int n, float *d_out, void *stream);

/* `on` is a bit mask: bit 0 = per-work-item counters, bit 1 = per-phase cycle
 * sums (see get_phase_cycles), 0 = off.  With bit 0 every later query also records, per (query,
 * partition) work item, what the reference's loop would have done:
 * [0] the outer iteration it stops at, [1] windows visited, [2] index entries
 * looked at, [3] points promoted, [4] promotions in lane 0, [5] 1 if every
 * window of the partition was visited.  get_work_stats copies the records of
 * the last query to the host as [num_queries][P][6] int64.  Synchronous. */
int dci_b200_enable_work_stats(dci_b200_t *h, int on);
int dci_b200_get_work_stats(dci_b200_t *h, long long *h_out, long long capacity_records);

/* With bit 1 of enable_work_stats set the traversal kernel also sums, over all work
 * items of the last query, the SM cycles one CTA spent in each of its phases:
 * h_out (16 entries): [0] query load + split search, [1] window priorities +
 * bucket counts, [2] window ranking inside buckets (or the radix-sort fallback),
 * [3] promotion iterations, [4] stop rule + candidate list (+ the counters
 * above), [5] distances, [6] top-k, [8] bucket scan, [9] bucket placement,
 * [10] counter reset; [11] queries per CTA pass of the last launch, [13] whether
 * the last projection used the TMA-fed kernel (host values); [15] = number of
 * work items.  Synchronous. */
int dci_b200_get_phase_cycles(dci_b200_t *h, long long *h_out);

/* Number of kernels this library launched on behalf of this handle so far. */
long long dci_b200_launch_count(dci_b200_t *h);

/* Number of cudaMalloc and cudaFree calls this library has issued in this process, over all
 * handles (every one of them goes through one counted wrapper).  Lets a caller, or a test, see
 * that a call allocated nothing: the count is the same before and after. */
long long dci_b200_device_alloc_calls(void);

/* Caps the number of CTAs of the traversal kernel (0, the default: as many as the device keeps
 * resident).  A diagnostic: with few CTAs each one works through many (query, partition) pairs in a
 * row, so tests reach whatever a CTA keeps from one pair to the next. */
int dci_b200_set_max_ctas(dci_b200_t *h, int max_ctas);

/* How data and queries are projected on the directions (replaces the
 * cublasSgemm calls of src/util_kernel.cu:45-80).  0 (default): exact fp32, one
 * fused multiply-add per term in ascending coordinate order -- the path every
 * parity test pins.  1: 5th-generation tensor cores (tcgen05.mma, fp32 operands
 * split into two tf32 terms, "3xTF32") in persistent, warp-specialised CTAs fed
 * by TMA (when dim is a multiple of 4 and the pointers are 16-byte aligned;
 * otherwise as mode 2); 2: the same MMAs with plain loads; 3: one TMA-fed tile
 * per CTA.  Keys of modes 1-3 differ from mode 0 by about
 * 1e-6 * |x|, which can move a point across a window boundary, so results are
 * not guaranteed identical to mode 0.  Modes 1-3 synchronise the stream after
 * each projection to check its bounded waits.  In mode 0, inputs of at least
 * 1024 rows whose dim is a multiple of 4 (16-byte aligned base, at most 40
 * directions) are streamed into shared memory by TMA copies; mode 4 is mode 0
 * with the rows always staged by the computing threads -- the same keys, bit
 * for bit.  A bounded wait of the TMA-fed mode-0 kernel that runs out is
 * reported by the next dci_b200_query_host (DCI_B200_ERR_CUDA).  Rejected
 * while the index holds points (data and queries must be projected the same
 * way). */
int dci_b200_set_projection(dci_b200_t *h, int mode);

/* When enabled, every later query brackets its kernels with CUDA events on the
 * caller's stream and synchronises after each batch (so it is for measurement,
 * not production).  get_timing returns, for the last query, milliseconds spent
 * in [0] query projection, [1] the traversal kernel (all launches), [2] the
 * partition merge, and [3] the number of traversal launches.  The reference
 * has no timers (example.py:74-84 prints wall-clock deltas). */
int dci_b200_enable_timing(dci_b200_t *h, int on);
int dci_b200_get_timing(dci_b200_t *h, float *h_ms);
/* Device time of the kernels of the most recent projection (data or queries) that ran while
 * timing was on, without the host-side set-up before them. */
int dci_b200_last_projection_ms(dci_b200_t *h, float *h_ms);

/* Replaces the merge of MDCI.query (dciknn_cuda/core.py:146-157): merges D
 * per-shard result lists, each [num_queries][k] ascending, into the k smallest
 * per query.  d_ids_in / d_dists_in are [D][num_queries][k] on the current
 * device; id_offsets[s] (host array) is added to the ids of shard s (the
 * reference adds data_per_device * s, core.py:149); ties go to the lower
 * global id, which for sorted shard lists equals the reference's stable sort
 * of the shard-ordered concatenation.  Negative ids (empty slots) stay -1.
 * For k above 1024 every shard list must be sorted ascending by (distance,
 * id) with its empty slots last, as dci_b200_query returns it; the merge then
 * places each entry by binary searches instead of a selection.
 * d_ids_out: [num_queries][k] int64; d_dists_out: [num_queries][k] fp32. */
int dci_b200_merge_shards(const int *d_ids_in, const float *d_dists_in, int num_shards,
                          int num_queries, int k, const long long *id_offsets,
                          long long *d_ids_out, float *d_dists_out, int device, void *stream);

/* The same merge for shard lists in dci_b200_query_packed's form: d_packed_in is
 * [D][num_queries][k] keys with shard-local ids.  k up to 1024. */
int dci_b200_merge_shards_packed(const unsigned long long *d_packed_in, int num_shards, int num_queries,
                                 int k, const long long *id_offsets, long long *d_ids_out,
                                 float *d_dists_out, int device, void *stream);

/* ---- MDCI: one point set sharded over the devices of one process -------------------------------
 * Replaces the MDCI class and its native fan-out (dciknn_cuda/core.py:110-169,
 * _dci_multi_query in src/dci_cuda.cpp:120-134, 182), so that a C or C++ host can run the sharded
 * query without the Python layer.  (dciknn_cuda_b200.MDCI additionally offers one process per
 * GPU over torch.distributed.)
 *
 * create: one index per entry of `devices` (the same device may appear more than once), each with
 * its own directions, as the reference's per-device instances have (core.py:117); seeds may be NULL.
 * dci_b200_mdci_shard returns the index of shard i (owned by the MDCI handle), e.g. for
 * dci_b200_set_proj / dci_b200_get_proj.
 * add (replaces MDCI.add, core.py:121-126): h_data is a HOST array [num_points][dim]; shard i
 * receives rows [i*dpd, (i+1)*dpd), dpd = num_points / D + 1, copies them to its device (the
 * reference's data[a:b].to(device)) and owns that copy.  A trailing shard without rows stays empty.
 * All shards are copied, projected and sorted side by side on their own streams.  Synchronous.
 * query (replaces MDCI.query, core.py:128-157): d_query [num_queries][dim] lives on devices[0] and is
 * ready in `stream` order; it is copied to the other devices (core.py:143), every shard answers
 * every query on its own stream, the lists come back to devices[0] as peer copies of 64-bit
 * (distance, id) keys and are merged there on `stream` (ids offset by dpd * shard, ties to the lower
 * global id: core.py:149-157).  d_ids int64 / d_dists fp32 [num_queries][num_neighbours] on
 * devices[0], -1 / +inf in slots no shard fills.  num_neighbours <= 0 is an error as in the reference
 * (core.py:131-132); num_neighbours up to 1024.  Asynchronous; one call in flight per handle.
 * query_host: the same from and to host arrays.  Synchronous. */
int dci_b200_mdci_create(dci_b200_mdci_t **out, int dim, int num_comp_indices, int num_simp_indices,
                         const int *devices, int num_devices, const unsigned long long *seeds);
int dci_b200_mdci_destroy(dci_b200_mdci_t *m);
int dci_b200_mdci_num_devices(dci_b200_mdci_t *m);
dci_b200_t *dci_b200_mdci_shard(dci_b200_mdci_t *m, int i);
long long dci_b200_mdci_data_per_device(dci_b200_mdci_t *m);
int dci_b200_mdci_add(dci_b200_mdci_t *m, const float *h_data, long long num_points, int block_size,
                      int thread_size);
int dci_b200_mdci_clear(dci_b200_mdci_t *m);
int dci_b200_mdci_query(dci_b200_mdci_t *m, const float *d_query, int num_queries, int num_neighbours,
                        int num_outer_iterations, int max_num_candidates, long long *d_ids,
                        float *d_dists, void *stream);
int dci_b200_mdci_query_host(dci_b200_mdci_t *m, const float *h_query, int num_queries,
                             int num_neighbours, int num_outer_iterations, int max_num_candidates,
                             long long *h_ids, float *h_dists);

/* Query for callers that must not allocate.  (No counterpart in the reference,
 * which allocates and frees managed and device memory inside every query,
 * src/dci_cuda_kernel.cu:792-831, 868-874.)
 *
 * dci_b200_query grows per-handle work buffers with cudaMalloc when a call
 * needs more room than the previous ones did.  Some callers cannot tolerate
 * that: a serving loop with a latency budget (cudaMalloc and cudaFree
 * synchronise the whole device), a process whose device memory is owned
 * entirely by another allocator or is already full, a plugin host that forbids
 * driver allocations after start-up.  This entry point answers the same query,
 * with the same results, and calls no cudaMalloc, cudaFree or other allocating
 * routine: its working memory (projected queries, per-partition result lists,
 * per-CTA slabs) is carved from one fixed array of
 * DCI_B200_NOALLOC_SCRATCH_BYTES bytes that is part of the library image, so
 * every GPU that loads the library holds that much memory until the process
 * exits.  The caller passes the inputs and the outputs exactly as for
 * dci_b200_query (blind querying is not offered).
 *
 * Limits: the query is rejected with DCI_B200_ERR_UNSUPPORTED, and a message
 * that states the need, when the index geometry and k do not fit the array
 * even for a single query (the per-CTA slabs grow with the partition size);
 * larger query batches are processed in as many passes as fit.
 * The first call on a device looks the array's device address up
 * (cudaGetSymbolAddress); make that first call before any stream capture.
 * All calls on a device share the array and it keeps the previous call's
 * contents; nothing in it needs to start at zero.  Two calls that overlap on
 * the GPU (different streams or threads, same device) race on it: serialise
 * them.  Work statistics and timing are not recorded on this path. */
#define DCI_B200_NOALLOC_SCRATCH_BYTES (32u << 20)
int dci_b200_query_noalloc(dci_b200_t *h, const float *d_query, int num_queries, int num_neighbours,
                           int num_outer_iterations, int max_num_candidates, int block_size,
                           int thread_size, int *d_ids, float *d_dists, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DCI_B200_H */
