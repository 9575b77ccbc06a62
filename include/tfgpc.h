/*
 * tfgpc.h -- C ABI of the B200 (sm_100a) implementation of the tfg_custom_ops
 * hot path of schellmi42/tensorflow_graphics_point_clouds.
 *
 * Every entry point takes plain pointers and sizes.  Unless a parameter is
 * marked [host], pointers are device pointers valid on the current CUDA
 * device; `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * Work is enqueued on `stream` and the call returns without synchronising,
 * except for the *_count entry points, which block on the stream once to
 * return a dynamic output size (the reference blocks at the same places:
 * find_neighbors/cc/kernels/scan_alg_kernels.cu.cc:253-265,
 * sampling/cc/kernels/count_sampling_pd_kernels.cu.cc:184-197).
 *
 * Return value: 0 on success, otherwise one of TFGPC_E*; the message of the
 * last failure on the calling thread is returned by tfgpc_last_error().  The
 * library never exits the process (the reference does on CUDA errors,
 * shared/cc/kernels/tf_gpu_device.cpp:89-100) and never allocates device
 * memory: scratch is passed in by the caller as `ws` / `ws_bytes`, sized by
 * the matching *_workspace_bytes() query (the reference takes it from
 * allocate_temp, shared/cc/kernels/tf_gpu_device.cpp:122-142).
 *
 * Index conventions kept from the reference:
 *   - keys are sorted in DESCENDING order (pylib/pc/Grid.py:56-57);
 *   - ranges[s] is the END offset of sample s in the neighbor list (inclusive
 *     prefix sum); its start is ranges[s-1], or 0 for s == 0;
 *   - a neighbor entry is the int pair (point index, sample index).
 * Orders the reference leaves to atomics are fixed here: neighbor lists are
 * ascending in point index within each sample, Poisson samples are ascending
 * in point index, cell-average samples are ascending in first point index.
 */
#ifndef TFGPC_H_
#define TFGPC_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TFGPC_OK 0
#define TFGPC_EINVAL 1   /* bad argument (the reference's InvalidArgument) */
#define TFGPC_ECUDA 2    /* a CUDA call failed */
#define TFGPC_ENOMEM 3   /* workspace too small */
#define TFGPC_ETIMEOUT 4 /* a bounded device-side wait ran out */

#define TFGPC_MIN_DIMS 2 /* shared/cc/kernels/defines.hpp:30-31 */
#define TFGPC_MAX_DIMS 6

/* Message of the last failed call on this thread ("" if none). */
const char* tfgpc_last_error(void);
/* ABI version, bumped when a signature changes. */
int tfgpc_version(void);

/* ---- ComputeKeys ---------------------------------------------------------
 * Replaces ComputeKeysOp::Compute (compute_keys/cc/ops/compute_keys_ops.cpp:
 * 65-117) -> compute_keys_gpu<D> (cc/kernels/compute_keys_kernels.cu.cc:
 * 76-115).  points [n,D] f32, batch_ids [n] i32, scaled_aabb_min [B,D] f32
 * (= aabb_min / cell_size), num_cells [D] i32, inv_cell_sizes [D] f32
 * -> keys [n] i64. */
int tfgpc_compute_keys(void* stream, int D, int64_t n, const float* points,
                       const int32_t* batch_ids, int64_t batch_size,
                       const float* scaled_aabb_min, const int32_t* num_cells,
                       const float* inv_cell_sizes, int64_t* keys_out);

/* ---- per-cloud bounding box ------------------------------------------------
 * Replaces the tf.math.unsorted_segment_min / _max pair of
 * pylib/pc/PointCloud.py:38-43 (the -+1e-9 margins stay with the caller).
 * points [n,D], batch_ids [n] -> aabb_min_out, aabb_max_out [batch_size,D];
 * clouds without points keep +inf / -inf. */
int tfgpc_compute_aabb(void* stream, int D, int64_t n, const float* points,
                       const int32_t* batch_ids, int64_t batch_size,
                       float* aabb_min_out, float* aabb_max_out);

/* ---- key sort + gather ---------------------------------------------------
 * Replaces tf.argsort(keys, 'DESCENDING') and the three tf.gather calls of
 * pylib/pc/Grid.py:56-64.  Stable: equal keys keep the lower original index
 * first.  key_bits = number of low key bits that can be non-zero (0 = 64).
 * perm_out [n] i32, sorted_keys_out [n] i64; sorted_points_out [n,D] and
 * sorted_batch_ids_out [n] may be NULL together to skip the gather. */
size_t tfgpc_sort_keys_workspace_bytes(int64_t n);
int tfgpc_sort_keys_desc(void* stream, int D, int64_t n, int key_bits,
                         const int64_t* keys, const float* points,
                         const int32_t* batch_ids, int32_t* perm_out,
                         int64_t* sorted_keys_out, float* sorted_points_out,
                         int32_t* sorted_batch_ids_out, void* ws,
                         size_t ws_bytes);

/* ---- BuildGridDs ---------------------------------------------------------
 * Replaces BuildGridDsOp::Compute (build_grid_ds/cc/ops/build_grid_ds_ops.cpp:
 * 67-106) -> build_grid_ds_gpu<D> (cc/kernels/build_grid_ds_kernels.cu.cc:
 * 76-114).  sorted_keys [n] i64, num_cells [D] i32 on the device and the same
 * values on the host [host] -> ds [batch_size, num_cells[0], num_cells[1], 2]
 * i32: (first, last+1) index of each (batch, c0, c1) tube, (0,0) if empty. */
int tfgpc_build_grid_ds(void* stream, int D, int64_t n,
                        const int64_t* sorted_keys, const int32_t* num_cells,
                        const int32_t* num_cells_host, int64_t batch_size,
                        int32_t* ds_out);

/* ---- FindNeighbors -------------------------------------------------------
 * Replaces FindNeighborsOp::Compute (find_neighbors/cc/ops/
 * find_neighbors_ops.cpp:86-250) and the kernels it drives
 * (find_ranges_grid_ds, count_neighbors, scan_alg, elem_wise_min,
 * store_neighbors).  Two calls, so that the caller owns the dynamic output:
 *   _count writes ranges_out [ns] i32 (end offsets), blocks on the stream and
 *          returns the number of pairs M in *total_out [host];
 *   _fill  writes neigh_out [M,2] i32 in canonical order.
 * samples [ns,D], samples_batch_ids [ns], points [n,D] (sorted), point_keys
 * [n] (sorted, descending), ds [batch_size,C0,C1,2], num_cells [D],
 * scaled_aabb_min [batch_size,D], inv_cell_sizes [D], inv_radii [D].
 * max_neighs > 0 keeps the first max_neighs neighbors in canonical order (the
 * reference keeps a time-seeded random subset,
 * store_neighbors_kernels.cu.cc:51-112,216). */
size_t tfgpc_find_neighbors_workspace_bytes(int64_t ns);
int tfgpc_find_neighbors_count(void* stream, int D, int64_t ns,
                               const float* samples,
                               const int32_t* samples_batch_ids, int64_t n,
                               const float* points, const int64_t* point_keys,
                               const int32_t* ds, int64_t batch_size,
                               const int32_t* num_cells,
                               const float* scaled_aabb_min,
                               const float* inv_cell_sizes,
                               const float* inv_radii, int max_neighs,
                               int32_t* ranges_out, void* ws, size_t ws_bytes,
                               int64_t* total_out);
int tfgpc_find_neighbors_fill(void* stream, int D, int64_t ns,
                              const float* samples,
                              const int32_t* samples_batch_ids, int64_t n,
                              const float* points, const int64_t* point_keys,
                              const int32_t* ds, int64_t batch_size,
                              const int32_t* num_cells,
                              const float* scaled_aabb_min,
                              const float* inv_cell_sizes,
                              const float* inv_radii, int max_neighs,
                              const int32_t* ranges, int64_t total,
                              int32_t* neigh_out);

/* The same two calls with a visiting order: sample_order [ns] is a permutation
 * of 0..ns-1, and the samples are worked on in that sequence.  The results are
 * the same as without it (ranges and lists stay indexed by the sample's own
 * position); an order that keeps spatial neighbors together (for samples that
 * are the grid's own points: the permutation the key sort returns) makes
 * consecutive warps read the same cells.  No counterpart in the reference. */
int tfgpc_find_neighbors_count_ordered(
    void* stream, int D, int64_t ns, const float* samples,
    const int32_t* samples_batch_ids, const int32_t* sample_order, int64_t n,
    const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells, const float* scaled_aabb_min,
    const float* inv_cell_sizes, const float* inv_radii, int max_neighs,
    int32_t* ranges_out, void* ws, size_t ws_bytes, int64_t* total_out);
int tfgpc_find_neighbors_fill_ordered(
    void* stream, int D, int64_t ns, const float* samples,
    const int32_t* samples_batch_ids, const int32_t* sample_order, int64_t n,
    const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells, const float* scaled_aabb_min,
    const float* inv_cell_sizes, const float* inv_radii, int max_neighs,
    const int32_t* ranges, int64_t total, int32_t* neigh_out);

/* Neighbor ids in the unsorted point order: ids_out[m] = (sorted_indices[
 * neighbors[m].x], neighbors[m].y), the gather + concat of
 * pylib/pc/Neighborhood.py:246-250; optionally also the per-pair density
 * pdf_out[m] = pdf_by_original[that original id] (:287).  Pass both density
 * pointers or neither. */
int tfgpc_original_neighbor_ids(void* stream, int64_t M,
                                const int32_t* neighbors, int64_t n,
                                const int32_t* sorted_indices,
                                const float* pdf_by_original, int32_t* ids_out,
                                float* pdf_out);

/* ---- Grid and neighbor count in one call ------------------------------------
 * Replaces, for one cloud and one neighborhood on it, the chain PointCloud.
 * get_AABB (pylib/pc/PointCloud.py:38-43) -> Grid (Grid.py:32-83: cell counts,
 * ComputeKeys, argsort + gathers, BuildGridDs) -> first half of Neighborhood
 * (Neighborhood.py:218-245: FindNeighbors up to the number of pairs), which in
 * pylib -- and through the separate entries above -- reads the cell counts back
 * to the host before it can size the tube array and once more for the number of
 * pairs.  Here the cell counts stay on the device; the tube array and the key
 * width of the sort are sized for max_cells cells per dimension (a bound the
 * caller chooses, e.g. what the previous batch needed); ONE blocking read at the
 * end returns the cell counts, whether they fit, and the number of pairs.
 * cell_sizes, radii [D] are HOST arrays.  Samples: samples_are_points 0 = the
 * given samples / samples_batch_ids [ns]; 1 = the points themselves in their own
 * order (ns == n; they are visited in the sequence of the key sort); 2 = the
 * sorted points (a self neighborhood, Neighborhood.py:229-233).
 * Outputs [device, caller-allocated]: aabb_min/max [B,D] (already widened by
 * 1e-9), num_cells [D], scaled_aabb_min [B,D], inv_cell_sizes, inv_radii [D],
 * keys [n], sorted_indices [n], sorted_keys [n], sorted_points [n,D],
 * sorted_batch_ids [n], ds [_ds_elems(D, B, max_cells)] int32 (the tubes fill
 * the first B * num_cells[0] * num_cells[1] pairs; pass it to the fill entries
 * as it is), ranges [ns]; [host] num_cells_host_out [D], total_out.  Returns
 * TFGPC_ENOMEM (and the cell counts the grid asked for) if max_cells was too
 * small: repeat with a larger bound.  Follow with one of the
 * tfgpc_find_neighbors_fill* entries.
 * A cloud that is one shard of a batch held by several processes needs the cell
 * counts of the whole batch (Grid.py:44-48: the maximum over all clouds):
 * tfgpc_grid_cells computes the boxes, this shard's counts and the scaled minima
 * / inverse sizes WITHOUT blocking; the caller reduces num_cells over the
 * processes on the same stream (a max all-reduce) and passes the result as
 * num_cells_in [D, device] together with the arrays tfgpc_grid_cells wrote
 * (aabb_*_out, scaled_aabb_min_out, inv_*_out are then inputs).  num_cells_in
 * NULL: the entry computes all of that itself.  num_cells_in is not modified
 * and must not alias num_cells_out, which receives the counts in use. */
size_t tfgpc_grid_neighborhood_workspace_bytes(int64_t n, int64_t ns);
size_t tfgpc_grid_neighborhood_ds_elems(int D, int64_t batch_size,
                                        int max_cells);
int tfgpc_grid_cells(void* stream, int D, int64_t n, const float* points,
                     const int32_t* batch_ids, int64_t batch_size,
                     const float* cell_sizes, const float* radii,
                     float* aabb_min_out, float* aabb_max_out,
                     int32_t* num_cells_out, float* scaled_aabb_min_out,
                     float* inv_cell_sizes_out, float* inv_radii_out);
int tfgpc_grid_neighborhood_count(
    void* stream, int D, int64_t n, const float* points,
    const int32_t* batch_ids, int64_t batch_size, const float* cell_sizes,
    const float* radii, int max_cells, const int32_t* num_cells_in,
    int64_t ns, const float* samples,
    const int32_t* samples_batch_ids, int samples_are_points, int max_neighs,
    float* aabb_min_out, float* aabb_max_out, int32_t* num_cells_out,
    float* scaled_aabb_min_out, float* inv_cell_sizes_out,
    float* inv_radii_out, int64_t* keys_out, int32_t* sorted_indices_out,
    int64_t* sorted_keys_out, float* sorted_points_out,
    int32_t* sorted_batch_ids_out, int32_t* ds_out, int32_t* ranges_out,
    void* ws, size_t ws_bytes, int32_t* num_cells_host_out,
    int64_t* total_out);

/* ---- FindNeighbors fill pass with original ids and densities --------------
 * tfgpc_find_neighbors_fill_ordered (sample_order may be NULL) that, in the same
 * pass, also writes what pylib computes from the neighbor list afterwards:
 * ids_out [M,2] = (sorted_indices[neighbors[m].x], neighbors[m].y), the pairs
 * with the neighbor's index in the unsorted point order (pylib/pc/
 * Neighborhood.py:246-250), and sample_pdf_out [ns], ComputePdf
 * (compute_pdf_kernels.cu.cc:107-128) at every sample over its neighbors
 * (inv_bandwidth [D], pdf_mode 0 / 1 as in tfgpc_compute_pdf, mode 1 with the
 * number of points n).  For samples that are the grid's own points this is the
 * density of tfgpc_compute_pdf_at_samples without walking the lists again;
 * sample_pdf_out may be NULL (ids only), which is the cheaper combination: the
 * densities take less time in a pass of their own over the finished lists. */
int tfgpc_find_neighbors_fill_fused(
    void* stream, int D, int64_t ns, const float* samples,
    const int32_t* samples_batch_ids, const int32_t* sample_order, int64_t n,
    const float* points, const int64_t* point_keys, const int32_t* ds,
    int64_t batch_size, const int32_t* num_cells,
    const float* scaled_aabb_min, const float* inv_cell_sizes,
    const float* inv_radii, int max_neighs, const int32_t* ranges,
    int64_t total, const int32_t* sorted_indices, const float* inv_bandwidth,
    int pdf_mode, int32_t* neigh_out, int32_t* ids_out,
    float* sample_pdf_out);

/* ---- FindNeighbors count pass with built-in scratch ------------------------
 * No counterpart in the reference.  Same inputs, outputs and blocking
 * behaviour as tfgpc_find_neighbors_count, but without the ws / ws_bytes
 * pair: the scan's scratch is a fixed array inside the library image, and the
 * call makes no cudaMalloc / cudaFree and uses no allocating routine.  It is
 * meant for hosts that cannot get temporary device memory at the point where
 * the neighbor count is needed -- e.g. a plugin whose framework owns all
 * device memory and only lends buffers for declared outputs, or a service that
 * has already committed its whole memory budget and must not trigger a device
 * allocation (with its implicit synchronisation) on the request path.
 * Limits: at most tfgpc_find_neighbors_static_max_samples() (2^24) samples per
 * call, larger ns is rejected with TFGPC_EINVAL; the array (about 33 KB) stays
 * resident on every GPU that loads the library until the process exits.
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) with that device current, and, like the first launch
 * of any kernel, makes the CUDA runtime load the kernels' code onto the device
 * (which the runtime may back with memory of its own and a synchronisation):
 * make that first call as a warm-up, outside of any stream capture and off the
 * request path.  The address is cached per device for the life of the process
 * and does not survive a cudaDeviceReset.  Per-launch timing
 * (tfgpc_profile_enable) is suspended inside this call, since it would create
 * CUDA events.  All calls on a device share the one array,
 * which keeps the previous call's contents (nothing in it needs clearing: each
 * call overwrites what it reads); two calls whose GPU work overlaps -- from
 * different streams or threads -- race on it, so serialise them. */
int64_t tfgpc_find_neighbors_static_max_samples(void);
int tfgpc_find_neighbors_count_static(void* stream, int D, int64_t ns,
                                      const float* samples,
                                      const int32_t* samples_batch_ids,
                                      int64_t n, const float* points,
                                      const int64_t* point_keys,
                                      const int32_t* ds, int64_t batch_size,
                                      const int32_t* num_cells,
                                      const float* scaled_aabb_min,
                                      const float* inv_cell_sizes,
                                      const float* inv_radii, int max_neighs,
                                      int32_t* ranges_out, int64_t* total_out);

/* ---- ComputePdf / ComputePdfWithPtGrads / ComputePdfPtGrads --------------
 * Replaces ComputePDFOp::Compute (compute_pdf/cc/ops/compute_pdf_ops.cpp:
 * 101-154) -> compute_pdf_gpu<D> (cc/kernels/compute_pdf_kernels.cu.cc:
 * 220-272) and ComputePDFPtGradsOp::Compute (:188-246) ->
 * compute_pdf_grads_gpu<D> (:275-335).  points [n,D], neighbors [M,2],
 * ranges [n], inv_bandwidth [D], inv_radii [D]; mode 0 = constant bandwidth,
 * 1 = sqrt(n) as inverse bandwidth.  pt_grads_out [n,D] is overwritten. */
int tfgpc_compute_pdf(void* stream, int D, int mode, int64_t n,
                      const float* points, const int32_t* neighbors, int64_t M,
                      const int32_t* ranges, const float* inv_bandwidth,
                      const float* inv_radii, float* pdf_out);
int tfgpc_compute_pdf_pt_grads(void* stream, int D, int mode, int64_t n,
                               const float* points, const int32_t* neighbors,
                               int64_t M, const int32_t* ranges,
                               const float* inv_bandwidth,
                               const float* inv_radii, const float* pdf_grads,
                               float* pt_grads_out);

/* Density at arbitrary sample positions: the same sum as tfgpc_compute_pdf but
 * centred on samples [ns,D] whose neighbor lists (neighbors [M,2], ranges
 * [ns]) index points [n,D]; mode 1 uses sqrt(n).  When the samples are the
 * grid's own points in another order this equals ComputePdf on the self
 * neighborhood, so MCConv on one cloud needs a single neighbor search where
 * pylib builds a second one (pylib/pc/Neighborhood.py:284). */
int tfgpc_compute_pdf_at_samples(void* stream, int D, int mode, int64_t ns,
                                 const float* samples, int64_t n,
                                 const float* points, const int32_t* neighbors,
                                 int64_t M, const int32_t* ranges,
                                 const float* inv_bandwidth,
                                 const float* inv_radii, float* pdf_out);

/* ---- BasisProj / BasisProjGrads ------------------------------------------
 * Replaces BasisProjOp::Compute (basis_proj/cc/ops/basis_proj_ops.cpp:77-132)
 * -> basis_proj_gpu<K> (cc/kernels/basis_proj_kernels.cu.cc:132-182) and
 * BasisProjGradsOp::Compute (:156-222) -> basis_proj_grads_gpu<K>
 * (cc/kernels/basis_proj_grads_kernels.cu.cc:157-211).
 * basis [M,K] (K in 8,16,32,64), features [n_in,C] (C < 8 or C % 8 == 0),
 * neighbors [M,2] (point index into features, sample index), ranges [ns]
 * -> out [ns,C,K].  Grads: in_grads [ns,C,K] -> dbasis_out [M,K],
 * dfeat_out [n_in,C] (both overwritten). */
int tfgpc_basis_proj(void* stream, int K, int C, int64_t ns, int64_t n_in,
                     int64_t M, const float* basis, const float* features,
                     const int32_t* neighbors, const int32_t* ranges,
                     float* out);
int tfgpc_basis_proj_grads(void* stream, int K, int C, int64_t ns,
                           int64_t n_in, int64_t M, const float* basis,
                           const float* features, const int32_t* neighbors,
                           const int32_t* ranges, const float* in_grads,
                           float* dbasis_out, float* dfeat_out);
/* The same two ops with caller scratch (what the reference takes from
 * IGPUDevice::getFloatTmpGPUBuffer, tf_gpu_device.cpp:122-142): for K in
 * {16, 32, 64} and C a multiple of 16 they run on tensor-core MMAs over a bf16
 * hi/mid copy of the features written into `ws` (three bf16 passes, fp32
 * accumulate: results within 1e-4 of the fp32 kernels).  The query returns 0
 * for shapes without such a path; with ws == NULL, too little scratch or a
 * shape without it, the calls fall through to the entries above. */
size_t tfgpc_basis_proj_workspace_bytes(int K, int C, int64_t n_in);
int tfgpc_basis_proj_ws(void* stream, int K, int C, int64_t ns, int64_t n_in,
                        int64_t M, const float* basis, const float* features,
                        const int32_t* neighbors, const int32_t* ranges,
                        float* out, void* ws, size_t ws_bytes);
int tfgpc_basis_proj_grads_ws(void* stream, int K, int C, int64_t ns,
                              int64_t n_in, int64_t M, const float* basis,
                              const float* features, const int32_t* neighbors,
                              const int32_t* ranges, const float* in_grads,
                              float* dbasis_out, float* dfeat_out, void* ws,
                              size_t ws_bytes);

/* ---- Sampling ------------------------------------------------------------
 * Replaces SamplingOp::Compute (sampling/cc/ops/sampling_ops.cpp:81-195) and
 * its kernels (count_unique_keys, store_unique_keys, count_sampling_pd,
 * store_sampled_pts, sampling_avg).  mode 0 = Poisson disk, 1 = cell average
 * (sampling_ops.cpp:141,174).  Two calls:
 *   _count selects (state kept in ws), blocks on the stream and returns the
 *          number of samples S in *num_samples_out [host];
 *   _store writes sample_pts_out [S,D], sample_batch_ids_out [S] and, for
 *          mode 0, sample_indices_out [S] (mode 1: not written, may be NULL;
 *          the reference leaves its [1] tensor unwritten too).
 * points [n,D], batch_ids [n], point_keys [n] (all sorted), num_cells [D],
 * neighbors [M,2] and ranges [n] of the self neighborhood.  The same ws must
 * be passed to both calls with nothing else written to it in between. */
size_t tfgpc_sampling_workspace_bytes(int64_t n);
int tfgpc_sampling_count(void* stream, int D, int mode, int64_t n,
                         const float* points, const int32_t* batch_ids,
                         const int64_t* point_keys, const int32_t* num_cells,
                         const int32_t* neighbors, int64_t M,
                         const int32_t* ranges, void* ws, size_t ws_bytes,
                         int64_t* num_samples_out);
/* tfgpc_sampling_count for SYMMETRIC neighbor lists: point j is listed for
 * point i exactly when i is listed for j, which holds for every self
 * neighborhood that tfgpc_find_neighbors_* builds with max_neighs = 0 (the
 * only input pylib/pc/sampling.py:123-150 and PointHierarchy.py:83-93 give
 * the op).  Same arguments and same result; the Poisson passes then walk only
 * the lists of the points they take.  With lists that are not symmetric the
 * selection differs from the reference's and may vary from run to run. */
int tfgpc_sampling_count_symmetric(void* stream, int D, int mode, int64_t n,
                                   const float* points,
                                   const int32_t* batch_ids,
                                   const int64_t* point_keys,
                                   const int32_t* num_cells,
                                   const int32_t* neighbors, int64_t M,
                                   const int32_t* ranges, void* ws,
                                   size_t ws_bytes, int64_t* num_samples_out);
int tfgpc_sampling_store(void* stream, int D, int mode, int64_t n,
                         const float* points, const int32_t* batch_ids,
                         const int64_t* point_keys, const int32_t* num_cells,
                         int64_t num_samples, void* ws, size_t ws_bytes,
                         float* sample_pts_out, int32_t* sample_batch_ids_out,
                         int32_t* sample_indices_out);

/* ---- MCConv: basis projection fused with the weight GEMMs ----------------
 * Replaces the BasisProj -> tf.matmul pair of pylib/pc/layers/MCConv.py:
 * 174-191 (forward) and what TensorFlow's autodiff makes of it (matmul
 * gradients + BasisProjGrads, custom_ops_wrapper.py:192-198) without writing
 * the fp32 [ns, C, K] tensor: the projection is produced as the bf16 operand
 * pair of a tcgen05 tensor-core GEMM (three bf16 passes, fp32 accumulate).
 * weights [C*K, Cout] row-major in the projection's own reduction order
 * (row c*K + k; for num_mlps == 1 this is MCConv's final weight matrix as
 * stored), out [ns, Cout].  Cout must be a multiple of 8
 * (16-byte rows of the bf16 weight operand).
 * Backward: out_grads [ns, Cout] -> dbasis_out [M, K], dfeat_out [n_in, C],
 * dweights_out [C*K, Cout] (all overwritten).  x_in_workspace != 0 tells it
 * that `ws` still holds the projection written by the forward call for the
 * same inputs (ws sized for backward); otherwise it is recomputed.  The
 * weights are read from `weights` on every call, never from what an earlier call
 * left in `ws`.  The status word of `ws` is cleared by the forward call and by a
 * backward call that recomputes the projection; a backward call that reuses it
 * keeps the forward call's word (a timeout there invalidates what it reads).  The
 * workspace size depends on n_in as well: for K in {16, 32, 64} and C a multiple
 * of 16 the projection and its gradients run on warp-level tensor-core MMAs
 * over a bf16 hi/mid copy of the features kept in the workspace.
 * tfgpc_mcconv_status blocks on the stream and returns TFGPC_ETIMEOUT if a
 * bounded wait inside one of the GEMM kernels that used `ws` ran out. */
size_t tfgpc_mcconv_workspace_bytes(int K, int C, int Cout, int64_t ns,
                                    int64_t n_in, int backward);
int tfgpc_mcconv_forward(void* stream, int K, int C, int Cout, int64_t ns,
                         int64_t n_in, int64_t M, const float* basis,
                         const float* features, const int32_t* neighbors,
                         const int32_t* ranges, const float* weights,
                         float* out, void* ws, size_t ws_bytes);
int tfgpc_mcconv_backward(void* stream, int K, int C, int Cout, int64_t ns,
                          int64_t n_in, int64_t M, const float* basis,
                          const float* features, const int32_t* neighbors,
                          const int32_t* ranges, const float* weights,
                          const float* out_grads, int x_in_workspace,
                          float* dbasis_out, float* dfeat_out,
                          float* dweights_out, void* ws, size_t ws_bytes);
int tfgpc_mcconv_status(void* stream, const void* ws, int* status_out);

/* ---- MCConv forward and backward on a group plan -------------------------
 * No counterpart in the reference; same results as tfgpc_mcconv_forward /
 * _backward.  BasisProj and BasisProjGrads (basis_proj_kernels.cu.cc:30-127,
 * basis_proj_grads_kernels.cu.cc:30-151) spend one gathered feature row -- and
 * the gradients one C-wide atomic update -- per neighbor PAIR.  Samples that lie
 * close together share most of their neighbors, so the work is regrouped: the
 * samples are taken four at a time in a spatially coherent visiting order
 * `order` [ns] (a permutation of the sample indices; for a cloud searched on its
 * own grid the key sort's permutation), and the plan lists every group's
 * distinct neighbors with the pairs through which its samples see them.  The
 * kernels then gather, multiply and reduce once per distinct neighbor of a
 * group (about half as often as per pair at 32 neighbors per point).
 * tfgpc_mcconv_group_plan: ranges [ns] and neighbors_sorted [M,2] as written by
 * FindNeighbors (ids ascending within each sample's list -- required),
 * neighbor_ids [M,2] the ids the features are indexed by (the original ids of
 * tfgpc_original_neighbor_ids; may equal neighbors_sorted).  plan: caller
 * buffer of _group_plan_bytes(ns, M) bytes, 256-byte aligned; it depends only on
 * the neighborhood and the order and can be reused by every call on them.
 * _forward_grouped / _backward_grouped: arguments of tfgpc_mcconv_forward /
 * _backward with the basis given as basis_pair [M,2,K] bf16
 * (tfgpc_kernel_basis_split; 32-byte aligned) instead of fp32, plus order and
 * plan; the neighbor list itself is not needed any more.  The projection is kept
 * in the workspace in the visiting order: x_in_workspace != 0 is only valid
 * after _forward_grouped on the same workspace, order and plan.  Only for shapes
 * with _grouped_supported(K, C) != 0 (K = 16, C = 128) and Cout >= 128;
 * 16-byte aligned features, 32-byte aligned out. */
int tfgpc_mcconv_grouped_supported(int K, int C);
size_t tfgpc_mcconv_group_plan_bytes(int64_t ns, int64_t M);
int tfgpc_mcconv_group_plan(void* stream, int64_t ns, int64_t M,
                            const int32_t* order, const int32_t* ranges,
                            const int32_t* neighbors_sorted,
                            const int32_t* neighbor_ids, void* plan,
                            size_t plan_bytes);
int tfgpc_mcconv_forward_grouped(void* stream, int K, int C, int Cout,
                                 int64_t ns, int64_t n_in, int64_t M,
                                 const void* basis_pair, const float* features,
                                 const float* weights, const int32_t* order,
                                 const void* plan, float* out, void* ws,
                                 size_t ws_bytes);
int tfgpc_mcconv_backward_grouped(void* stream, int K, int C, int Cout,
                                  int64_t ns, int64_t n_in, int64_t M,
                                  const void* basis_pair,
                                  const float* features, const int32_t* ranges,
                                  const float* weights,
                                  const float* out_grads, int x_in_workspace,
                                  const int32_t* order, const void* plan,
                                  float* dbasis_out, float* dfeat_out,
                                  float* dweights_out, void* ws,
                                  size_t ws_bytes);

/* ---- MCConv kernel basis --------------------------------------------------
 * Replaces the TensorFlow op chain of pylib/pc/layers/MCConv.py:264-269 and
 * :163-171 for a kernel MLP with one hidden layer: per neighbor pair
 *   diff = (points_in[nbr.x] - points_out[nbr.y]) * inv_radius
 *   basis[m, k] = act(diff . w1[:, k] + b1[k]) / pdf[m]
 * points_in [n_in,D], points_out [ns,D], neighbors [M,2] (point index into
 * points_in, sample index into points_out), pdf [M] (density per pair), w1
 * [D,K] row-major (column k = mlp * hidden + h of the reference's
 * [num_mlps, D, hidden] weights), b1 [K].  activation 0 = leaky ReLU with slope
 * alpha (0.2 is tf.nn.leaky_relu's default, 0 gives ReLU), 1 = ELU.
 * pdf_by_neighbor != 0: pdf is not the per-pair array but a table with one
 * density per point of points_in, read at nbr.x (what pylib gathers into the
 * per-pair array at Neighborhood.py:287); the same flag on every entry below.
 * pdf_by_neighbor == 2 (these three entries, D == 3): points_in is the packed
 * table of tfgpc_pack_points_density, [n_in,4] = (x, y, z, 1 / density),
 * 16-byte aligned, and pdf is not read (may be NULL): one 16-byte gather per
 * pair instead of four scattered loads; same results, bit for bit.
 * _grads: basis_grads [M,K] -> dw1_out [D,K], db1_out [K] (overwritten). */
int tfgpc_pack_points_density(void* stream, int64_t n, const float* points,
                              const float* pdf, float* packed_out);
int tfgpc_kernel_basis(void* stream, int D, int K, int64_t M,
                       const float* points_in, const float* points_out,
                       const int32_t* neighbors, const float* pdf,
                       const float* w1, const float* b1, float inv_radius,
                       int activation, float alpha, int pdf_by_neighbor,
                       float* basis_out);
int tfgpc_kernel_basis_grads(void* stream, int D, int K, int64_t M,
                             const float* points_in, const float* points_out,
                             const int32_t* neighbors, const float* pdf,
                             const float* w1, const float* b1, float inv_radius,
                             int activation, float alpha, int pdf_by_neighbor,
                             const float* basis_grads, float* dw1_out,
                             float* db1_out);
/* tfgpc_kernel_basis that also writes every basis row as the bf16 pair the
 * tensor-core kernels multiply with: basis_pair_out [M,2,K] bf16 (32-byte
 * aligned), row m = (hi terms k = 0..K-1, mid terms), basis ~= hi + mid.
 * basis_out may be NULL (only the pair is written). */
int tfgpc_kernel_basis_split(void* stream, int D, int K, int64_t M,
                             const float* points_in, const float* points_out,
                             const int32_t* neighbors, const float* pdf,
                             const float* w1, const float* b1,
                             float inv_radius, int activation, float alpha,
                             int pdf_by_neighbor, float* basis_out,
                             void* basis_pair_out);

/* ---- MCConv kernel MLP, general form ---------------------------------------
 * Replaces the TensorFlow ops of pylib/pc/layers/MCConv.py:163-171 and :264-269
 * and what autodiff makes of them, for kernel MLPs with any number of hidden
 * layers (the loop of MCConv.py:165-168), including the gradients with respect
 * to the point coordinates that monte_carlo_conv_test.py:182-219 checks.
 * num_mlps independent MLPs; layer l of each maps H_{l-1} values (H_0 = D) to
 * layer_sizes[l-1] = H_l values [host, num_layers <= 4 entries, each <= 64] and
 * is followed by the activation (0 = leaky ReLU with slope alpha, 1 = ELU).
 * weights: the layers' tensors [num_mlps, H_{l-1}, H_l] one after the other;
 * biases: [num_mlps, H_l] per layer, one after the other (at most 8192 floats in
 * all).  basis_out [M, num_mlps * H_last], column g * H_last + h, divided by
 * pdf [M].
 * _grads: basis_grads [M, num_mlps * H_last] -> dweights_out / dbiases_out in
 * the layouts of weights / biases (overwritten); optional (NULL to skip)
 * dpoints_in_out [n_in, D], dpoints_out_out [ns, D] (overwritten; the two may
 * be the SAME array when points_in and points_out are one cloud) and dpdf_out
 * [M], the gradient with respect to the per-pair density. */
int tfgpc_kernel_mlp_basis(void* stream, int D, int num_mlps, int num_layers,
                           const int32_t* layer_sizes, int64_t M,
                           const float* points_in, const float* points_out,
                           const int32_t* neighbors, const float* pdf,
                           const float* weights, const float* biases,
                           float inv_radius, int activation, float alpha,
                           int pdf_by_neighbor, float* basis_out);
int tfgpc_kernel_mlp_grads(void* stream, int D, int num_mlps, int num_layers,
                           const int32_t* layer_sizes, int64_t M, int64_t n_in,
                           int64_t ns, const float* points_in,
                           const float* points_out, const int32_t* neighbors,
                           const float* pdf, const float* weights,
                           const float* biases, float inv_radius,
                           int activation, float alpha, int pdf_by_neighbor,
                           const float* basis_grads, float* dweights_out,
                           float* dbiases_out, float* dpoints_in_out,
                           float* dpoints_out_out, float* dpdf_out);

/* ---- KPConv and PointConv bases --------------------------------------------
 * The per-pair basis values of the other two convolutions of pylib/pc/layers,
 * which feed the same BasisProj (+ weight product) as the MCConv basis.
 *
 * tfgpc_kp_basis replaces the op chain of KPConv.py:194-212 (rigid kernel
 * points): diff as above, basis[m, k] = weighting(|diff - kernel_points[k]|,
 * sigma) for k < num_kernel_points and 0 for the padding columns up to K
 * (the tf.pad of KPConv.py:199-212).  interpolation 0 = linear,
 * max(0, 1 - dist / sigma) (KPConv.py:28-40); 1 = gaussian,
 * exp(-(dist / (sigma / 3))^2) (:43-56).  kernel_points [num_kernel_points, D]
 * as the layer holds them (already scaled by 0.75, KPConv.py:129).
 *
 * tfgpc_pointconv_pdf replaces PointConv.py:168-183: per sample the largest
 * density among its pairs (pairs of sample s end at ranges[s]), then per pair
 * out[m] = relu(pdf[m] / max * w1 + b1) . w2 + b2 with w1, b1, w2 [16], b2 [1].
 * The PointConv basis is then tfgpc_kernel_basis with inv_radius 1, pdf_out as
 * its density and the layer's non-linearity (PointConv.py:160-166, 186). */
int tfgpc_kp_basis(void* stream, int D, int K, int num_kernel_points, int64_t M,
                   const float* points_in, const float* points_out,
                   const int32_t* neighbors, const float* kernel_points,
                   float inv_radius, float sigma, int interpolation,
                   float* basis_out);
int tfgpc_pointconv_pdf(void* stream, int64_t ns, int64_t M,
                        const int32_t* ranges, const float* pdf,
                        const float* w1, const float* b1, const float* w2,
                        const float* b2, float* pdf_out);

/* ---- pooling and the bias of Conv1x1 ----------------------------------------
 * tfgpc_neighborhood_pool replaces the gather + unsorted_segment_max / _mean
 * of pylib/pc/layers/Pooling.py:148-162 (MaxPooling, AveragePooling):
 * out[s, c] = max or mean over the pairs of sample s of features[nbr.x, c];
 * features [n_in,C], neighbors [M,2], ranges [ns] (end offsets), out [ns,C].
 * tfgpc_global_pool replaces the segment ops over the batch ids of
 * Pooling.py:51-57 (GlobalMaxPooling) and :90-96 (GlobalAveragePooling):
 * features [n,C], batch_ids [n], out [batch_size,C].  mode 0 = max, 1 = mean;
 * an empty segment gives the lowest float (max), as TensorFlow does, or 0 (mean).
 * tfgpc_add_bias adds bias [C] to every row of x [n,C] in place: with
 * tfgpc_matmul_f32 it is Conv1x1.py:97. */
int tfgpc_neighborhood_pool(void* stream, int mode, int C, int64_t ns,
                            int64_t n_in, int64_t M, const float* features,
                            const int32_t* neighbors, const int32_t* ranges,
                            float* out);
size_t tfgpc_global_pool_workspace_bytes(int64_t batch_size);
int tfgpc_global_pool(void* stream, int mode, int C, int64_t n,
                      int64_t batch_size, const float* features,
                      const int32_t* batch_ids, float* out, void* ws,
                      size_t ws_bytes);
int tfgpc_add_bias(void* stream, int64_t n, int C, float* x, const float* bias);
/* x = act(x * scale + bias) in place, x [n,C], bias [C] or NULL: a batch
 * normalisation in inference mode (its stored statistics folded into scale and
 * bias) followed by the activation, as between the layers of
 * modelnet40_small.py:236-243.  activation 0 = none, 1 = leaky ReLU with slope
 * alpha (tf.keras.layers.LeakyReLU's default is 0.3). */
int tfgpc_scale_bias_activation(void* stream, int64_t n, int C, float* x,
                                float scale, const float* bias, int activation,
                                float alpha);

/* ---- fp32 matrix product on the tensor cores -----------------------------
 * c[M,N] = op(a) * op(b) in fp32 accuracy (three bf16 passes), the tf.matmul
 * of MCConv.py:187-191 as a stand-alone call.  a is [M,K] row-major, or
 * [K,M] if a_transposed; b is [K,N] row-major, or [N,K] if b_transposed.
 * Row lengths must be multiples of 8.  The first int of ws is the same
 * time-out flag that tfgpc_mcconv_status reads. */
size_t tfgpc_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K);
int tfgpc_matmul_f32(void* stream, int64_t M, int64_t N, int64_t K,
                     const float* a, int a_transposed, const float* b,
                     int b_transposed, float* c, void* ws, size_t ws_bytes);

/* ---- bounded-wait self test -------------------------------------------------
 * No counterpart in the reference (its kernels have no device-side waits).
 * Every device-side wait of the tensor-core kernels (mbarrier phases of the
 * GEMMs and of the gradient kernel) gives up after a time limit, records that
 * in the first int of the workspace and lets the kernel drain and return.  This
 * entry makes that happen on purpose without disturbing anything: one warp
 * waits, through the same wait routine, for a barrier phase that nothing
 * completes, with a limit of limit_us microseconds (1 .. 100000).  It blocks on
 * the stream; *returned_out [host] is 1 if the kernel ran to its end.
 * Afterwards tfgpc_mcconv_status(stream, ws, ..) reports TFGPC_ETIMEOUT until
 * the next GEMM call on `ws` clears the word.  ws: any workspace of the GEMM
 * entries (256-byte aligned, at least 1024 bytes). */
int tfgpc_debug_bounded_wait(void* stream, void* ws, size_t ws_bytes,
                             unsigned limit_us, int* returned_out);

/* ---- small blocking reads -------------------------------------------------
 * No counterpart in the reference (it reads its counts with cudaMemcpy behind
 * cudaEventSynchronize, scan_alg_kernels.cu.cc:259-265).  Copies `bytes`
 * (4 .. 4096, a multiple of 4) from device memory to host_dst [host] and
 * blocks on the stream.  The values travel through a page of mapped pinned
 * host memory written by a kernel, not through a copy engine, so the read
 * does not queue behind bulk transfers that other streams have in flight.
 * The blocking entries (tfgpc_find_neighbors_count, tfgpc_sampling_count,
 * tfgpc_mcconv_status) read their results the same way; the first such call
 * of a host thread on a device allocates that page (4 KB) and keeps it.
 * tfgpc_find_neighbors_count_static allocates nothing and uses cudaMemcpy. */
int tfgpc_read_device(void* stream, const void* device_src, size_t bytes,
                      void* host_dst);

/* ---- per-launch timing ---------------------------------------------------
 * No counterpart in the reference (its DEBUG_INFO timing blocks do not
 * compile, store_neighbors_kernels.cu.cc:256-269).  While enabled on the
 * calling thread, every kernel launch group of the library is bracketed by
 * two CUDA events on its stream; _collect waits for them and returns up to
 * max_records durations in milliseconds [host] with the matching names joined
 * by newlines in names_out [host], then clears the records. */
int tfgpc_profile_enable(int on);
int tfgpc_profile_collect(char* names_out, size_t names_bytes, float* ms_out,
                          int max_records, int* count_out);

#ifdef __cplusplus
}
#endif
#endif /* TFGPC_H_ */
