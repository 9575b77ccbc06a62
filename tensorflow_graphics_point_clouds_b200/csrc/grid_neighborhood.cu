// Grid and neighbor count in one call.
//
// pylib builds a Grid (bounding boxes, cell counts, keys, key sort, sorted
// copies: Grid.py:32-66), its tube ranges (Grid.py:68-83) and the first half of a
// Neighborhood (Neighborhood.py:218-245) as a chain of TensorFlow and custom ops
// with a device-to-host read in the middle (the cell counts, which size the tube
// array and bound the sort keys) and another at the end (the number of pairs,
// which sizes the neighbor list).  Here the chain is one entry with ONE blocking
// read at its end: the cell counts stay on the device, the tube array and the
// sort's key width are sized for a caller-given upper bound of cells per
// dimension, and the counts, an overflow flag and the pair total travel to the
// host together.  If a cell count exceeds the bound the call reports it and the
// caller repeats it with a larger one.
//
// A cloud that is one shard of a batch spread over several processes needs the
// cell counts of the WHOLE batch (Grid.py:44-48 takes the maximum over all
// clouds).  For it the chain is cut once, on the device: tfgpc_grid_cells
// computes boxes and this shard's counts without blocking, the caller reduces the
// counts over the processes on the same stream (an all-reduce, still no host
// read), and the main entry continues from the reduced counts.
#include <string.h>

#include "common.cuh"

namespace tfgpc {

int find_neighbors_count_async(const int32_t* order, void* stream, int D, int64_t ns,
                               const float* samples, const int32_t* samples_batch_ids, int64_t n,
                               const float* points, const int64_t* point_keys, const int32_t* ds,
                               int64_t batch_size, const int32_t* num_cells,
                               const float* scaled_aabb_min, const float* inv_cell_sizes,
                               const float* inv_radii, int max_neighs, int32_t* ranges_out, void* ws,
                               size_t ws_bytes, int64_t** total_dev_out);
int build_grid_ds_capacity(cudaStream_t st, int D, int64_t n, const int64_t* sorted_keys,
                           const int32_t* num_cells, int64_t capacity, int32_t* ds_out);

namespace {

struct DimValues { float v[TFGPC_MAX_DIMS]; };

// One block.  From the per-cloud bounding boxes: the boxes widened by 1e-9
// (PointCloud.py:38-43), cells per dimension = max over the clouds of
// ceil(size / cell), at least 1 (Grid.py:44-48), the scaled box minima and the
// inverse cell sizes and radii (custom_ops_wrapper.py:37-43).  Every division is
// the IEEE one the float32 TensorFlow / NumPy expressions perform.
__global__ void grid_params_kernel(int D, int batch_size, float* __restrict__ aabb_min,
                                   float* __restrict__ aabb_max, DimValues cell_sizes,
                                   DimValues radii, int32_t* __restrict__ num_cells,
                                   float* __restrict__ scaled_min, float* __restrict__ inv_cell,
                                   float* __restrict__ inv_radii) {
  __shared__ int cells[TFGPC_MAX_DIMS];
  if (threadIdx.x < TFGPC_MAX_DIMS) cells[threadIdx.x] = 1;
  __syncthreads();
  for (int i = threadIdx.x; i < batch_size * D; i += blockDim.x) {
    const int d = i % D;
    const float cs = cell_sizes.v[d];
    const float mn = __fsub_rn(aabb_min[i], 1e-9f), mx = __fadd_rn(aabb_max[i], 1e-9f);
    aabb_min[i] = mn;
    aabb_max[i] = mx;
    scaled_min[i] = __fdiv_rn(mn, cs);
    const float c = ceilf(__fdiv_rn(__fsub_rn(mx, mn), cs));
    // (a cloud without points has an empty box: it asks for no cells)
    if (c > 0.0f && c < 2147483000.0f) atomicMax(&cells[d], (int)c);
  }
  __syncthreads();
  if (threadIdx.x < D) {
    const int d = threadIdx.x;
    num_cells[d] = cells[d];
    inv_cell[d] = __fdiv_rn(1.0f, cell_sizes.v[d]);
    inv_radii[d] = __fdiv_rn(1.0f, radii.v[d]);
  }
}

// The cell counts the grid asks for go to the report; the kernels index with
// the counts cut to max_cells (what the tube array and the sort keys were sized
// for), and the report says if anything was cut.
// (`asked` and `used` may be the same array)
__global__ void clip_cells_kernel(int D, const int32_t* asked, int max_cells, int32_t* used,
                                  int32_t* __restrict__ report) {
  const int d = threadIdx.x;
  if (d >= D) return;
  const int c = max(asked[d], 1);
  if (c > max_cells) report[TFGPC_MAX_DIMS] = 1;
  report[d] = c;
  used[d] = min(c, max_cells);
}

// report words: [0, D) cell counts, [TFGPC_MAX_DIMS] overflow flag, then the
// 64-bit pair total
__global__ void pack_report_kernel(int32_t* report, const int64_t* total) {
  if (threadIdx.x == 0) *reinterpret_cast<int64_t*>(report + TFGPC_MAX_DIMS + 2) = total ? *total : 0;
}

constexpr int kReportWords = TFGPC_MAX_DIMS + 4;

struct GnWs {
  int32_t* report;        // [kReportWords]
  void* sort_ws;
  size_t sort_bytes;
  void* count_ws;
  size_t count_bytes;
  size_t bytes;
};

GnWs carve(void* ws, int64_t n, int64_t ns) {
  GnWs w;
  char* p = (char*)ws;
  auto take = [&](size_t b) { char* r = p; p += align_up(b, 256); return r; };
  w.report = (int32_t*)take(sizeof(int32_t) * kReportWords);
  w.sort_bytes = tfgpc_sort_keys_workspace_bytes(n);
  w.sort_ws = take(w.sort_bytes);
  w.count_bytes = tfgpc_find_neighbors_workspace_bytes(ns);
  w.count_ws = take(w.count_bytes);
  w.bytes = (size_t)(p - (char*)ws);
  return w;
}

}  // namespace
}  // namespace tfgpc

using namespace tfgpc;

extern "C" size_t tfgpc_grid_neighborhood_workspace_bytes(int64_t n, int64_t ns) {
  if (n < 0 || ns < 0) return 0;
  return carve(nullptr, n, ns).bytes + 256;
}

extern "C" size_t tfgpc_grid_neighborhood_ds_elems(int D, int64_t batch_size, int max_cells) {
  (void)D;
  if (batch_size <= 0 || max_cells <= 0) return 0;
  return (size_t)batch_size * (size_t)max_cells * (size_t)max_cells * 2;
}

static int grid_cells_impl(cudaStream_t st, int D, int64_t n, const float* points,
                           const int32_t* batch_ids, int64_t batch_size, const float* cell_sizes,
                           const float* radii, float* aabb_min_out, float* aabb_max_out,
                           int32_t* num_cells_out, float* scaled_aabb_min_out,
                           float* inv_cell_sizes_out, float* inv_radii_out) {
  DimValues cs{}, rr{};
  for (int d = 0; d < D; ++d) { cs.v[d] = cell_sizes[d]; rr.v[d] = radii[d]; }
  int rc = tfgpc_compute_aabb(st, D, n, points, batch_ids, batch_size, aabb_min_out, aabb_max_out);
  if (rc) return rc;
  ProfScope prof(st, "grid_params");
  grid_params_kernel<<<1, 256, 0, st>>>(D, (int)batch_size, aabb_min_out, aabb_max_out, cs, rr,
                                        num_cells_out, scaled_aabb_min_out, inv_cell_sizes_out,
                                        inv_radii_out);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}

static int check_cells_args(const char* op, int D, int64_t n, int64_t batch_size,
                            const float* cell_sizes, const float* radii) {
  TFGPC_REQUIRE(valid_dims(D), "%s expects a valid number of dimension (got %d)", op, D);
  TFGPC_REQUIRE(n > 0 && n < (int64_t)INT32_MAX && batch_size > 0 && batch_size < (int64_t)INT32_MAX,
                "%s expects 0 < n, 0 < batch size, both below 2^31", op);
  TFGPC_REQUIRE(cell_sizes && radii, "%s got a null pointer", op);
  for (int d = 0; d < D; ++d)
    TFGPC_REQUIRE(cell_sizes[d] > 0.0f && radii[d] > 0.0f,
                  "%s expects positive cell sizes and radii", op);
  return TFGPC_OK;
}

extern "C" int tfgpc_grid_cells(void* stream, int D, int64_t n, const float* points,
                                const int32_t* batch_ids, int64_t batch_size,
                                const float* cell_sizes, const float* radii, float* aabb_min_out,
                                float* aabb_max_out, int32_t* num_cells_out,
                                float* scaled_aabb_min_out, float* inv_cell_sizes_out,
                                float* inv_radii_out) {
  int rc = check_cells_args("GridCells", D, n, batch_size, cell_sizes, radii);
  if (rc) return rc;
  TFGPC_REQUIRE(points && batch_ids && aabb_min_out && aabb_max_out && num_cells_out &&
                scaled_aabb_min_out && inv_cell_sizes_out && inv_radii_out,
                "GridCells got a null pointer");
  return grid_cells_impl((cudaStream_t)stream, D, n, points, batch_ids, batch_size, cell_sizes,
                         radii, aabb_min_out, aabb_max_out, num_cells_out, scaled_aabb_min_out,
                         inv_cell_sizes_out, inv_radii_out);
}

extern "C" int tfgpc_grid_neighborhood_count(
    void* stream, int D, int64_t n, const float* points, const int32_t* batch_ids,
    int64_t batch_size, const float* cell_sizes, const float* radii, int max_cells,
    const int32_t* num_cells_in, int64_t ns, const float* samples,
    const int32_t* samples_batch_ids, int samples_are_points, int max_neighs,
    float* aabb_min_out, float* aabb_max_out, int32_t* num_cells_out, float* scaled_aabb_min_out,
    float* inv_cell_sizes_out, float* inv_radii_out, int64_t* keys_out,
    int32_t* sorted_indices_out, int64_t* sorted_keys_out, float* sorted_points_out,
    int32_t* sorted_batch_ids_out, int32_t* ds_out, int32_t* ranges_out, void* ws, size_t ws_bytes,
    int32_t* num_cells_host_out, int64_t* total_out) {
  int rc = check_cells_args("GridNeighborhood", D, n, batch_size, cell_sizes, radii);
  if (rc) return rc;
  TFGPC_REQUIRE(ns >= 0 && ns < (int64_t)INT32_MAX, "GridNeighborhood expects 0 <= ns < 2^31");
  TFGPC_REQUIRE(max_cells >= 1 && max_cells <= 4096, "GridNeighborhood expects 1 <= max_cells <= 4096");
  TFGPC_REQUIRE(max_neighs >= 0, "GridNeighborhood expects max_neighs >= 0");
  TFGPC_REQUIRE(points && batch_ids && aabb_min_out && aabb_max_out && num_cells_out &&
                scaled_aabb_min_out && inv_cell_sizes_out && inv_radii_out && keys_out &&
                sorted_indices_out && sorted_keys_out && sorted_points_out &&
                sorted_batch_ids_out && ds_out && ws && num_cells_host_out && total_out &&
                (ns == 0 || ranges_out), "GridNeighborhood got a null pointer");
  TFGPC_REQUIRE(num_cells_in != num_cells_out,
                "GridNeighborhood expects the given cell counts outside the output array");
  TFGPC_REQUIRE(samples_are_points == 0 || samples_are_points == 1 || samples_are_points == 2,
                "GridNeighborhood expects samples_are_points 0, 1 or 2");
  TFGPC_REQUIRE(samples_are_points != 0 || ns == 0 || (samples && samples_batch_ids),
                "GridNeighborhood got a null pointer");
  TFGPC_REQUIRE(samples_are_points == 0 || ns == n,
                "GridNeighborhood expects as many samples as points when the samples are the points");
  TFGPC_REQUIRE((uintptr_t)ws % 256 == 0, "GridNeighborhood expects a 256-byte aligned workspace");
  if (ws_bytes < tfgpc_grid_neighborhood_workspace_bytes(n, ns))
    return fail(TFGPC_ENOMEM, "GridNeighborhood workspace too small: %zu < %zu", ws_bytes,
                tfgpc_grid_neighborhood_workspace_bytes(n, ns));
  // key < batch_size * max_cells^D must fit the sort's key width
  double key_space = (double)batch_size;
  for (int d = 0; d < D; ++d) key_space *= (double)max_cells;
  TFGPC_REQUIRE(key_space < 9.0e18, "GridNeighborhood: batch size x max_cells^D exceeds 63 bits");
  int key_bits = 1;
  while (key_bits < 63 && (double)(1ull << key_bits) <= key_space) ++key_bits;

  cudaStream_t st = (cudaStream_t)stream;
  GnWs w = carve(ws, n, ns);
  TFGPC_CUDA(cudaMemsetAsync(w.report, 0, sizeof(int32_t) * kReportWords, st));
  const int32_t* asked = num_cells_in;
  if (!asked) {
    // boxes and cell counts from this cloud alone; the counts are cut in place
    rc = grid_cells_impl(st, D, n, points, batch_ids, batch_size, cell_sizes, radii, aabb_min_out,
                         aabb_max_out, num_cells_out, scaled_aabb_min_out, inv_cell_sizes_out,
                         inv_radii_out);
    if (rc) return rc;
    asked = num_cells_out;
  }
  clip_cells_kernel<<<1, 32, 0, st>>>(D, asked, max_cells, num_cells_out, w.report);
  TFGPC_LAUNCH_CHECK();
  rc = tfgpc_compute_keys(stream, D, n, points, batch_ids, batch_size, scaled_aabb_min_out,
                          num_cells_out, inv_cell_sizes_out, keys_out);
  if (rc) return rc;
  rc = tfgpc_sort_keys_desc(stream, D, n, key_bits, keys_out, points, batch_ids, sorted_indices_out,
                            sorted_keys_out, sorted_points_out, sorted_batch_ids_out, w.sort_ws,
                            w.sort_bytes);
  if (rc) return rc;
  rc = build_grid_ds_capacity(st, D, n, sorted_keys_out, num_cells_out,
                              batch_size * (int64_t)max_cells * max_cells, ds_out);
  if (rc) return rc;
  int64_t* total_dev = nullptr;
  if (ns > 0) {
    // samples_are_points 1: the samples are the points in their own order, visited
    // in the sequence of the key sort; 2: the samples are the SORTED points
    const float* smp = samples_are_points == 1 ? points
                       : samples_are_points == 2 ? sorted_points_out : samples;
    const int32_t* sb = samples_are_points == 1 ? batch_ids
                        : samples_are_points == 2 ? sorted_batch_ids_out : samples_batch_ids;
    const int32_t* order = samples_are_points == 1 ? sorted_indices_out : nullptr;
    rc = find_neighbors_count_async(order, stream, D, ns, smp, sb, n, sorted_points_out,
                                    sorted_keys_out, ds_out, batch_size, num_cells_out,
                                    scaled_aabb_min_out, inv_cell_sizes_out, inv_radii_out, max_neighs,
                                    ranges_out, w.count_ws, w.count_bytes, &total_dev);
    if (rc) return rc;
  }
  pack_report_kernel<<<1, 32, 0, st>>>(w.report, total_dev);
  TFGPC_LAUNCH_CHECK();
  int32_t host[kReportWords];
  rc = read_small(st, w.report, sizeof(host), host);    // the one blocking read
  if (rc) return rc;
  for (int d = 0; d < D; ++d) num_cells_host_out[d] = host[d];
  int64_t total;
  memcpy(&total, host + TFGPC_MAX_DIMS + 2, sizeof(total));
  *total_out = 0;
  if (host[TFGPC_MAX_DIMS])
    return fail(TFGPC_ENOMEM, "GridNeighborhood: the grid needs more than max_cells = %d cells in "
                "a dimension; repeat the call with a larger bound", max_cells);
  if (total > (int64_t)INT32_MAX)
    return fail(TFGPC_EINVAL, "FindNeighbors found %lld pairs; the int32 ranges of the op "
                "contract hold at most 2^31-1", (long long)total);
  *total_out = total;
  return TFGPC_OK;
}
