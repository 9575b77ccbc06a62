// Row plan of the grouped projection kernels.
//
// The projection and its gradients touch one feature row per neighbor PAIR.
// Samples that lie close to one another share most of their neighbors, so a
// group of four samples taken in a spatially coherent sequence (the visiting
// order: for a cloud searched on its own grid the key sort's permutation) needs
// about half as many distinct neighbor rows as it has pairs (measured on 16384
// uniform points per cloud with 32 neighbors each: 128 pairs, 67 distinct
// neighbors per group).  The plan lists, for every group, its distinct
// neighbors ("rows", ascending) and for each row the pair through which each of
// the group's four samples sees that neighbor (or -1).  The tensor-core kernels
// then gather, multiply and reduce per ROW instead of per pair.
//
// Layout of the plan buffer (all offsets 256-byte aligned):
//   int32 group_begin[groups + 1]   first row of group g (rows of a group are
//                                   contiguous; the space between two groups is
//                                   sized for "no sharing at all" and partly unused)
//   int32 group_rows[groups]        number of rows of group g
//   int32 rows_id[M + 3 groups + pad]   neighbor id of a row (index into the features)
//   int4  rows_pair[same]               pair index per sample slot of the group, -1
//                                       if the sample does not see this neighbor
// (every group starts on a multiple of four rows)
//   scratch of the scan
// Groups whose pair count exceeds kMaxMerge are not merged (one row per pair).
#include "group_plan.cuh"

namespace tfgpc {

int64_t scan_block_sums_elems(int64_t n);
int inclusive_scan_i32(cudaStream_t stream, const int32_t* in, int32_t* out, int64_t n,
                       int64_t* block_sums, int64_t* total);

namespace gp {

PlanView plan_view(void* buf, int64_t ns, int64_t M) {
  PlanView v;
  v.groups = (ns + kG - 1) / kG;
  char* p = (char*)buf;
  auto take = [&](size_t b) { char* r = p; p += align_up(b, 256); return r; };
  const size_t rows = (size_t)M + 3 * (size_t)v.groups + kRowPad;
  v.group_begin = (int32_t*)take((size_t)(v.groups + 1) * 4);
  v.group_rows = (int32_t*)take((size_t)(v.groups > 0 ? v.groups : 1) * 4);
  v.rows_id = (int32_t*)take(rows * 4);
  v.rows_pair = (int4*)take(rows * 16);
  v.scan_sums = (int64_t*)take((size_t)(scan_block_sums_elems(v.groups) + 1) * 8);
  v.bytes = (size_t)(p - (char*)buf);
  return v;
}

namespace {

constexpr int kPlanThreads = 256;
constexpr int kPlanWarps = kPlanThreads / 32;

// Pairs of sample s: [a, a + n).
__device__ __forceinline__ void sample_range(const int32_t* __restrict__ ranges, int64_t s, int& a,
                                             int& n) {
  a = s > 0 ? __ldg(ranges + s - 1) : 0;
  n = __ldg(ranges + s) - a;
}

__global__ void __launch_bounds__(kPlanThreads)
group_pairs_kernel(int64_t ns, int64_t groups, const int32_t* __restrict__ order,
                   const int32_t* __restrict__ ranges, int32_t* __restrict__ pairs_out) {
  const int64_t g = (int64_t)blockIdx.x * kPlanThreads + threadIdx.x;
  if (g >= groups) return;
  int total = 0;
#pragma unroll
  for (int q = 0; q < kG; ++q) {
    const int64_t v = g * kG + q;
    if (v < ns) {
      int a, n;
      sample_range(ranges, order ? __ldg(order + v) : v, a, n);
      total += n;
    }
  }
  // rounded up to four rows: every group then starts 16-byte aligned in rows_id
  pairs_out[g] = (total + 3) & ~3;
}

// Number of elements of the ascending list l[0..n) that are smaller than x.
__device__ __forceinline__ int lower_bound(const int32_t* l, int n, int x) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (l[mid] < x) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// One warp per group.  Where the ids of a group span fewer than kBitmapBits
// values (neighbors of samples in one or two cells: a few tube segments of the
// sorted points) the warp sets one bit per id and ranks an id by the bits below
// it; the group may then hold any number of pairs.  Otherwise
// the four neighbor lists (ascending ids of the sorted
// points, as FindNeighbors writes them) are copied to shared memory; an element
// is "first" if no list of a lower slot holds the same id; the row of an id is
// the number of first elements with a smaller id, counted list by list with one
// binary search each and a running count of the first flags.
__global__ void __launch_bounds__(kPlanThreads)
group_merge_kernel(int64_t ns, int64_t groups, const int32_t* __restrict__ order,
                   const int32_t* __restrict__ ranges, const int2* __restrict__ nb_sorted,
                   const int2* __restrict__ nb_ids, const int32_t* __restrict__ group_begin,
                   int32_t* __restrict__ group_rows, int32_t* __restrict__ rows_id,
                   int4* __restrict__ rows_pair) {
  __shared__ int32_t s_val[kPlanWarps][kMaxMerge];
  __shared__ int16_t s_pre[kPlanWarps][kMaxMerge + 2];
  __shared__ uint32_t s_bits[kPlanWarps][kBitmapBits / 32];
  __shared__ uint16_t s_wpre[kPlanWarps][kBitmapBits / 32];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* val = s_val[w];
  int16_t* pre = s_pre[w];
  const int64_t warps = (int64_t)gridDim.x * kPlanWarps;
  for (int64_t g = (int64_t)blockIdx.x * kPlanWarps + w; g < groups; g += warps) {
    int a0 = 0, a1 = 0, a2 = 0, a3 = 0, n0 = 0, n1 = 0, n2 = 0, n3 = 0;
    {
      const int64_t v = g * kG;
      if (v < ns) sample_range(ranges, order ? __ldg(order + v) : v, a0, n0);
      if (v + 1 < ns) sample_range(ranges, order ? __ldg(order + v + 1) : v + 1, a1, n1);
      if (v + 2 < ns) sample_range(ranges, order ? __ldg(order + v + 2) : v + 2, a2, n2);
      if (v + 3 < ns) sample_range(ranges, order ? __ldg(order + v + 3) : v + 3, a3, n3);
    }
    const int o1 = n0, o2 = o1 + n1, o3 = o2 + n2, total = o3 + n3;
    const int base = __ldg(group_begin + g);
    // element e of the concatenation -> (slot q, position i, pair index m)
    auto locate = [&](int e, int& q, int& i, int& m) {
      q = (e >= o1) + (e >= o2) + (e >= o3);
      const int off = q == 0 ? 0 : q == 1 ? o1 : q == 2 ? o2 : o3;
      const int a = q == 0 ? a0 : q == 1 ? a1 : q == 2 ? a2 : a3;
      i = e - off;
      m = a + i;
    };
    // ---- groups whose ids span few values: one bit per value, rank = bits below
    int lo = INT32_MAX, hi = -1;
    if (lane < 8 && total > 0) {
      // lists ascend: the smallest id is a list's first, the largest its last element
      const int q = lane & 3;
      const int a = q == 0 ? a0 : q == 1 ? a1 : q == 2 ? a2 : a3;
      const int n = q == 0 ? n0 : q == 1 ? n1 : q == 2 ? n2 : n3;
      if (n > 0) {
        const int x = __ldg(&nb_sorted[lane < 4 ? a : a + n - 1].x);
        lo = x; hi = x;
      }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    lo = __shfl_sync(0xffffffffu, lo, 0);
    hi = __shfl_sync(0xffffffffu, hi, 0);
    if (total > 0 && hi - lo < kBitmapBits) {
      uint32_t* bits = s_bits[w];
      uint16_t* wpre = s_wpre[w];
      const int words = ((hi - lo) >> 5) + 1;
      for (int i = lane; i < words; i += 32) bits[i] = 0u;
      __syncwarp();
      for (int e = lane; e < total; e += 32) {
        int q, i, m;
        locate(e, q, i, m);
        const int x = __ldg(&nb_sorted[m].x) - lo;
        atomicOr(&bits[x >> 5], 1u << (x & 31));
      }
      __syncwarp();
      // exclusive running count of the set bits, word by word
      const int per = (words + 31) >> 5;
      int mine = 0;
      for (int i = lane * per; i < min(words, (lane + 1) * per); ++i) mine += __popc(bits[i]);
      int run = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, run, o);
        if (lane >= o) run += v;
      }
      const int rows = __shfl_sync(0xffffffffu, run, 31);
      run -= mine;
      for (int i = lane * per; i < min(words, (lane + 1) * per); ++i) {
        wpre[i] = (uint16_t)run;
        run += __popc(bits[i]);
      }
      for (int r = lane; r < rows; r += 32) rows_pair[base + r] = make_int4(-1, -1, -1, -1);
      __syncwarp();
      for (int e = lane; e < total; e += 32) {
        int q, i, m;
        locate(e, q, i, m);
        const int x = __ldg(&nb_sorted[m].x) - lo;
        const int rank = wpre[x >> 5] + __popc(bits[x >> 5] & ((1u << (x & 31)) - 1u));
        rows_id[base + rank] = __ldg(&nb_ids[m].x);   // every pair of a row holds the same id
        reinterpret_cast<int32_t*>(rows_pair + base + rank)[q] = m;
      }
      if (lane == 0) group_rows[g] = rows;
      __syncwarp();
      continue;
    }
    if (total > kMaxMerge) {
      // too many pairs to merge in shared memory: every pair is its own row
      for (int e = lane; e < total; e += 32) {
        int q, i, m;
        locate(e, q, i, m);
        rows_id[base + e] = __ldg(&nb_ids[m].x);
        rows_pair[base + e] = make_int4(q == 0 ? m : -1, q == 1 ? m : -1, q == 2 ? m : -1,
                                        q == 3 ? m : -1);
      }
      if (lane == 0) group_rows[g] = total;
      continue;
    }
    for (int e = lane; e < total; e += 32) {
      int q, i, m;
      locate(e, q, i, m);
      val[e] = __ldg(&nb_sorted[m].x);
    }
    __syncwarp();
    // first flags and their running count
    int firsts = 0;
    for (int e0 = 0; e0 < total; e0 += 32) {
      const int e = e0 + lane;
      bool first = false;
      if (e < total) {
        int q, i, m;
        locate(e, q, i, m);
        const int x = val[e];
        first = true;
        if (q > 0) { const int p = lower_bound(val, n0, x); first = first && !(p < n0 && val[p] == x); }
        if (q > 1) { const int p = lower_bound(val + o1, n1, x); first = first && !(p < n1 && val[o1 + p] == x); }
        if (q > 2) { const int p = lower_bound(val + o2, n2, x); first = first && !(p < n2 && val[o2 + p] == x); }
      }
      const unsigned ballot = __ballot_sync(0xffffffffu, first);
      if (e < total) pre[e] = (int16_t)(firsts + __popc(ballot & ((1u << lane) - 1u)));
      firsts += __popc(ballot);
    }
    if (lane == 0) pre[total] = (int16_t)firsts;
    const int rows = firsts;
    for (int r = lane; r < rows; r += 32) rows_pair[base + r] = make_int4(-1, -1, -1, -1);
    __syncwarp();
    for (int e = lane; e < total; e += 32) {
      int q, i, m;
      locate(e, q, i, m);
      const int x = val[e];
      // first elements smaller than x, list by list (pre[] counts over the concatenation)
      int rank = 0;
      { const int p = q == 0 ? i : lower_bound(val, n0, x); rank += pre[p] - pre[0]; }
      { const int p = q == 1 ? i : lower_bound(val + o1, n1, x); rank += pre[o1 + p] - pre[o1]; }
      { const int p = q == 2 ? i : lower_bound(val + o2, n2, x); rank += pre[o2 + p] - pre[o2]; }
      { const int p = q == 3 ? i : lower_bound(val + o3, n3, x); rank += pre[o3 + p] - pre[o3]; }
      if (pre[e + 1] != pre[e]) rows_id[base + rank] = __ldg(&nb_ids[m].x);
      reinterpret_cast<int32_t*>(rows_pair + base + rank)[q] = m;
    }
    if (lane == 0) group_rows[g] = rows;
    __syncwarp();
  }
}

}  // namespace
}  // namespace gp
}  // namespace tfgpc

using namespace tfgpc;

extern "C" size_t tfgpc_mcconv_group_plan_bytes(int64_t ns, int64_t M) {
  if (ns < 0 || M < 0) return 0;
  return gp::plan_view(nullptr, ns, M).bytes + 256;
}

extern "C" int tfgpc_mcconv_group_plan(void* stream, int64_t ns, int64_t M, const int32_t* order,
                                       const int32_t* ranges, const int32_t* neighbors_sorted,
                                       const int32_t* neighbor_ids, void* plan,
                                       size_t plan_bytes) {
  TFGPC_REQUIRE(ns >= 0 && ns < (int64_t)INT32_MAX && M >= 0 &&
                M + 3 * ((ns + gp::kG - 1) / gp::kG) + gp::kRowPad <= (int64_t)INT32_MAX,
                "group plan expects 0 <= ns and M + ns < 2^31");
  TFGPC_REQUIRE(plan && (uintptr_t)plan % 256 == 0, "group plan expects a 256-byte aligned buffer");
  if (plan_bytes < tfgpc_mcconv_group_plan_bytes(ns, M))
    return fail(TFGPC_ENOMEM, "group plan buffer too small: %zu < %zu", plan_bytes,
                tfgpc_mcconv_group_plan_bytes(ns, M));
  cudaStream_t st = (cudaStream_t)stream;
  gp::PlanView v = gp::plan_view(plan, ns, M);
  TFGPC_CUDA(cudaMemsetAsync(v.group_begin, 0, sizeof(int32_t), st));
  if (ns == 0) return TFGPC_OK;
  TFGPC_REQUIRE(ranges && (M == 0 || (neighbors_sorted && neighbor_ids)),
                "group plan got a null pointer");
  ProfScope prof(st, "group_plan");
  gp::group_pairs_kernel<<<blocks_for(v.groups, gp::kPlanThreads), gp::kPlanThreads, 0, st>>>(
      ns, v.groups, order, ranges, v.group_begin + 1);
  TFGPC_LAUNCH_CHECK();
  int rc = inclusive_scan_i32(st, v.group_begin + 1, v.group_begin + 1, v.groups, v.scan_sums,
                              v.scan_sums + scan_block_sums_elems(v.groups));
  if (rc) return rc;
  unsigned grid = min(blocks_for(v.groups, gp::kPlanWarps), (unsigned)(sm_count() * 8));
  gp::group_merge_kernel<<<grid, gp::kPlanThreads, 0, st>>>(
      ns, v.groups, order, ranges, (const int2*)neighbors_sorted, (const int2*)neighbor_ids,
      v.group_begin, v.group_rows, v.rows_id, v.rows_pair);
  TFGPC_LAUNCH_CHECK();
  return TFGPC_OK;
}
