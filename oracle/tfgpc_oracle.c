/*
 * CPU oracle for the tfg_custom_ops hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's CUDA kernels (schellmi42/tensorflow_graphics_point_clouds,
 * custom_ops/tfg_custom_ops).  It is the checker for the CUDA library and the
 * timed CPU baseline of the benchmark; the product path never links or calls
 * it.  Every function cites the reference file:line it follows.
 *
 * Conventions fixed here (the CUDA kernels use the identical sequences):
 *   - cell coordinate:  rel = fmaf(p, inv_cell, -s_min)  (what nvcc's default
 *     -fmad=true makes of `pPosition*pInvCellSize - pSMinPoint`,
 *     shared/cc/kernels/grid_utils.h:71); the unfused form is selectable.
 *   - neighbor test: t_d = (s_d - p_d) * inv_r_d, d2 = fma chain starting from
 *     t_0*t_0, sqrtf(d2) < 1.0f (count_neighbors_kernels.cu.cc:84-85,
 *     math_helper.h:311-327).
 *   - canonical orders: neighbor lists ascending in sorted point index within
 *     each sample; Poisson samples ascending in sorted index; cell-average
 *     samples ascending in run start.  (The reference places these with
 *     atomics, so its order is not reproducible; its own tests compare sets.)
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_MAX_D 6

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ---------------------------------------------------------------- keys -- */

/* grid_utils.h:63-74 (compute_cell_gpu_funct) */
static inline void cell_of(int D, const float* p, const float* smin,
                           const int* num_cells, const float* inv_cell,
                           int fused, int* cell) {
  for (int d = 0; d < D; ++d) {
    float rel = fused ? fmaf(p[d], inv_cell[d], -smin[d])
                      : (p[d] * inv_cell[d]) - smin[d];
    int c = (int)floorf(rel);
    if (c < 0) c = 0;
    if (c > num_cells[d] - 1) c = num_cells[d] - 1;
    cell[d] = c;
  }
}

/* grid_utils.h:85-100 (compute_key_gpu_funct) */
static inline int64_t key_of(int D, const int* cell, const int* num_cells,
                             int batch) {
  int64_t key = 0, acc = 1;
  for (int d = D - 1; d >= 0; --d) {
    key += (int64_t)cell[d] * acc;
    acc *= num_cells[d];
  }
  return key + acc * (int64_t)batch;
}

/* compute_keys_kernels.cu.cc:41-71 */
void orc_compute_keys(int D, int64_t n, const float* pts, const int* batch_ids,
                      const float* s_aabb_min, const int* num_cells,
                      const float* inv_cell, int fused, int64_t* keys_out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int cell[ORC_MAX_D];
    int b = batch_ids[i];
    cell_of(D, pts + i * D, s_aabb_min + (int64_t)b * D, num_cells, inv_cell,
            fused, cell);
    keys_out[i] = key_of(D, cell, num_cells, b);
  }
}

/* ---------------------------------------------------------------- sort -- */
/* pylib/pc/Grid.py:56-57: tf.argsort(keys, direction='DESCENDING'); ties keep
 * the lower original index first (stable).  Implemented as a merge sort on
 * (key desc, index asc). */
typedef struct { int64_t k; int32_t i; } orc_ki;

static int ki_cmp(const void* a, const void* b) {
  const orc_ki* x = (const orc_ki*)a;
  const orc_ki* y = (const orc_ki*)b;
  if (x->k != y->k) return x->k > y->k ? -1 : 1;
  return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0);
}

void orc_sort_keys_desc(int64_t n, const int64_t* keys, int32_t* perm_out,
                        int64_t* sorted_keys_out) {
  orc_ki* a = (orc_ki*)malloc(sizeof(orc_ki) * (size_t)(n > 0 ? n : 1));
  for (int64_t i = 0; i < n; ++i) { a[i].k = keys[i]; a[i].i = (int32_t)i; }
  qsort(a, (size_t)n, sizeof(orc_ki), ki_cmp);
  for (int64_t i = 0; i < n; ++i) {
    perm_out[i] = a[i].i;
    if (sorted_keys_out) sorted_keys_out[i] = a[i].k;
  }
  free(a);
}

/* ------------------------------------------------------------ grid ds -- */
/* build_grid_ds_kernels.cu.cc:38-71 with grid_utils.h:133-143: the entry of a
 * (batch, c0, c1) tube is (first index, last index + 1) in the sorted array;
 * untouched tubes stay (0,0) from the memset at :104. */
void orc_build_grid_ds(int D, int64_t n, const int64_t* sorted_keys,
                       const int* num_cells, int batch_size, int32_t* ds_out) {
  int64_t div = 1;
  for (int d = 2; d < D; ++d) div *= num_cells[d];
  int64_t n_ds = (int64_t)batch_size * num_cells[0] * num_cells[1];
  memset(ds_out, 0, sizeof(int32_t) * 2 * (size_t)n_ds);
  for (int64_t i = 0; i < n; ++i) {
    int64_t ds = sorted_keys[i] / div;
    if (i > 0 && sorted_keys[i - 1] / div != ds) ds_out[2 * ds] = (int32_t)i;
    if (i + 1 == n || sorted_keys[i + 1] / div != ds)
      ds_out[2 * ds + 1] = (int32_t)(i + 1);
  }
}

/* ------------------------------------------------------ find neighbors -- */

/* first index in [lo,hi) of the descending array with key <= v */
static inline int64_t lb_desc_le(const int64_t* keys, int64_t lo, int64_t hi,
                                 int64_t v) {
  while (lo < hi) {
    int64_t mid = (lo + hi) >> 1;
    if (keys[mid] > v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

/* count_neighbors_kernels.cu.cc:84-85 + math_helper.h:311-327 */
static inline int within(int D, const float* s, const float* p,
                         const float* inv_r) {
  float t = (s[0] - p[0]) * inv_r[0];
  float d2 = t * t;
  for (int d = 1; d < D; ++d) {
    t = (s[d] - p[d]) * inv_r[d];
    d2 = fmaf(t, t, d2);
  }
  return sqrtf(d2) < 1.0f;
}

/* Visits, in ascending sorted-point index, every candidate range of sample s:
 * all cells of the sample's batch whose coordinates differ by at most one from
 * the sample's cell in every dimension (find_ranges_grid_ds_kernels.cu.cc:
 * 80-139: offsets over the leading D-1 coordinates, key range +-1 on the last
 * one, clamped to the grid and to the batch).  Calls fn(lo, hi, ctx). */
typedef void (*range_fn)(int64_t lo, int64_t hi, void* ctx);

static void for_candidate_ranges(int D, const int* cell, int batch, int64_t n,
                                 const int64_t* keys, const int* num_cells,
                                 range_fn fn, void* ctx) {
  int n_off = 1;
  for (int d = 0; d < D - 1; ++d) n_off *= 3;
  /* descending cell key == ascending sorted index */
  for (int o = n_off - 1; o >= 0; --o) {
    int c[ORC_MAX_D];
    int rem = o, ok = 1;
    for (int d = D - 2; d >= 0; --d) {
      c[d] = cell[d] + (rem % 3) - 1;
      rem /= 3;
      if (c[d] < 0 || c[d] >= num_cells[d]) ok = 0;
    }
    if (!ok) continue;
    int lo_l = cell[D - 1] - 1, hi_l = cell[D - 1] + 1;
    if (lo_l < 0) lo_l = 0;
    if (hi_l > num_cells[D - 1] - 1) hi_l = num_cells[D - 1] - 1;
    c[D - 1] = hi_l;
    int64_t k_hi = key_of(D, c, num_cells, batch);
    c[D - 1] = lo_l;
    int64_t k_lo = key_of(D, c, num_cells, batch);
    int64_t a = lb_desc_le(keys, 0, n, k_hi);
    int64_t b = lb_desc_le(keys, a, n, k_lo - 1);
    if (b > a) fn(a, b, ctx);
  }
}

typedef struct {
  int D; const float* s; const float* pts; const float* inv_r;
  int64_t count; int32_t* out; int32_t sample; int64_t limit;
} fn_ctx;

static void fn_visit(int64_t lo, int64_t hi, void* vctx) {
  fn_ctx* c = (fn_ctx*)vctx;
  for (int64_t j = lo; j < hi; ++j) {
    if (c->limit > 0 && c->count >= c->limit) return;
    if (within(c->D, c->s, c->pts + j * c->D, c->inv_r)) {
      if (c->out) {
        c->out[2 * c->count] = (int32_t)j;
        c->out[2 * c->count + 1] = c->sample;
      }
      c->count++;
    }
  }
}

/* find_neighbors_ops.cpp:86-250.  ranges_out[s] = inclusive prefix sum (end
 * offset of sample s).  neigh_out may be NULL (count only); otherwise it must
 * hold 2*M ints, M = ranges_out[ns-1] of a previous count call.  max_neighs>0
 * keeps the first max_neighs hits in canonical order (the reference keeps a
 * time-seeded random subset, store_neighbors_kernels.cu.cc:51-112,216). */
int64_t orc_find_neighbors(int D, int64_t ns, const float* samples,
                           const int* sample_batch, int64_t n,
                           const float* pts, const int64_t* keys,
                           const int* num_cells, const float* s_aabb_min,
                           const float* inv_cell, const float* inv_radii,
                           int max_neighs, int fused, int32_t* ranges_out,
                           int32_t* neigh_out) {
  int64_t* cnt = (int64_t*)malloc(sizeof(int64_t) * (size_t)(ns > 0 ? ns : 1));
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t s = 0; s < ns; ++s) {
    int cell[ORC_MAX_D];
    int b = sample_batch[s];
    cell_of(D, samples + s * D, s_aabb_min + (int64_t)b * D, num_cells,
            inv_cell, fused, cell);
    fn_ctx c = {D, samples + s * D, pts, inv_radii, 0, NULL, (int32_t)s,
                max_neighs};
    for_candidate_ranges(D, cell, b, n, keys, num_cells, fn_visit, &c);
    cnt[s] = c.count;
  }
  int64_t total = 0;
  for (int64_t s = 0; s < ns; ++s) { total += cnt[s]; ranges_out[s] = (int32_t)total; }
  if (neigh_out) {
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t s = 0; s < ns; ++s) {
      int cell[ORC_MAX_D];
      int b = sample_batch[s];
      int64_t start = s ? ranges_out[s - 1] : 0;
      cell_of(D, samples + s * D, s_aabb_min + (int64_t)b * D, num_cells,
              inv_cell, fused, cell);
      fn_ctx c = {D, samples + s * D, pts, inv_radii, 0,
                  neigh_out + 2 * start, (int32_t)s, max_neighs};
      for_candidate_ranges(D, cell, b, n, keys, num_cells, fn_visit, &c);
    }
  }
  free(cnt);
  return total;
}

/* ----------------------------------------------------------------- pdf -- */

/* compute_pdf_kernels.cu.cc:73-130.  mode 0: inv_bw as given; mode 1:
 * sqrtf(n) in every dimension (:47-56, applied with numSamples at :102). */
void orc_compute_pdf(int D, int mode, int64_t n, const float* pts,
                     const int32_t* neigh, const int32_t* ranges,
                     const float* inv_bw, const float* inv_r, float* pdf_out) {
  float bw[ORC_MAX_D];
  for (int d = 0; d < D; ++d) bw[d] = mode == 1 ? sqrtf((float)n) : inv_bw[d];
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t i = 0; i < n; ++i) {
    int64_t a = i ? ranges[i - 1] : 0, b = ranges[i];
    float acc = 0.0f, err = 0.0f;
    for (int64_t m = a; m < b; ++m) {
      const float* q = pts + (int64_t)neigh[2 * m] * D;
      float local = 1.0f;
      for (int d = 0; d < D; ++d) {
        float t = (q[d] - pts[i * D + d]) * bw[d] * inv_r[d];
        local *= bw[d] * expf(t * t * (-0.5f)) * 0.39894228f;
      }
      float v1 = local - err;
      float v2 = acc + v1;
      err = (v2 - acc) - v1;
      acc = v2;
    }
    pdf_out[i] = acc;
  }
}

/* compute_pdf_kernels.cu.cc:149-215.  Sequential here (the reference scatters
 * with atomicAdd, so its summation order is not fixed). */
void orc_compute_pdf_pt_grads(int D, int mode, int64_t n, const float* pts,
                              const int32_t* neigh, const int32_t* ranges,
                              const float* inv_bw, const float* inv_r,
                              const float* pdf_grads, float* pt_grads_out) {
  float bw[ORC_MAX_D];
  for (int d = 0; d < D; ++d) bw[d] = mode == 1 ? sqrtf((float)n) : inv_bw[d];
  double* acc = (double*)calloc((size_t)(n * D > 0 ? n * D : 1), sizeof(double));
  for (int64_t i = 0; i < n; ++i) {
    int64_t a = i ? ranges[i - 1] : 0, b = ranges[i];
    float g = pdf_grads[i];
    for (int64_t m = a; m < b; ++m) {
      int64_t j = neigh[2 * m];
      float diff[ORC_MAX_D];
      float local = g;
      for (int d = 0; d < D; ++d) {
        diff[d] = (pts[j * D + d] - pts[i * D + d]) * bw[d] * inv_r[d];
        local *= bw[d] * expf(diff[d] * diff[d] * (-0.5f)) * 0.39894228f;
      }
      for (int d = 0; d < D; ++d) {
        float v = diff[d] * bw[d] * inv_r[d] * local;
        acc[i * D + d] += (double)v;
        acc[j * D + d] -= (double)v;
      }
    }
  }
  for (int64_t i = 0; i < n * D; ++i) pt_grads_out[i] = (float)acc[i];
  free(acc);
}

/* ---------------------------------------------------------- basis proj -- */

/* basis_proj_kernels.cu.cc:30-127: out[s,c,k] = sum over the sample's range of
 * basis[m,k] * feat[neigh[m].x, c]. */
void orc_basis_proj(int K, int C, int64_t ns, const float* basis,
                    const float* feat, const int32_t* neigh,
                    const int32_t* ranges, float* out) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t s = 0; s < ns; ++s) {
    int64_t a = s ? ranges[s - 1] : 0, b = ranges[s];
    float* o = out + s * (int64_t)C * K;
    for (int64_t i = 0; i < (int64_t)C * K; ++i) o[i] = 0.0f;
    for (int64_t m = a; m < b; ++m) {
      const float* f = feat + (int64_t)neigh[2 * m] * C;
      const float* w = basis + m * K;
      for (int c = 0; c < C; ++c)
        for (int k = 0; k < K; ++k) o[c * K + k] += f[c] * w[k];
    }
  }
}

/* basis_proj_grads_kernels.cu.cc:30-151: dbasis[m,k] = sum_c g[s,c,k] *
 * feat[nbr,c]; dfeat[nbr,c] += sum_k g[s,c,k] * basis[m,k].  Accumulated in
 * double (the reference adds with fp32 atomics in an unspecified order). */
void orc_basis_proj_grads(int K, int C, int64_t ns, int64_t n_in,
                          const float* basis, const float* feat,
                          const int32_t* neigh, const int32_t* ranges,
                          const float* in_grads, float* dbasis, float* dfeat) {
  double* df = (double*)calloc((size_t)(n_in * C > 0 ? n_in * C : 1), sizeof(double));
  for (int64_t s = 0; s < ns; ++s) {
    int64_t a = s ? ranges[s - 1] : 0, b = ranges[s];
    const float* g = in_grads + s * (int64_t)C * K;
    for (int64_t m = a; m < b; ++m) {
      int64_t j = neigh[2 * m];
      const float* f = feat + j * C;
      const float* w = basis + m * K;
      for (int k = 0; k < K; ++k) {
        double acc = 0.0;
        for (int c = 0; c < C; ++c) acc += (double)g[c * K + k] * f[c];
        dbasis[m * K + k] = (float)acc;
      }
      for (int c = 0; c < C; ++c) {
        double acc = 0.0;
        for (int k = 0; k < K; ++k) acc += (double)g[c * K + k] * w[k];
        df[j * C + c] += acc;
      }
    }
  }
  for (int64_t i = 0; i < n_in * C; ++i) dfeat[i] = (float)df[i];
  free(df);
}

/* ------------------------------------------------------------ sampling -- */

/* count_sampling_pd_kernels.cu.cc:42-108 with the 2^D pass loop of :157-180:
 * pass p handles the cells whose coordinate d has parity bit d of p; inside a
 * cell the points are visited in sorted order; a point is taken iff none of
 * its neighbors is taken already.  used_out[n] receives 0/1; returns the
 * number taken.  idx_out (optional) receives the taken sorted indices in
 * ascending order. */
int64_t orc_sampling_poisson(int D, int64_t n, const int64_t* keys,
                             const int* num_cells, const int32_t* neigh,
                             const int32_t* ranges, int32_t* used_out,
                             int32_t* idx_out) {
  memset(used_out, 0, sizeof(int32_t) * (size_t)n);
  int passes = 1 << D;
  for (int p = 0; p < passes; ++p) {
    int64_t i = 0;
    while (i < n) {
      int64_t key = keys[i];
      int64_t e = i;
      while (e < n && keys[e] == key) ++e;
      /* grid_utils.h:110-125 (compute_cell_from_key_gpu_funct) */
      int64_t aux = key; int ok = 1;
      for (int d = D - 1; d >= 0; --d) {
        int c = (int)(aux % num_cells[d]);
        aux /= num_cells[d];
        if ((c % 2) != ((p >> d) & 1)) ok = 0;
      }
      if (ok) {
        for (int64_t q = i; q < e; ++q) {
          int64_t a = q ? ranges[q - 1] : 0, b = ranges[q];
          int valid = 1;
          for (int64_t m = a; m < b && valid; ++m)
            if (used_out[neigh[2 * m]]) valid = 0;
          if (valid) used_out[q] = 1;
        }
      }
      i = e;
    }
  }
  int64_t cnt = 0;
  for (int64_t i = 0; i < n; ++i)
    if (used_out[i]) { if (idx_out) idx_out[cnt] = (int32_t)i; ++cnt; }
  return cnt;
}

/* sampling_avg_kernels.cu.cc:43-88 + store_unique_keys_kernels.cu.cc:36-56:
 * one output per run of equal keys, in ascending run start; mean = sequential
 * fp32 sum / count; batch = key / prod(num_cells).  Returns the run count;
 * pts_out/batch_out may be NULL to count only. */
int64_t orc_sampling_avg(int D, int64_t n, const float* pts,
                         const int64_t* keys, const int* num_cells,
                         float* pts_out, int32_t* batch_out) {
  int64_t total_cells = 1;
  for (int d = 0; d < D; ++d) total_cells *= num_cells[d];
  int64_t cnt = 0, i = 0;
  while (i < n) {
    int64_t key = keys[i];
    float acc[ORC_MAX_D] = {0};
    int64_t e = i;
    while (e < n && keys[e] == key) {
      for (int d = 0; d < D; ++d) acc[d] += pts[e * D + d];
      ++e;
    }
    if (pts_out) {
      for (int d = 0; d < D; ++d) pts_out[cnt * D + d] = acc[d] / (float)(e - i);
      batch_out[cnt] = (int32_t)(key / total_cells);
    }
    ++cnt;
    i = e;
  }
  return cnt;
}
