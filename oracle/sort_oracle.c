/* CPU oracle for the DSMC particle sort, in plain C.  TEST INFRASTRUCTURE ONLY.
 *
 * Restates the reference's result contract so that large cases can be checked
 * and timed on host cores:
 *   - key generation: project_aether/src/custom_kernels/triton/
 *     fused_radix_sort.py:93-103 (float32 cell index, x-fastest cell id,
 *     7 Philox shuffle bits);
 *   - Philox4x32-10: project_aether/src/custom_kernels/cuda/philox.h:56-72,
 *     counter (i,0,0,0), key (seed lo32, seed hi32), word 0;
 *   - the sort: a stable least-significant-digit counting sort, which the
 *     reference pins equal to its replay
 *     (project_aether/tests/test_radix_sort.py:22-33);
 *   - per-cell counts and exclusive starts: fused_radix_sort.py:201-203,277-279;
 *   - payload gather: project_aether/src/physics_engine/dsmc_gpu_pipeline.py:107-109.
 *
 * Parity status: pinned through tests/golden (Philox known answers made from
 * the reference header, replay cases made by importing the reference module).
 * Nothing in the product links or loads this file.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline uint32_t philox_word0(uint32_t c0, uint32_t k0, uint32_t k1) {
  uint32_t c1 = 0, c2 = 0, c3 = 0;
  for (int r = 0; r < 10; ++r) {
    if (r > 0) {
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)p1;
    c3 = (uint32_t)p0;
    c0 = n0;
    c2 = n2;
  }
  return c0;
}

/* Known-answer hook for the tests. */
void oracle_philox_word0(const uint32_t* counters, int64_t n, uint64_t seed, uint32_t* out) {
  for (int64_t i = 0; i < n; ++i)
    out[i] = philox_word0(counters[i], (uint32_t)seed, (uint32_t)(seed >> 32));
}

static inline int axis_index(float c, float lo, float inv, int cells) {
  /* Separate rounded subtract and multiply (no fused multiply-add), then a
   * round-toward-zero conversion that saturates like the GPU's.  Build with
   * -ffp-contract=off. */
  float d = c - lo;
  float v = d * inv;
  int i;
  if (!(v == v)) i = 0;
  else if (v >= 2147483648.0f) i = 2147483647;
  else if (v <= -2147483648.0f) i = -2147483647 - 1;
  else i = (int)v;
  if (i < 0) i = 0;
  if (i > cells - 1) i = cells - 1;
  return i;
}

/* Threads a call with `threads` <= 0 would use (the OpenMP maximum, which the
 * environment variable OMP_NUM_THREADS caps), so that a benchmark can print the
 * number really used. */
int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* 1 when the library was built with OpenMP, else 0 (every call then runs on one thread). */
int oracle_has_openmp(void) {
#ifdef _OPENMP
  return 1;
#else
  return 0;
#endif
}

static int resolve_threads(int threads) {
#ifdef _OPENMP
  if (threads <= 0) threads = omp_get_max_threads();
#else
  threads = 1;
#endif
  return threads < 1 ? 1 : threads;
}

/* Stable LSD counting sort of (key, index) pairs by 8-bit digits, parallel over
 * contiguous blocks: block b's elements of digit d go after all smaller digits
 * and after the same digit of blocks < b, which keeps the sort stable. */
static int lsd_sort_pairs(uint32_t* keys, int32_t* vals, int64_t n, int key_bits, int threads) {
  uint32_t* k2 = (uint32_t*)malloc((size_t)(n > 0 ? n : 1) * sizeof(uint32_t));
  int32_t* v2 = (int32_t*)malloc((size_t)(n > 0 ? n : 1) * sizeof(int32_t));
  int64_t* hist = (int64_t*)malloc((size_t)threads * 256 * sizeof(int64_t));
  if (!k2 || !v2 || !hist) { free(k2); free(v2); free(hist); return -1; }
  uint32_t *ka = keys, *kb = k2;
  int32_t *va = vals, *vb = v2;
  int passes = (key_bits + 7) / 8;
  int64_t block = (n + threads - 1) / threads;
  for (int p = 0; p < passes; ++p) {
    int shift = 8 * p;
#pragma omp parallel num_threads(threads)
    {
#ifdef _OPENMP
      int t = omp_get_thread_num();
#else
      int t = 0;
#endif
      int64_t lo = t * block, hi = lo + block;
      if (lo > n) lo = n;
      if (hi > n) hi = n;
      int64_t* h = hist + (size_t)t * 256;
      memset(h, 0, 256 * sizeof(int64_t));
      for (int64_t i = lo; i < hi; ++i) h[(ka[i] >> shift) & 255]++;
#pragma omp barrier
#pragma omp single
      {
        int64_t run = 0;
        for (int d = 0; d < 256; ++d)
          for (int b = 0; b < threads; ++b) {
            int64_t c = hist[(size_t)b * 256 + d];
            hist[(size_t)b * 256 + d] = run;
            run += c;
          }
      }
      for (int64_t i = lo; i < hi; ++i) {
        int64_t dst = h[(ka[i] >> shift) & 255]++;
        kb[dst] = ka[i];
        vb[dst] = va[i];
      }
    }
    uint32_t* tk = ka; ka = kb; kb = tk;
    int32_t* tv = va; va = vb; vb = tv;
  }
  if (ka != keys) {
    memcpy(keys, ka, (size_t)n * sizeof(uint32_t));
    memcpy(vals, va, (size_t)n * sizeof(int32_t));
  }
  free(k2); free(v2); free(hist);
  return 0;
}

int oracle_stable_argsort_u32(const uint32_t* keys, int64_t n, int32_t* order, int threads) {
  threads = resolve_threads(threads);
  uint32_t* k = (uint32_t*)malloc((size_t)(n > 0 ? n : 1) * sizeof(uint32_t));
  if (!k) return -1;
  uint32_t any = 0;
  for (int64_t i = 0; i < n; ++i) { k[i] = keys[i]; order[i] = (int32_t)i; any |= keys[i]; }
  int bits = 0;
  while (bits < 32 && (any >> bits)) ++bits;
  int rc = lsd_sort_pairs(k, order, n, bits, threads);
  free(k);
  return rc;
}

/* The whole path.  `velocity` is (3, padded) row-major or NULL; outputs with a
 * NULL pointer are skipped.  Cell ids are local to the x-slab
 * [ix_offset, ix_offset + nx_local) of the global grid (nx_local = nx and
 * ix_offset = 0 for the whole grid). */
int oracle_sort_particles(const float* x, const float* y, const float* z, const float* velocity,
                          int64_t n, int64_t padded, float x0, float y0, float z0, float inv_dx,
                          float inv_dy, float inv_dz, int nx, int ny, int nz, int ix_offset,
                          int nx_local, uint64_t seed, uint32_t* keys, int32_t* order,
                          int32_t* cell_counts, int32_t* cell_start, float* xs, float* ys,
                          float* zs, float* vs, int threads) {
  threads = resolve_threads(threads);
  int64_t cells = (int64_t)nx_local * ny * nz;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  uint32_t any = 0;
#pragma omp parallel for num_threads(threads) reduction(| : any) schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int ix = axis_index(x[i], x0, inv_dx, nx);
    int iy = axis_index(y[i], y0, inv_dy, ny);
    int iz = axis_index(z[i], z0, inv_dz, nz);
    /* Slab form (an extension of the reference's formula): a particle outside the slab is
     * binned into the slab's nearest column, so that a cell id is never out of range. */
    int ixl = ix - ix_offset;
    if (ixl < 0) ixl = 0;
    if (ixl > nx_local - 1) ixl = nx_local - 1;
    uint32_t cell = (uint32_t)(((int64_t)iz * ny + iy) * nx_local + ixl);
    uint32_t key = (cell << 7) | (philox_word0((uint32_t)i, k0, k1) >> 25);
    keys[i] = key;
    order[i] = (int32_t)i;
    any |= key;
  }
  int bits = 0;
  while (bits < 32 && (any >> bits)) ++bits;
  if (lsd_sort_pairs(keys, order, n, bits, threads) != 0) return -1;
  if (cell_counts) {
    memset(cell_counts, 0, (size_t)cells * sizeof(int32_t));
    for (int64_t i = 0; i < n; ++i) cell_counts[keys[i] >> 7]++;
    if (cell_start) {
      int32_t run = 0;
      cell_start[0] = 0;
      for (int64_t c = 0; c < cells; ++c) { run += cell_counts[c]; cell_start[c + 1] = run; }
    }
  }
  if (xs) {
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
      int32_t p = order[i];
      xs[i] = x[p]; ys[i] = y[p]; zs[i] = z[p];
      if (velocity && vs) {
        vs[i] = velocity[p];
        vs[padded + i] = velocity[padded + p];
        vs[2 * padded + i] = velocity[2 * padded + p];
      }
    }
  }
  return 0;
}
