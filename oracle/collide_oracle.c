/* CPU restatement of the reference's NTC collision step on cell-sorted
 * particles.  TEST INFRASTRUCTURE ONLY: the product never links or calls this.
 *
 * Follows project_aether/src/custom_kernels/cuda/dsmc_collide_tma.h:59-107
 * (selection count, random words, pair collision) and the per-cell loop of
 * project_aether/src/custom_kernels/cuda/dsmc_collide_tma_test.cu:45-84
 * (CPU replay of the kernel), with the Philox generator of
 * project_aether/src/custom_kernels/cuda/philox.h:56-79.
 *
 * Pinned: tests/golden/collide_cases.npz holds outputs of the reference's own
 * inline functions (compiled from its header by oracle/collide_ref_main.cpp);
 * tests/test_oracle.py compares this file with them bit for bit.
 * Built with -ffp-contract=off: every product and sum rounds on its own, as in
 * the reference's host build.
 */
#include <math.h>
#include <stdint.h>

typedef struct { uint32_t v[4]; } words4;

static words4 philox4x32_10(words4 c, uint32_t k0, uint32_t k1) {
  for (int round = 0; round < 10; ++round) {
    if (round > 0) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
    const uint64_t p0 = (uint64_t)0xD2511F53u * c.v[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c.v[2];
    words4 next;
    next.v[0] = (uint32_t)(p1 >> 32) ^ c.v[1] ^ k0;
    next.v[1] = (uint32_t)p1;
    next.v[2] = (uint32_t)(p0 >> 32) ^ c.v[3] ^ k1;
    next.v[3] = (uint32_t)p0;
    c = next;
  }
  return c;
}

static float unit_float(uint32_t bits) { return (float)(bits >> 8) * (1.0f / 16777216.0f); }

/* dsmc_collide_tma.h:75-82: counter (cell, pair, step lo, step hi), key = seed. */
static words4 collision_words(int cell, uint32_t pair, uint64_t seed, uint64_t step) {
  words4 c = {{(uint32_t)cell, pair, (uint32_t)step, (uint32_t)(step >> 32)}};
  return philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
}

/* dsmc_collide_tma.h:63-72. */
static int ntc_selections(int count, float majorant, float selection_factor, float u) {
  const float expected = 0.5f * (float)count * (float)(count - 1) * selection_factor * majorant;
  const int selections = (int)floorf(expected + u);
  return selections < count / 2 ? selections : count / 2;
}

/* dsmc_collide_tma.h:89-113.  Returns 1 when the pair collided. */
static int collide_pair(float* a, float* b, float majorant, float coefficient, float exponent,
                        const words4* r, float* sigma_g) {
  const float gx = a[0] - b[0], gy = a[1] - b[1], gz = a[2] - b[2];
  const float g = sqrtf(gx * gx + gy * gy + gz * gz);
  *sigma_g = g > 0.0f ? coefficient * powf(g, exponent) : 0.0f;
  if (unit_float(r->v[0]) * majorant >= *sigma_g) return 0;
  const float cos_chi = 2.0f * unit_float(r->v[1]) - 1.0f;
  const float sin_chi = sqrtf(fmaxf(1.0f - cos_chi * cos_chi, 0.0f));
  const float azimuth = 6.28318530718f * unit_float(r->v[2]);
  const float post[3] = {g * sin_chi * cosf(azimuth), g * sin_chi * sinf(azimuth), g * cos_chi};
  for (int c = 0; c < 3; ++c) {
    const float center = 0.5f * (a[c] + b[c]);
    a[c] = center + 0.5f * post[c];
    b[c] = center - 0.5f * post[c];
  }
  return 1;
}

/* velocity is (3, padded) row-major, updated in place; sigma_g_max (C,) is raised
 * to the largest sigma*g seen; collisions (C,) receives the accepted pairs.
 * pair_sigma_g, when not null, receives sigma*g of every tested pair at the index
 * of its first particle (diagnostics for tolerance tests).
 * dsmc_collide_tma_test.cu:45-84. */
void collide_cells(float* velocity, const int32_t* cell_start, float* sigma_g_max,
                   int32_t* collisions, int32_t num_cells, int64_t padded,
                   float selection_factor, float coefficient, float exponent, uint64_t seed,
                   uint64_t step, float* pair_sigma_g) {
#pragma omp parallel for schedule(dynamic, 1024)
  for (int32_t cell = 0; cell < num_cells; ++cell) {
    const int32_t start = cell_start[cell];
    const int32_t count = cell_start[cell + 1] - start;
    const float majorant = sigma_g_max[cell];
    const words4 draw = collision_words(cell, 0xFFFFFFFFu, seed, step);
    const int selections = ntc_selections(count, majorant, selection_factor, unit_float(draw.v[0]));
    float observed = 0.0f;
    int accepted = 0;
    for (int pair = 0; pair < selections; ++pair) {
      const int64_t i = (int64_t)start + 2 * pair;
      float a[3], b[3];
      for (int c = 0; c < 3; ++c) {
        a[c] = velocity[c * padded + i];
        b[c] = velocity[c * padded + i + 1];
      }
      const words4 r = collision_words(cell, (uint32_t)pair, seed, step);
      float sigma_g = 0.0f;
      if (collide_pair(a, b, majorant, coefficient, exponent, &r, &sigma_g)) {
        for (int c = 0; c < 3; ++c) {
          velocity[c * padded + i] = a[c];
          velocity[c * padded + i + 1] = b[c];
        }
        ++accepted;
      }
      if (pair_sigma_g) pair_sigma_g[i] = sigma_g;
      observed = observed > sigma_g ? observed : sigma_g;
    }
    sigma_g_max[cell] = majorant > observed ? majorant : observed;
    collisions[cell] = accepted;
  }
}

/* Number of candidate pairs per cell (what a cell's draw selects). */
void collide_selections(const int32_t* cell_start, const float* sigma_g_max, int32_t* selections,
                        int32_t num_cells, float selection_factor, uint64_t seed, uint64_t step) {
  for (int32_t cell = 0; cell < num_cells; ++cell) {
    const int32_t count = cell_start[cell + 1] - cell_start[cell];
    const words4 draw = collision_words(cell, 0xFFFFFFFFu, seed, step);
    selections[cell] = ntc_selections(count, sigma_g_max[cell], selection_factor, unit_float(draw.v[0]));
  }
}
