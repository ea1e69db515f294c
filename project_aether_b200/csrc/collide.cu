// No-Time-Counter collisions on cell-sorted particles for sm_100a.
//
// Replaces the reference's sm_90a kernel (custom_kernels/cuda/dsmc_collide_tma.cu:
// one warp per cell, 2-D TMA boxes of a fixed window, a second kernel for large
// cells) behind the same C entry point (dsmc_collide_tma.h:121-129).  The
// arithmetic of a pair follows dsmc_collide_tma.h:59-113 with every product and
// sum rounded on its own, as the reference's host replay computes them
// (dsmc_collide_tma_test.cu:45-84).
//
// Layout of the work: a block owns a run of consecutive cells.  It packs as many
// whole cells as fit into a shared-memory stage (4096 particles), reads their
// velocities with coalesced 128-bit loads, draws every cell's number of candidate
// pairs, and then hands the pairs of ALL staged cells out to its threads one pair
// per thread, so that cells of ten particles keep a block as busy as cells of a
// thousand.  Velocities are updated in shared memory and the stage is written
// back with coalesced stores only when a pair in it collided.  A cell larger
// than the stage is worked on in global memory by the whole block.
#include <algorithm>

#include "common.cuh"

namespace aether {
namespace {

constexpr int kCollideThreads = 256;
constexpr int kMaxCellsPerBlock = 256;
constexpr int kStageParticles = 4096;
constexpr int kStageRow = kStageParticles + 4;  // room for the aligned start of the first quad
constexpr uint32_t kCellDraw = 0xFFFFFFFFu;     // pair id of a cell's selection draw

struct CollideArgs {
  float* velocity;
  const int* cell_start;
  float* sigma_g_max;
  int* collisions;
  int padded;
  int num_cells;
  int cells_per_block;
  int aligned;  // velocity rows start on 16-byte boundaries
  float selection_factor, coefficient, exponent;
  uint32_t key0, key1, step_lo, step_hi;
};

// Philox4x32-10, all four words (cuda/philox.h:56-72).
__device__ __forceinline__ uint4 philox4(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                         uint32_t k0, uint32_t k1) {
  constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u;
  constexpr uint32_t kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    if (r > 0) {
      k0 += kW0;
      k1 += kW1;
    }
    const uint32_t hi0 = __umulhi(kM0, c0), lo0 = kM0 * c0;
    const uint32_t hi1 = __umulhi(kM1, c2), lo1 = kM1 * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
  }
  return make_uint4(c0, c1, c2, c3);
}

// 24 random bits as a float in [0, 1) (cuda/philox.h:77-79).
__device__ __forceinline__ float unit_float(uint32_t bits) {
  return __fmul_rn(static_cast<float>(bits >> 8), 1.0f / 16777216.0f);
}

__device__ __forceinline__ uint4 collision_words(int cell, uint32_t pair, const CollideArgs& a) {
  return philox4(static_cast<uint32_t>(cell), pair, a.step_lo, a.step_hi, a.key0, a.key1);
}

// floor(1/2 N (N-1) F sigma_g_max + U), at most N/2 (dsmc_collide_tma.h:63-72).
__device__ __forceinline__ int ntc_selections(int count, float majorant, float factor, float u) {
  float expected = __fmul_rn(0.5f, static_cast<float>(count));
  expected = __fmul_rn(expected, static_cast<float>(count - 1));
  expected = __fmul_rn(expected, factor);
  expected = __fmul_rn(expected, majorant);
  const int selections = static_cast<int>(floorf(__fadd_rn(expected, u)));
  return min(selections, count / 2);
}

// Tests one candidate pair and scatters it isotropically in the centre-of-mass
// frame when it is accepted (dsmc_collide_tma.h:89-113).
__device__ __forceinline__ bool collide_pair(float* a, float* b, float majorant,
                                             const CollideArgs& p, const uint4& r,
                                             float* sigma_g) {
  const float gx = __fsub_rn(a[0], b[0]), gy = __fsub_rn(a[1], b[1]), gz = __fsub_rn(a[2], b[2]);
  const float g = sqrtf(__fadd_rn(__fadd_rn(__fmul_rn(gx, gx), __fmul_rn(gy, gy)), __fmul_rn(gz, gz)));
  *sigma_g = g > 0.0f ? __fmul_rn(p.coefficient, powf(g, p.exponent)) : 0.0f;
  if (__fmul_rn(unit_float(r.x), majorant) >= *sigma_g) return false;
  const float cos_chi = __fsub_rn(__fmul_rn(2.0f, unit_float(r.y)), 1.0f);
  const float sin_chi = sqrtf(fmaxf(__fsub_rn(1.0f, __fmul_rn(cos_chi, cos_chi)), 0.0f));
  const float azimuth = __fmul_rn(6.28318530718f, unit_float(r.z));
  const float gs = __fmul_rn(g, sin_chi);
  const float post[3] = {__fmul_rn(gs, cosf(azimuth)), __fmul_rn(gs, sinf(azimuth)),
                         __fmul_rn(g, cos_chi)};
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const float center = __fmul_rn(0.5f, __fadd_rn(a[c], b[c]));
    const float half = __fmul_rn(0.5f, post[c]);
    a[c] = __fadd_rn(center, half);
    b[c] = __fsub_rn(center, half);
  }
  return true;
}

struct CollideSmem {
  float stage[3][kStageRow];
  int start[kMaxCellsPerBlock + 1];        // cell_start of the block's cells
  int pair_first[kMaxCellsPerBlock + 1];   // exclusive prefix of candidate pairs of the staged cells
  int accepted[kMaxCellsPerBlock];
  uint32_t observed[kMaxCellsPerBlock];    // largest sigma*g seen, as float bits (non-negative)
  float majorant[kMaxCellsPerBlock];       // sigma_g_max of the staged cells before this step
  uint32_t warp_sum[32];
  uint32_t total;
  int any_accepted;
};

__global__ void __launch_bounds__(kCollideThreads)
collide_kernel(CollideArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  CollideSmem& s = *reinterpret_cast<CollideSmem*>(smem_raw);
  const int tid = threadIdx.x;
  const int first_cell = blockIdx.x * a.cells_per_block;
  const int cells_here = min(a.cells_per_block, a.num_cells - first_cell);
  for (int i = tid; i <= cells_here; i += kCollideThreads) s.start[i] = a.cell_start[first_cell + i];
  __syncthreads();

  int lo = 0;  // first cell of the block not yet done
  while (lo < cells_here) {
    const int origin = s.start[lo];
    // Whole cells lo..hi-1 fit the stage: hi = last index with start[hi] <= origin + stage.
    int hi;
    {
      int left = lo, right = cells_here;  // invariant: start[left] <= limit
      const int limit = origin + kStageParticles;
      while (left < right) {
        const int mid = (left + right + 1) >> 1;
        if (s.start[mid] <= limit) left = mid; else right = mid - 1;
      }
      hi = left;
    }
    if (hi == lo) {
      // One cell larger than the stage: the block works on it in global memory.
      const int cell = first_cell + lo;
      const int count = s.start[lo + 1] - origin;
      const float majorant = a.sigma_g_max[cell];
      if (tid == 0) {
        s.accepted[0] = 0;
        s.observed[0] = 0;
      }
      __syncthreads();
      const int selections = ntc_selections(count, majorant, a.selection_factor,
                                            unit_float(collision_words(cell, kCellDraw, a).x));
      int mine = 0;
      float seen = 0.0f;
      for (int pair = tid; pair < selections; pair += kCollideThreads) {
        const size_t i = static_cast<size_t>(origin) + 2 * pair;
        float v1[3], v2[3];
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          v1[c] = a.velocity[static_cast<size_t>(c) * a.padded + i];
          v2[c] = a.velocity[static_cast<size_t>(c) * a.padded + i + 1];
        }
        float sigma_g = 0.0f;
        if (collide_pair(v1, v2, majorant, a, collision_words(cell, static_cast<uint32_t>(pair), a),
                         &sigma_g)) {
#pragma unroll
          for (int c = 0; c < 3; ++c) {
            a.velocity[static_cast<size_t>(c) * a.padded + i] = v1[c];
            a.velocity[static_cast<size_t>(c) * a.padded + i + 1] = v2[c];
          }
          ++mine;
        }
        seen = fmaxf(seen, sigma_g);
      }
      if (mine) atomicAdd(&s.accepted[0], mine);
      if (seen > 0.0f) atomicMax(&s.observed[0], __float_as_uint(seen));
      __syncthreads();
      if (tid == 0) {
        a.sigma_g_max[cell] = fmaxf(majorant, __uint_as_float(s.observed[0]));
        a.collisions[cell] = s.accepted[0];
      }
      __syncthreads();
      lo += 1;
      continue;
    }

    const int staged_cells = hi - lo;
    const int end = s.start[hi];
    const int shift = a.aligned ? (origin & 3) : 0;  // stage index 0 holds particle origin - shift
    const int base = origin - shift;
    // Stage the velocities of particles [origin, end).
    if (a.aligned) {
      const int quads = (end - base + 3) >> 2;  // the rows are padded to a multiple of four
      for (int q = tid; q < quads; q += kCollideThreads) {
#pragma unroll
        for (int c = 0; c < 3; ++c)
          *reinterpret_cast<float4*>(&s.stage[c][4 * q]) = *reinterpret_cast<const float4*>(
              a.velocity + static_cast<size_t>(c) * a.padded + base + 4 * q);
      }
    } else {
      for (int i = tid; i < end - origin; i += kCollideThreads) {
#pragma unroll
        for (int c = 0; c < 3; ++c)
          s.stage[c][i] = a.velocity[static_cast<size_t>(c) * a.padded + origin + i];
      }
    }
    // Candidate pairs of every staged cell (one cell per thread; at most 256 cells).
    float majorant = 0.0f;
    uint32_t selections = 0;
    if (tid < staged_cells) {
      const int cell = first_cell + lo + tid;
      const int count = s.start[lo + tid + 1] - s.start[lo + tid];
      majorant = a.sigma_g_max[cell];
      selections = static_cast<uint32_t>(max(
          0, ntc_selections(count, majorant, a.selection_factor,
                            unit_float(collision_words(cell, kCellDraw, a).x))));
      s.accepted[tid] = 0;
      s.observed[tid] = 0;
      s.majorant[tid] = majorant;
    }
    if (tid == 0) s.any_accepted = 0;
    const uint32_t before = block_exclusive_scan(selections, s.warp_sum, &s.total);
    if (tid < staged_cells) s.pair_first[tid] = static_cast<int>(before);
    __syncthreads();
    const int pairs = static_cast<int>(s.total);
    if (tid == 0) s.pair_first[staged_cells] = pairs;
    __syncthreads();

    for (int p = tid; p < pairs; p += kCollideThreads) {
      // The cell of pair p: last t with pair_first[t] <= p (cells without pairs share a value).
      int left = 0, right = staged_cells - 1;
      while (left < right) {
        const int mid = (left + right + 1) >> 1;
        if (s.pair_first[mid] <= p) left = mid; else right = mid - 1;
      }
      const int t = left;
      const int pair = p - s.pair_first[t];
      const int cell = first_cell + lo + t;
      const int k = s.start[lo + t] - base + 2 * pair;
      float v1[3], v2[3];
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        v1[c] = s.stage[c][k];
        v2[c] = s.stage[c][k + 1];
      }
      const float cell_majorant = s.majorant[t];
      float sigma_g = 0.0f;
      if (collide_pair(v1, v2, cell_majorant, a,
                       collision_words(cell, static_cast<uint32_t>(pair), a), &sigma_g)) {
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          s.stage[c][k] = v1[c];
          s.stage[c][k + 1] = v2[c];
        }
        atomicAdd(&s.accepted[t], 1);
        s.any_accepted = 1;
      }
      if (sigma_g > 0.0f) atomicMax(&s.observed[t], __float_as_uint(sigma_g));
    }
    __syncthreads();
    if (tid < staged_cells) {
      const int cell = first_cell + lo + tid;
      a.sigma_g_max[cell] = fmaxf(majorant, __uint_as_float(s.observed[tid]));
      a.collisions[cell] = s.accepted[tid];
    }
    if (s.any_accepted) {
      // Write the stage back: 128-bit stores over the quads that lie wholly inside
      // [origin, end), single words at the ragged ends.
      if (a.aligned) {
        const int first_quad = (shift + 3) >> 2;          // first quad starting at or after origin
        const int last_quad = (end - base) >> 2;           // quads below this end inside the range
        for (int q = first_quad + tid; q < last_quad; q += kCollideThreads) {
#pragma unroll
          for (int c = 0; c < 3; ++c)
            *reinterpret_cast<float4*>(a.velocity + static_cast<size_t>(c) * a.padded + base +
                                       4 * q) = *reinterpret_cast<const float4*>(&s.stage[c][4 * q]);
        }
        const int head_end = min(end - base, 4 * first_quad);
        const int tail_begin = max(head_end, 4 * last_quad);
        if (tid < 8) {
          const int i = tid < 4 ? shift + tid : tail_begin + (tid - 4);
          const bool ok = tid < 4 ? i < head_end : i < end - base;
          if (ok) {
#pragma unroll
            for (int c = 0; c < 3; ++c)
              a.velocity[static_cast<size_t>(c) * a.padded + base + i] = s.stage[c][i];
          }
        }
      } else {
        for (int i = tid; i < end - origin; i += kCollideThreads) {
#pragma unroll
          for (int c = 0; c < 3; ++c)
            a.velocity[static_cast<size_t>(c) * a.padded + origin + i] = s.stage[c][i];
        }
      }
    }
    __syncthreads();
    lo = hi;
  }
}

}  // namespace

// Enqueues one collision step.  velocity (3, padded) is updated in place,
// sigma_g_max (C,) is raised to the largest sigma*g observed, collisions (C,)
// receives the accepted pairs of every cell.
cudaError_t collide_cells(float* velocity, const int* cell_start, float* sigma_g_max,
                          int* collisions, int num_particles, int padded, int num_cells,
                          float selection_factor, float coefficient, float exponent,
                          uint64_t seed, uint64_t step, cudaStream_t stream) {
  if (num_particles < 0 || num_cells < 0 || padded < num_particles || padded % 4 != 0)
    return cudaErrorInvalidValue;
  if (num_cells == 0) return cudaSuccess;
  if (!velocity || !cell_start || !sigma_g_max || !collisions) return cudaErrorInvalidValue;
  CollideArgs a{};
  a.velocity = velocity;
  a.cell_start = cell_start;
  a.sigma_g_max = sigma_g_max;
  a.collisions = collisions;
  a.padded = padded;
  a.num_cells = num_cells;
  // Cells per block: about three quarters of a stage at the average occupancy, so
  // that most blocks fill the stage once.
  const double per_cell = std::max(1.0, static_cast<double>(num_particles) / num_cells);
  int cells = static_cast<int>(0.75 * kStageParticles / per_cell);
  cells = std::max(32, std::min(kMaxCellsPerBlock, cells / 32 * 32));
  a.cells_per_block = cells;
  a.aligned = (reinterpret_cast<uintptr_t>(velocity) & 15) == 0;
  a.selection_factor = selection_factor;
  a.coefficient = coefficient;
  a.exponent = exponent;
  a.key0 = static_cast<uint32_t>(seed);
  a.key1 = static_cast<uint32_t>(seed >> 32);
  a.step_lo = static_cast<uint32_t>(step);
  a.step_hi = static_cast<uint32_t>(step >> 32);
  cudaError_t e = cudaFuncSetAttribute(collide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(CollideSmem)));
  if (e != cudaSuccess) return e;
  const int blocks = (num_cells + cells - 1) / cells;
  stage_begin(kStageCollide, stream);
  collide_kernel<<<blocks, kCollideThreads, sizeof(CollideSmem), stream>>>(a);
  stage_end(kStageCollide, stream);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace aether
