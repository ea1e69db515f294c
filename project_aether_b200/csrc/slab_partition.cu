// Stable partition of a rank's particles by destination x-slab, the step before
// the all-to-all of the multi-GPU sort.  The reference has no multi-GPU particle
// path; the destination rule extends its cell formula
// (fused_radix_sort.py:93-99): every rank computes the GLOBAL ix with the
// global grid scalars and sends the particle to rank ix / (nx / world).
//
//   slab_count_kernel    particles per (tile, destination)
//   slab_scan_kernel     output offset of every (tile, destination) run,
//                        destination-major so each destination's block is
//                        contiguous and keeps the source order
//   slab_scatter_kernel  stable in-tile ranks per destination, coalesced SoA writes
#include <algorithm>

#include "common.cuh"

namespace aether {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kSlabThreads = 256;
constexpr int kSlabItems = 8;
constexpr int kSlabTile = kSlabThreads * kSlabItems;  // 2048 particles, blocked per thread

__device__ __forceinline__ int slab_of(float x, const AetherGrid& g, int slab_width) {
  return axis_index(x, g.x0, g.inv_dx, g.nx) / slab_width;
}

__device__ __forceinline__ void load8(const float* p, int64_t i0, int64_t n, bool vec, float* out) {
  if (vec && i0 + kSlabItems <= n) {
    const float4 a = ldcs4(p + i0), b = ldcs4(p + i0 + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
#pragma unroll
    for (int k = 0; k < kSlabItems; ++k) out[k] = i0 + k < n ? p[i0 + k] : 0.f;
  }
}

__global__ void __launch_bounds__(kSlabThreads)
slab_count_kernel(const float* __restrict__ x, int64_t n, AetherGrid g, int slab_width, int world,
                  bool vec, uint32_t* __restrict__ tile_count) {
  __shared__ uint32_t count[kMaxWorld];
  if (threadIdx.x < kMaxWorld) count[threadIdx.x] = 0;
  __syncthreads();
  const int64_t i0 = (static_cast<int64_t>(blockIdx.x) * kSlabThreads + threadIdx.x) * kSlabItems;
  float px[kSlabItems];
  load8(x, i0, n, vec, px);
  uint32_t mine[kMaxWorld] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int k = 0; k < kSlabItems; ++k)
    if (i0 + k < n) {
      const int d = slab_of(px[k], g, slab_width);
#pragma unroll
      for (int w = 0; w < kMaxWorld; ++w) mine[w] += (d == w);
    }
#pragma unroll
  for (int w = 0; w < kMaxWorld; ++w) {
    uint32_t c = mine[w];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0 && c) atomicAdd(&count[w], c);
  }
  __syncthreads();
  if (threadIdx.x < world)
    tile_count[static_cast<size_t>(threadIdx.x) * gridDim.x + blockIdx.x] = count[threadIdx.x];
}

// tile_count is [world][tiles]; one block turns it into exclusive offsets in
// that order and writes the per-destination totals.
__global__ void __launch_bounds__(1024)
slab_scan_kernel(uint32_t* __restrict__ tile_count, int64_t entries, int tiles, int world,
                 int64_t* __restrict__ totals) {
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < entries; base += 1024) {
    const int64_t i = base + tid;
    const uint32_t v = i < entries ? tile_count[i] : 0u;
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = warp_sum[lane];
      uint32_t wi = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += t;
      }
      warp_sum[lane] = wi - w;
    }
    __syncthreads();
    const uint32_t excl = carry + warp_sum[warp] + incl - v;
    if (i < entries) tile_count[i] = excl;
    __syncthreads();
    if (tid == 1023) carry = excl + v;
    __syncthreads();
  }
  // Totals: start of destination d+1 minus start of destination d.
  if (tid < world) {
    const uint32_t begin = tile_count[static_cast<size_t>(tid) * tiles];
    const uint32_t end = tid + 1 < world ? tile_count[static_cast<size_t>(tid + 1) * tiles] : carry;
    totals[tid] = static_cast<int64_t>(end - begin);
  }
}

__global__ void __launch_bounds__(kSlabThreads)
slab_scatter_kernel(const float* __restrict__ x, const float* __restrict__ y,
                    const float* __restrict__ z, const float* __restrict__ v, int64_t padded,
                    int64_t n, AetherGrid g, int slab_width, int world, bool vec,
                    const uint32_t* __restrict__ tile_offset, float* __restrict__ ox,
                    float* __restrict__ oy, float* __restrict__ oz, float* __restrict__ ovx,
                    float* __restrict__ ovy, float* __restrict__ ovz) {
  __shared__ unsigned long long warp_lo[8], warp_hi[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t i0 = (static_cast<int64_t>(blockIdx.x) * kSlabThreads + tid) * kSlabItems;
  float f[6][kSlabItems];
  load8(x, i0, n, vec, f[0]);
  load8(y, i0, n, vec, f[1]);
  load8(z, i0, n, vec, f[2]);
  load8(v, i0, n, vec && padded % 4 == 0, f[3]);
  load8(v + padded, i0, n, vec && padded % 4 == 0, f[4]);
  load8(v + 2 * padded, i0, n, vec && padded % 4 == 0, f[5]);
  int dest[kSlabItems];
  // Per-thread counts of the eight destinations, 16 bits each in two words.
  unsigned long long lo = 0, hi = 0;
#pragma unroll
  for (int k = 0; k < kSlabItems; ++k) {
    dest[k] = i0 + k < n ? slab_of(f[0][k], g, slab_width) : -1;
    if (dest[k] >= 0) {
      if (dest[k] < 4) lo += 1ull << (16 * dest[k]);
      else hi += 1ull << (16 * (dest[k] - 4));
    }
  }
  // Exclusive scan over the block's threads (thread order is index order).
  unsigned long long ilo = lo, ihi = hi;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long a = __shfl_up_sync(0xffffffffu, ilo, o);
    const unsigned long long b = __shfl_up_sync(0xffffffffu, ihi, o);
    if (lane >= o) { ilo += a; ihi += b; }
  }
  if (lane == 31) { warp_lo[warp] = ilo; warp_hi[warp] = ihi; }
  __syncthreads();
  unsigned long long base_lo = ilo - lo, base_hi = ihi - hi;
  for (int w = 0; w < warp; ++w) { base_lo += warp_lo[w]; base_hi += warp_hi[w]; }
  uint32_t next[kMaxWorld];
#pragma unroll
  for (int w = 0; w < kMaxWorld; ++w) {
    const uint32_t before = static_cast<uint32_t>(((w < 4 ? base_lo : base_hi) >> (16 * (w & 3))) & 0xffffu);
    next[w] = w < world ? tile_offset[static_cast<size_t>(w) * gridDim.x + blockIdx.x] + before : 0u;
  }
#pragma unroll
  for (int k = 0; k < kSlabItems; ++k) {
    if (dest[k] < 0) continue;
    uint32_t o = 0;
#pragma unroll
    for (int w = 0; w < kMaxWorld; ++w)
      if (dest[k] == w) o = next[w]++;
    ox[o] = f[0][k];
    oy[o] = f[1][k];
    oz[o] = f[2][k];
    ovx[o] = f[3][k];
    ovy[o] = f[4][k];
    ovz[o] = f[5][k];
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

size_t slab_partition_workspace_bytes(int64_t n, int world) {
  const int64_t tiles = std::max<int64_t>(1, (n + kSlabTile - 1) / kSlabTile);
  return static_cast<size_t>(align_up(tiles * world * sizeof(uint32_t), 256));
}

cudaError_t slab_partition(const float* x, const float* y, const float* z, const float* v,
                           int64_t padded, int64_t n, const AetherGrid& g, int world, float* ox,
                           float* oy, float* oz, float* ovx, float* ovy, float* ovz,
                           int64_t* totals, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  if (world < 1 || world > kMaxWorld || g.nx % world != 0) return cudaErrorInvalidValue;
  if (workspace_bytes < slab_partition_workspace_bytes(n, world)) return cudaErrorInvalidValue;
  const int tiles = static_cast<int>(std::max<int64_t>(1, (n + kSlabTile - 1) / kSlabTile));
  uint32_t* tile_count = static_cast<uint32_t*>(workspace);
  const bool vec = aligned16(x) && aligned16(y) && aligned16(z) && aligned16(v);
  const int slab_width = g.nx / world;
  stage_begin(kStageSlabPartition, stream);
  slab_count_kernel<<<tiles, kSlabThreads, 0, stream>>>(x, n, g, slab_width, world, vec, tile_count);
  slab_scan_kernel<<<1, 1024, 0, stream>>>(tile_count, static_cast<int64_t>(tiles) * world, tiles,
                                           world, totals);
  slab_scatter_kernel<<<tiles, kSlabThreads, 0, stream>>>(x, y, z, v, padded, n, g, slab_width,
                                                          world, vec, tile_count, ox, oy, oz, ovx,
                                                          ovy, ovz);
  stage_end(kStageSlabPartition, stream);
  count_launches(3);
  return cudaGetLastError();
}

}  // namespace aether
