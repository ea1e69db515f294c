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

constexpr int kSlabThreads = 256;
constexpr int kSlabItems = 8;
constexpr int kSlabTile = kSlabThreads * kSlabItems;  // 2048 particles, blocked per thread

// Destination rank of a particle: ix / slab_width, as a chain of compares (at
// most eight slabs; an integer division costs several times more).
__device__ __forceinline__ int slab_of(float x, const AetherGrid& g, int slab_width) {
  const int ix = axis_index(x, g.x0, g.inv_dx, g.nx);
  int d = 0;
#pragma unroll
  for (int w = 1; w < kMaxWorld; ++w) d += ix >= w * slab_width;
  return d;
}

// Staged tiles are written eight consecutive places per thread, which would put
// eight lanes of a warp on every bank; flipping the low three bits of a place by
// bits 5-7 spreads them over all 32 banks, for the quad reads as well.
__device__ __forceinline__ int swizzle(int p) { return p ^ ((p >> 5) & 7); }

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

// One warp counts one tile of 2048 particles: eight rounds of 32 lanes x 8
// particles, per-lane counts of the eight destinations packed 16 bits apart
// (at most 64 per lane, 2048 per warp), summed over the warp with four
// hardware reductions.  No shared memory and no block barrier; a warp walks
// over tiles grid-wide, so the kernel streams x at memory speed.
__global__ void __launch_bounds__(kSlabThreads)
slab_count_kernel(const float* __restrict__ x, const float* __restrict__ vx, PushSpec push,
                  int64_t n, AetherGrid g, int slab_width, int world, bool vec, int tiles,
                  uint32_t* __restrict__ tile_count) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kSlabThreads / 32;
  const int warp_global = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int warp_stride = gridDim.x * warps_per_block;
  for (int tile = warp_global; tile < tiles; tile += warp_stride) {
    uint32_t packed[4] = {0, 0, 0, 0};  // destinations (0,1) (2,3) (4,5) (6,7)
    const int64_t tile_first = static_cast<int64_t>(tile) * kSlabTile;
#pragma unroll
    for (int round = 0; round < kSlabTile / (32 * kSlabItems); ++round) {
      const int64_t i0 = tile_first + (static_cast<int64_t>(round) * 32 + lane) * kSlabItems;
      if (i0 >= n) continue;
      float px[kSlabItems];
      load8(x, i0, n, vec, px);
      if (push.enabled) {  // the destination of the particle as the fused move stage leaves it
        float w[kSlabItems];
        load8(vx, i0, n, vec, w);
#pragma unroll
        for (int k = 0; k < kSlabItems; ++k) push_axis(px[k], w[k], push.dt, push.lo[0], push.hi[0]);
      }
#pragma unroll
      for (int k = 0; k < kSlabItems; ++k)
        if (i0 + k < n) {
          const int d = slab_of(px[k], g, slab_width);
#pragma unroll
          for (int w = 0; w < 4; ++w) packed[w] += (d >> 1) == w ? 1u << (16 * (d & 1)) : 0u;
        }
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) packed[w] = __reduce_add_sync(0xffffffffu, packed[w]);
    if (lane < world) {
      uint32_t word = packed[0];
#pragma unroll
      for (int w = 1; w < 4; ++w) word = (lane >> 1) == w ? packed[w] : word;
      tile_count[static_cast<size_t>(lane) * tiles + tile] = (word >> (16 * (lane & 1))) & 0xffffu;
    }
  }
}

// tile_count is [world][tiles].  Its exclusive scan in that order is the output
// offset of every (destination, tile) run.  Two levels: each block scans 1024
// entries in place and records its total; one block scans the block totals and
// writes the per-destination totals.
constexpr int kScanBlock = 1024;

__global__ void __launch_bounds__(kScanBlock)
slab_scan_local_kernel(uint32_t* __restrict__ tile_count, int64_t entries,
                       uint32_t* __restrict__ block_sum) {
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t total;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kScanBlock + threadIdx.x;
  const uint32_t v = i < entries ? tile_count[i] : 0u;
  const uint32_t excl = block_exclusive_scan(v, warp_sum, &total);
  if (i < entries) tile_count[i] = excl;
  if (threadIdx.x == 0) block_sum[blockIdx.x] = total;
}

// One block: exclusive scan of the block totals (any number of them, 1024 at a
// time with a running carry), then the number of particles per destination.
__global__ void __launch_bounds__(kScanBlock)
slab_scan_blocks_kernel(const uint32_t* __restrict__ tile_count, uint32_t* __restrict__ block_sum,
                        int blocks, int tiles, int world, int64_t n,
                        int64_t* __restrict__ totals) {
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t total, carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < blocks; base += kScanBlock) {
    const int i = base + threadIdx.x;
    const uint32_t v = i < blocks ? block_sum[i] : 0u;
    const uint32_t excl = block_exclusive_scan(v, warp_sum, &total);
    if (i < blocks) block_sum[i] = carry + excl;
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }
  if (threadIdx.x < world) {
    const int64_t first = static_cast<int64_t>(threadIdx.x) * tiles;
    const int64_t begin = tile_count[first] + block_sum[first / kScanBlock];
    int64_t end = n;
    if (threadIdx.x + 1 < world) {
      const int64_t next = first + tiles;
      end = tile_count[next] + block_sum[next / kScanBlock];
    }
    totals[threadIdx.x] = end - begin;
  }
}

// Where each destination's particles go: six arrays per destination.  In the
// local form every destination shares the same six arrays and the position is
// the rank-wide prefix (destination-major).  In the exchange form the arrays are
// the receive buffers of the destination GPUs, written over NVLink, and the
// position is recv_base[d] (what lower ranks send to d) plus the offset inside
// this rank's block for d.
struct SliceFlags {
  uint32_t* peer[kMaxWorld];  // rank d's flag array [world * slices], in rank d's memory
};

struct SlabTargets {
  float* array[kMaxWorld][6];
  const int64_t* count_matrix;  // exchange form: [world][world] on the device, [s][d] = s sends d
  int64_t capacity;             // exchange form: particles a receive buffer holds
  int rank;
  int exchange;
  int aligned;                  // every output array starts on a 16-byte boundary
  int32_t* error;               // exchange form: set to kErrReceiveOverflow if a buffer is too small
};

// Stages the tile in shared memory grouped by destination (stable inside a
// destination), then writes every destination's run with coalesced stores:
// plain stores, to local memory or straight into a peer GPU's memory.
// EAGER: all six arrays of the tile are requested before anything waits (one memory latency
// per tile instead of three, at twice the registers: two blocks per multiprocessor); otherwise
// one axis at a time passes through the registers and four blocks fit.
template <bool EAGER>
__global__ void __launch_bounds__(kSlabThreads, EAGER ? 2 : 4)
slab_scatter_kernel(const float* __restrict__ x, const float* __restrict__ y,
                    const float* __restrict__ z, const float* __restrict__ v, int64_t padded,
                    int64_t n, AetherGrid g, int slab_width, int world, bool vec, int tiles,
                    int tile_begin, int tile_end, const uint32_t* __restrict__ tile_offset,
                    const uint32_t* __restrict__ block_sum, SlabTargets tg, PushSpec push) {
  extern __shared__ float stage_raw[];  // [6][kSlabTile]
  float (*stage)[kSlabTile] = reinterpret_cast<float (*)[kSlabTile]>(stage_raw);
  __shared__ unsigned long long warp_lo[8], warp_hi[8];
  __shared__ uint32_t local_base[kMaxWorld + 1];  // start of each destination's run in the tile
  __shared__ uint32_t out_base[kMaxWorld];        // start of that run in the output arrays
  __shared__ int run_head[kMaxWorld], run_quads[kMaxWorld];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // A block takes tiles tile_begin + blockIdx.x, + gridDim.x, ... of the launch's range of
  // tiles: with fewer blocks than tiles the kernel leaves room on every multiprocessor for the
  // kernels of the local sort that run beside it in the sliced exchange.
  for (int tile = tile_begin + blockIdx.x; tile < tile_end; tile += gridDim.x) {
  const int64_t tile_first = static_cast<int64_t>(tile) * kSlabTile;
  const int64_t i0 = tile_first + static_cast<int64_t>(tid) * kSlabItems;
  // Where this tile's runs go (global reads: started before anything waits on them).
  if (tid < world) {
    const size_t entry = static_cast<size_t>(tid) * tiles + tile;
    uint32_t base = tile_offset[entry] + block_sum[entry / kScanBlock];
    if (tg.exchange) {
      // Receive position: what lower ranks send to destination tid, then this rank's block.
      int64_t lower = 0, all = 0;
      for (int s = 0; s < world; ++s) {
        const int64_t c = tg.count_matrix[s * world + tid];
        if (s < tg.rank) lower += c;
        all += c;
      }
      const size_t first = static_cast<size_t>(tid) * tiles;  // this rank's first tile for tid
      base = base - (tile_offset[first] + block_sum[first / kScanBlock]) +
             static_cast<uint32_t>(lower);
      if (all > tg.capacity) {  // never store past a peer's buffer
        base = 0xffffffffu;
        if (tile == 0) atomicCAS(tg.error, 0, kErrReceiveOverflow);
      }
    }
    out_base[tid] = base;
  }
  // The x pair comes first because the destination depends on it.
  const bool vec_v = vec && padded % 4 == 0;
  float pc[kSlabItems], pw[kSlabItems];
  float later[EAGER ? 4 : 1][kSlabItems];  // EAGER: y, vy, z, vz
  load8(x, i0, n, vec, pc);
  load8(v, i0, n, vec_v, pw);
  if (EAGER) {
    load8(y, i0, n, vec, later[0]);
    load8(v + padded, i0, n, vec_v, later[1]);
    load8(z, i0, n, vec, later[EAGER ? 2 : 0]);
    load8(v + 2 * padded, i0, n, vec_v, later[EAGER ? 3 : 0]);
  }
  if (push.enabled) {  // fused move stage: the particle travels as it is after the move
#pragma unroll
    for (int k = 0; k < kSlabItems; ++k) push_axis(pc[k], pw[k], push.dt, push.lo[0], push.hi[0]);
  }
  int dest[kSlabItems];
  // Per-thread counts of the eight destinations, 16 bits each in two words.
  unsigned long long lo = 0, hi = 0;
#pragma unroll
  for (int k = 0; k < kSlabItems; ++k) {
    dest[k] = i0 + k < n ? slab_of(pc[k], g, slab_width) : -1;
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
  if (tid == kSlabThreads - 1) {
    const unsigned long long all_lo = base_lo + lo, all_hi = base_hi + hi;
    uint32_t run = 0;
    for (int w = 0; w < kMaxWorld; ++w) {
      local_base[w] = run;
      run += static_cast<uint32_t>(((w < 4 ? all_lo : all_hi) >> (16 * (w & 3))) & 0xffffu);
    }
    local_base[kMaxWorld] = run;
  }
  __syncthreads();
  uint32_t next[kMaxWorld];
#pragma unroll
  for (int w = 0; w < kMaxWorld; ++w)
    next[w] = local_base[w] +
              static_cast<uint32_t>(((w < 4 ? base_lo : base_hi) >> (16 * (w & 3))) & 0xffffu);
  int pos[kSlabItems];  // place of each particle in the staged tile, -1 past the end
#pragma unroll
  for (int k = 0; k < kSlabItems; ++k) {
    pos[k] = -1;
    if (dest[k] < 0) continue;
#pragma unroll
    for (int w = 0; w < kMaxWorld; ++w)
      if (dest[k] == w) pos[k] = static_cast<int>(next[w]++);
  }
#pragma unroll
  for (int k = 0; k < kSlabItems; ++k)
    if (pos[k] >= 0) {
      stage[0][swizzle(pos[k])] = pc[k];
      stage[3][swizzle(pos[k])] = pw[k];
    }
#pragma unroll
  for (int axis = 1; axis < 3; ++axis) {
    if (EAGER) {
#pragma unroll
      for (int k = 0; k < kSlabItems; ++k) {
        pc[k] = later[EAGER ? 2 * axis - 2 : 0][k];
        pw[k] = later[EAGER ? 2 * axis - 1 : 0][k];
      }
    } else {
      load8(axis == 1 ? y : z, i0, n, vec, pc);
      load8(v + axis * padded, i0, n, vec_v, pw);
    }
    if (push.enabled) {
#pragma unroll
      for (int k = 0; k < kSlabItems; ++k)
        push_axis(pc[k], pw[k], push.dt, push.lo[axis], push.hi[axis]);
    }
#pragma unroll
    for (int k = 0; k < kSlabItems; ++k)
      if (pos[k] >= 0) {
        stage[axis][swizzle(pos[k])] = pc[k];
        stage[3 + axis][swizzle(pos[k])] = pw[k];
      }
  }
  __syncthreads();
  // Write every destination's run: 16-byte stores over the part of the run whose
  // destination is 16-byte aligned (longer NVLink and HBM bursts), scalar stores for
  // the up to three elements before and after it.  The quads of all destinations
  // form one list that the block's threads share, so that short runs (eight
  // destinations) keep every thread storing.
  if (tid < world) {
    const int lb = static_cast<int>(local_base[tid]), le = static_cast<int>(local_base[tid + 1]);
    int head = 0, quads = 0;
    if (out_base[tid] != 0xffffffffu && le > lb) {
      head = tg.aligned ? min(le - lb, static_cast<int>((4 - (out_base[tid] & 3)) & 3)) : le - lb;
      quads = (le - lb - head) / 4;
    } else if (out_base[tid] == 0xffffffffu) {
      head = -1;  // nothing of this run is written
    }
    run_head[tid] = head;
    run_quads[tid] = quads;
  }
  __syncthreads();
  int quad_first[kMaxWorld + 1];
  quad_first[0] = 0;
#pragma unroll
  for (int d = 0; d < kMaxWorld; ++d) quad_first[d + 1] = quad_first[d] + (d < world ? run_quads[d] : 0);
  for (int q = tid; q < quad_first[kMaxWorld]; q += kSlabThreads) {
    int d = 0;
#pragma unroll
    for (int w = 1; w < kMaxWorld; ++w) d += q >= quad_first[w];
    const int lb = static_cast<int>(local_base[d]);
    const int j = lb + run_head[d] + 4 * (q - quad_first[d]);
    const size_t o = static_cast<size_t>(out_base[d]) + (j - lb);
#pragma unroll
    for (int c = 0; c < 6; ++c) {
      const float4 quad = make_float4(stage[c][swizzle(j)], stage[c][swizzle(j + 1)],
                                      stage[c][swizzle(j + 2)], stage[c][swizzle(j + 3)]);
      *reinterpret_cast<float4*>(tg.array[d][c] + o) = quad;  // (streaming stores: no gain)
    }
  }
  // Heads and tails: at most three elements each per destination when aligned;
  // the whole run when the buffers are not 16-byte aligned.
  for (int d = 0; d < world; ++d) {
    const int head = run_head[d];
    if (head < 0) continue;
    const int lb = static_cast<int>(local_base[d]), le = static_cast<int>(local_base[d + 1]);
    const size_t g0 = out_base[d];
    const int tail_first = lb + head + 4 * run_quads[d];
    for (int i = tid; i < head; i += kSlabThreads) {
#pragma unroll
      for (int c = 0; c < 6; ++c) tg.array[d][c][g0 + i] = stage[c][swizzle(lb + i)];
    }
    for (int j = tail_first + tid; j < le; j += kSlabThreads) {
#pragma unroll
      for (int c = 0; c < 6; ++c) tg.array[d][c][g0 + (j - lb)] = stage[c][swizzle(j)];
    }
  }
  __syncthreads();  // the staged tile and the run tables are reused by the block's next tile
  }
}

// Tells every destination that this rank's slice `slice` of step `epoch` is stored: word
// [rank * slices + slice] of rank d's flag array.  Launched behind the exchange kernel of the
// slice in the same stream: a kernel is complete only when its stores, to whichever GPU, are
// performed, so the flag can never overtake the data.
__global__ void __launch_bounds__(32)
slab_signal_kernel(SliceFlags flags, int world, int rank, int slices, int slice, uint32_t epoch) {
  const int d = threadIdx.x;
  if (d >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.peer[d] + rank * slices + slice),
               "r"(epoch) : "memory");
}

// Particles per (slice, destination) from the scanned tile offsets: slice k is the tiles
// [k * tiles_per_slice, (k + 1) * tiles_per_slice) of this rank's input.
__global__ void __launch_bounds__(256)
slab_slice_counts_kernel(const uint32_t* __restrict__ tile_offset,
                         const uint32_t* __restrict__ block_sum, int tiles, int world, int slices,
                         int tiles_per_slice, int64_t n, int64_t* __restrict__ slice_counts) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= slices * world) return;
  const int k = i / world, d = i % world;
  auto offset = [&](int tile) -> int64_t {  // particles for destinations < d, and for d in tiles < tile
    const int64_t entry = static_cast<int64_t>(d) * tiles + tile;  // (d, tiles) is (d + 1, 0)
    if (entry >= static_cast<int64_t>(world) * tiles) return n;
    return static_cast<int64_t>(tile_offset[entry]) + block_sum[entry / kScanBlock];
  };
  const int lo = min(tiles, k * tiles_per_slice), hi = min(tiles, (k + 1) * tiles_per_slice);
  slice_counts[i] = offset(hi) - offset(lo);
}

// Waits (bounded) until every source rank has signalled slice `slice` of step `epoch`: one
// lane per source polls its flag in this GPU's own memory.  A wait that runs out records
// kErrExchangeTimeout and returns; the kernels behind it then work on incomplete data and
// the caller must discard the step.
__global__ void __launch_bounds__(32)
slab_wait_kernel(const uint32_t* __restrict__ flags, int world, int slices, int slice,
                 uint32_t epoch, uint32_t poll_limit, int32_t* __restrict__ error) {
  const int s = threadIdx.x;
  if (s >= world) return;
  const uint32_t* flag = flags + s * slices + slice;
  for (uint32_t polls = 0;; ++polls) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (static_cast<int32_t>(seen - epoch) >= 0) return;  // epochs only grow (wrap-safe compare)
    if (polls >= poll_limit) break;
    __nanosleep(256);
  }
  atomicCAS(error, 0, kErrExchangeTimeout);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

size_t slab_partition_workspace_bytes(int64_t n, int world) {
  const int64_t tiles = std::max<int64_t>(1, (n + kSlabTile - 1) / kSlabTile);
  const int64_t entries = tiles * world;
  const int64_t blocks = (entries + kScanBlock - 1) / kScanBlock;
  return static_cast<size_t>(align_up(entries * sizeof(uint32_t), 256) +
                             align_up(blocks * sizeof(uint32_t), 256));
}

namespace {

// Counts and scans: leaves the (destination, tile) offsets in the workspace and
// the per-destination totals in `totals`.
cudaError_t slab_count(const float* x, const float* vx, const PushSpec& push, int64_t n,
                       const AetherGrid& g, int world, bool vec, int64_t* totals, void* workspace,
                       cudaStream_t stream) {
  const int tiles = static_cast<int>(std::max<int64_t>(1, (n + kSlabTile - 1) / kSlabTile));
  uint32_t* tile_count = static_cast<uint32_t*>(workspace);
  const int64_t entries = static_cast<int64_t>(tiles) * world;
  const int blocks = static_cast<int>((entries + kScanBlock - 1) / kScanBlock);
  uint32_t* block_sum = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(workspace) +
                                                    align_up(entries * sizeof(uint32_t), 256));
  const int count_grid = std::max(1, std::min((tiles + kSlabThreads / 32 - 1) / (kSlabThreads / 32),
                                              sm_count() * 8));
  slab_count_kernel<<<count_grid, kSlabThreads, 0, stream>>>(x, vx, push, n, g, g.nx / world, world,
                                                             vec, tiles, tile_count);
  slab_scan_local_kernel<<<blocks, kScanBlock, 0, stream>>>(tile_count, entries, block_sum);
  slab_scan_blocks_kernel<<<1, kScanBlock, 0, stream>>>(tile_count, block_sum, blocks, tiles, world,
                                                        n, totals);
  count_launches(3);
  return cudaGetLastError();
}

// Resident blocks of the exchange kernel per multiprocessor in the sliced exchange (1..4), or
// 0 for one block per tile.
int g_exchange_blocks_per_sm = 2;
int exchange_blocks_per_sm() { return g_exchange_blocks_per_sm; }

cudaError_t slab_scatter(const float* x, const float* y, const float* z, const float* v,
                         int64_t padded, int64_t n, const AetherGrid& g, int world, bool vec,
                         const SlabTargets& tg, const PushSpec& push, void* workspace,
                         cudaStream_t stream, int slices = 0, int slice = 0) {
  const int tiles = static_cast<int>(std::max<int64_t>(1, (n + kSlabTile - 1) / kSlabTile));
  uint32_t* tile_count = static_cast<uint32_t*>(workspace);
  const int64_t entries = static_cast<int64_t>(tiles) * world;
  uint32_t* block_sum = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(workspace) +
                                                    align_up(entries * sizeof(uint32_t), 256));
  constexpr int kStageBytes = 6 * kSlabTile * sizeof(float);
  // Alone on the GPU (the one-piece exchange, or a plain partition) the kernel wants every
  // load of a tile in flight at once; beside the local sort it keeps to few registers.
  const bool eager = slices <= 1;
  auto kernel = eager ? slab_scatter_kernel<true> : slab_scatter_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kStageBytes);
  if (e != cudaSuccess) return e;
  // The whole input, or the tiles of one slice.  Blocks per multiprocessor: all four that fit
  // when the kernel runs alone; fewer in the sliced exchange, where the local sort's kernels
  // work beside it on what has arrived.
  int tile_begin = 0, tile_end = tiles;
  if (slices > 0) {
    const int tiles_per_slice = (tiles + slices - 1) / slices;
    tile_begin = std::min(tiles, slice * tiles_per_slice);
    tile_end = std::min(tiles, tile_begin + tiles_per_slice);
  }
  if (tile_end == tile_begin) return cudaSuccess;  // a slice without tiles
  const int per_sm = eager ? 2 : exchange_blocks_per_sm();
  // per_sm 0: one block per tile (blocks come and go, so that a kernel of higher priority
  // takes the multiprocessors over as they retire).
  const int grid = per_sm > 0 ? std::min(tile_end - tile_begin, sm_count() * per_sm)
                              : tile_end - tile_begin;
  kernel<<<grid, kSlabThreads, kStageBytes, stream>>>(
      x, y, z, v, padded, n, g, g.nx / world, world, vec, tiles, tile_begin, tile_end, tile_count,
      block_sum, tg, push);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace

cudaError_t slab_partition(const float* x, const float* y, const float* z, const float* v,
                           int64_t padded, int64_t n, const AetherGrid& g, int world, float* ox,
                           float* oy, float* oz, float* ovx, float* ovy, float* ovz,
                           int64_t* totals, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  if (world < 1 || world > kMaxWorld || g.nx % world != 0) return cudaErrorInvalidValue;
  if (workspace_bytes < slab_partition_workspace_bytes(n, world)) return cudaErrorInvalidValue;
  const bool vec = aligned16(x) && aligned16(y) && aligned16(z) && aligned16(v);
  stage_begin(kStageSlabPartition, stream);
  cudaError_t e = slab_count(x, nullptr, PushSpec{}, n, g, world, vec, totals, workspace, stream);
  if (e != cudaSuccess) return e;
  SlabTargets tg{};
  for (int d = 0; d < world; ++d) {
    float* arrays[6] = {ox, oy, oz, ovx, ovy, ovz};
    for (int c = 0; c < 6; ++c) tg.array[d][c] = arrays[c];
  }
  tg.aligned = aligned16(ox) && aligned16(oy) && aligned16(oz) && aligned16(ovx) &&
               aligned16(ovy) && aligned16(ovz);
  e = slab_scatter(x, y, z, v, padded, n, g, world, vec, tg, PushSpec{}, workspace, stream);
  stage_end(kStageSlabPartition, stream);
  return e;
}

// The two halves of the fused partition + exchange: count, then (after the
// ranks have exchanged their counts) scatter straight into the peers' buffers.
cudaError_t slab_exchange_count(const float* x, const float* vx, const PushSpec& push, int64_t n,
                                const AetherGrid& g, int world, int64_t* totals, void* workspace,
                                size_t workspace_bytes, cudaStream_t stream) {
  if (push.enabled && n > 0 && !vx) return cudaErrorInvalidValue;
  if (world < 1 || world > kMaxWorld || g.nx % world != 0) return cudaErrorInvalidValue;
  if (workspace_bytes < slab_partition_workspace_bytes(n, world)) return cudaErrorInvalidValue;
  stage_begin(kStageSlabPartition, stream);
  const bool vec = aligned16(x) && (!push.enabled || aligned16(vx));
  cudaError_t e = slab_count(x, vx, push, n, g, world, vec, totals, workspace, stream);
  stage_end(kStageSlabPartition, stream);
  return e;
}

namespace {
// One thread: the sums are over at most kMaxWorld * kMaxSlices small numbers.
__global__ void slab_prepare_kernel(const int64_t* __restrict__ matrix, int world, int slices,
                                    int rank, int64_t* __restrict__ totals2d,
                                    SliceSegments* __restrict__ seg) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  auto m = [&](int s, int k, int d) { return matrix[(static_cast<int64_t>(s) * slices + k) * world + d]; };
  for (int s = 0; s < world; ++s)
    for (int d = 0; d < world; ++d) {
      int64_t sum = 0;
      for (int k = 0; k < slices; ++k) sum += m(s, k, d);
      totals2d[s * world + d] = sum;
    }
  uint32_t before = 0;  // particles of lower sources
  for (int s = 0; s < world; ++s) {
    uint32_t run = before;
    for (int k = 0; k < slices; ++k) {
      seg->first[k][s] = run;
      seg->length[k][s] = static_cast<uint32_t>(m(s, k, rank));
      run += static_cast<uint32_t>(m(s, k, rank));
    }
    before = run;
  }
  uint32_t base = 0;
  for (int k = 0; k < slices; ++k) {
    seg->chunk_base[k] = base;
    for (int s = 0; s < world; ++s) base += static_cast<uint32_t>(m(s, k, rank));
  }
  seg->chunk_base[slices] = base;
  seg->n = base;
  seg->slices = static_cast<uint32_t>(slices);
  seg->sources = static_cast<uint32_t>(world);
  seg->pad = 0;
}

int slab_tiles(int64_t n) {
  return static_cast<int>(std::max<int64_t>(1, (n + kSlabTile - 1) / kSlabTile));
}
}  // namespace

void slab_exchange_set_blocks_per_sm(int blocks) {
  g_exchange_blocks_per_sm = std::max(0, std::min(4, blocks));
}

cudaError_t slab_exchange_prepare(const int64_t* matrix, int world, int slices, int rank,
                                  int64_t* totals2d, SliceSegments* segments, cudaStream_t stream) {
  if (!matrix || !totals2d || !segments || world < 1 || world > kMaxWorld || slices < 1 ||
      slices > kMaxSlices || rank < 0 || rank >= world)
    return cudaErrorInvalidValue;
  slab_prepare_kernel<<<1, 32, 0, stream>>>(matrix, world, slices, rank, totals2d, segments);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t slab_exchange_slice_counts(int64_t n, int world, int slices, int64_t* slice_counts,
                                       void* workspace, size_t workspace_bytes,
                                       cudaStream_t stream) {
  if (world < 1 || world > kMaxWorld || slices < 1 || slices > kMaxSlices || !slice_counts)
    return cudaErrorInvalidValue;
  if (workspace_bytes < slab_partition_workspace_bytes(n, world)) return cudaErrorInvalidValue;
  const int tiles = slab_tiles(n);
  const int64_t entries = static_cast<int64_t>(tiles) * world;
  const uint32_t* tile_offset = static_cast<const uint32_t*>(workspace);
  const uint32_t* block_sum = reinterpret_cast<const uint32_t*>(
      static_cast<const unsigned char*>(workspace) + align_up(entries * sizeof(uint32_t), 256));
  const int tiles_per_slice = (tiles + slices - 1) / slices;
  slab_slice_counts_kernel<<<(slices * world + 255) / 256, 256, 0, stream>>>(
      tile_offset, block_sum, tiles, world, slices, tiles_per_slice, n, slice_counts);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t slab_wait_slice(const uint32_t* flags, int world, int slices, int slice, uint32_t epoch,
                            uint32_t poll_limit, int32_t* error, cudaStream_t stream) {
  if (!flags || !error || world < 1 || world > kMaxWorld || slices < 1 || slices > kMaxSlices ||
      slice < 0 || slice >= slices)
    return cudaErrorInvalidValue;
  slab_wait_kernel<<<1, 32, 0, stream>>>(flags, world, slices, slice, epoch, poll_limit, error);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t slab_signal_slice(int world, int rank, int slices, int slice, uint32_t epoch,
                              uint32_t* const* peer_flags, cudaStream_t stream) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || slices < 1 ||
      slices > kMaxSlices || slice < 0 || slice >= slices || !peer_flags)
    return cudaErrorInvalidValue;
  SliceFlags flags{};
  for (int d = 0; d < world; ++d) {
    if (!peer_flags[d]) return cudaErrorInvalidValue;
    flags.peer[d] = peer_flags[d];
  }
  slab_signal_kernel<<<1, 32, 0, stream>>>(flags, world, rank, slices, slice, epoch);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t slab_exchange_scatter(const float* x, const float* y, const float* z, const float* v,
                                  int64_t padded, int64_t n, const AetherGrid& g, int world,
                                  int rank, float* const* peer_buffers, int64_t capacity,
                                  const int64_t* count_matrix, int32_t* error,
                                  const PushSpec& push, void* workspace, size_t workspace_bytes,
                                  cudaStream_t stream, const SliceSignal* signal) {
  if (world < 1 || world > kMaxWorld || g.nx % world != 0) return cudaErrorInvalidValue;
  if (rank < 0 || rank >= world || !count_matrix || !error) return cudaErrorInvalidValue;
  if (workspace_bytes < slab_partition_workspace_bytes(n, world)) return cudaErrorInvalidValue;
  SlabTargets tg{};
  if (signal && (signal->slices < 1 || signal->slices > kMaxSlices || signal->slice < 0 ||
                 signal->slice >= signal->slices || !signal->peer_flags))
    return cudaErrorInvalidValue;
  tg.exchange = 1;
  tg.count_matrix = count_matrix;
  tg.capacity = capacity;
  tg.rank = rank;
  tg.error = error;
  for (int d = 0; d < world; ++d) {
    if (!peer_buffers[d]) return cudaErrorInvalidValue;
    for (int c = 0; c < 6; ++c) tg.array[d][c] = peer_buffers[d] + static_cast<size_t>(c) * capacity;
    tg.aligned = (d == 0 ? 1 : tg.aligned) && aligned16(peer_buffers[d]);
  }
  const bool vec = aligned16(x) && aligned16(y) && aligned16(z) && aligned16(v);
  stage_begin(kStageSlabExchange, stream);
  cudaError_t e = slab_scatter(x, y, z, v, padded, n, g, world, vec, tg, push, workspace, stream,
                               signal ? signal->slices : 0, signal ? signal->slice : 0);
  if (e == cudaSuccess && signal) {
    SliceFlags flags{};
    for (int d = 0; d < world; ++d) {
      if (!signal->peer_flags[d]) return cudaErrorInvalidValue;
      flags.peer[d] = signal->peer_flags[d];
    }
    slab_signal_kernel<<<1, 32, 0, stream>>>(flags, world, rank, signal->slices, signal->slice,
                                             signal->epoch);
    count_launches(1);
    e = cudaGetLastError();
  }
  stage_end(kStageSlabExchange, stream);
  return e;
}

}  // namespace aether
