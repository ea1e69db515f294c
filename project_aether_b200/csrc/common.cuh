// Shared device helpers of the particle sort: key generation (cell id from
// float32 positions and Philox4x32-10 shuffle bits), small PTX wrappers and the
// workspace layout.  sm_100a only.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/aether_sort.h"

namespace aether {

constexpr int kShuffleBits = 7;  // radix_sort_reference.py:33
constexpr int kRadixBits = 8;    // digit width of this implementation
constexpr int kRadix = 1 << kRadixBits;
constexpr int kMaxPasses = 4;    // 32-bit keys / 8-bit digits

// Status word of the chained scan: flag in bits 30-31, count in bits 0-29.
// (The reference packs a 2-bit flag over a 29-bit count into a signed word,
// radix_sort_reference.py:36-40; the unsigned form here leaves 30 value bits.)
constexpr uint32_t kFlagAggregate = 1u << 30;
constexpr uint32_t kFlagInclusive = 2u << 30;
constexpr uint32_t kFlagMask = 3u << 30;
constexpr uint32_t kValueMask = ~kFlagMask;

// Error codes left in the workspace header by a device wait that gave up.
constexpr int kErrLookbackTimeout = 1;
constexpr int kErrBucketOverflow = 2;
constexpr int kErrBulkCopyTimeout = 3;
constexpr int kErrReceiveOverflow = 5;
constexpr int kErrExchangeTimeout = 6;

constexpr int kMaxWorld = 8;    // ranks of the multi-GPU decomposition
constexpr int kMaxSlices = 32;  // slices of one rank's input in the sliced exchange

// What a rank receives in the sliced exchange, slice by slice (device memory, written by
// slab_exchange_prepare).  The received array is the concatenation over sources s of what s
// sent, in s's order; source s's slice k occupies [first[k][s], first[k][s] + length[k][s]).
// The local sort lays its records out with one chunk per slice: chunk k's records start at
// chunk_base[k] (the particles of all sources' slices before k).
struct SliceSegments {
  uint32_t n;        // particles received in all
  uint32_t slices;
  uint32_t sources;
  uint32_t pad;
  uint32_t chunk_base[kMaxSlices + 1];
  uint32_t first[kMaxSlices][kMaxWorld];
  uint32_t length[kMaxSlices][kMaxWorld];
};

// Workspace header (first 1 KiB of the workspace, zeroed by every call).
struct alignas(16) Header {
  int32_t error;              // first error code seen, 0 when clean
  int32_t use_standard;       // bucketed path: 1 when it handed over to the digit passes
  uint32_t tile_counter[kMaxPasses];  // ticket dispenser of each digit pass
  uint32_t aux_counter[8];
  uint32_t max_bucket;        // bucketed path: largest bucket seen
  uint32_t pad[49];
  uint32_t digit_hist[kMaxPasses][kRadix];  // global digit histograms (upsweep)
};
static_assert(sizeof(Header) % 256 == 0, "header must keep 256-byte alignment");

__host__ __device__ inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Word 0 of Philox4x32-10 with counter (c0, 0, 0, 0) and key (k0, k1): the
// value tl.randint(seed, i) gives the reference's key kernel
// (fused_radix_sort.py:101), restated after the reference's own generator
// (cuda/philox.h:56-72).  The zero counter words let the first two rounds and
// the unused outputs of the last round fold away at compile time.
__device__ __forceinline__ uint32_t philox_word0(uint32_t c0, uint32_t k0, uint32_t k1) {
  constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u;
  constexpr uint32_t kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
  uint32_t c1 = 0, c2 = 0, c3 = 0;
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
  return c0;
}

// clamp(int32_rz((c - lo) * inv), 0, cells - 1) with separately rounded
// subtract and multiply (fused_radix_sort.py:93-98).  The intrinsics keep the
// compiler from contracting the pair into a fused multiply-add.
__device__ __forceinline__ int axis_index(float c, float lo, float inv, int cells) {
  const int i = __float2int_rz(__fmul_rn(__fsub_rn(c, lo), inv));
  return min(max(i, 0), cells - 1);
}

// Cell id over the x-slab [ix_offset, ix_offset + nx_local) of the grid.  A particle whose
// column lies outside the slab (the caller's precondition broken) is binned into the slab's
// nearest column: every table the kernels index with a cell id stays in range.
__device__ __forceinline__ uint32_t cell_of(float x, float y, float z, const AetherGrid& g) {
  const int ix = axis_index(x, g.x0, g.inv_dx, g.nx);
  const int iy = axis_index(y, g.y0, g.inv_dy, g.ny);
  const int iz = axis_index(z, g.z0, g.inv_dz, g.nz);
  const int ix_local = min(max(ix - g.ix_offset, 0), g.nx_local - 1);
  return static_cast<uint32_t>((iz * g.ny + iy) * g.nx_local + ix_local);
}

__device__ __forceinline__ uint32_t make_key(uint32_t cell, uint32_t index, uint32_t k0,
                                             uint32_t k1) {
  return (cell << kShuffleBits) | (philox_word0(index, k0, k1) >> (32 - kShuffleBits));
}

__device__ __forceinline__ uint32_t ld_relaxed(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Adds one to a histogram bin per lane.  Lanes hitting the same bin share one add
// when the whole warp agrees, or (through match.any) when neighbouring lanes do.
__device__ __forceinline__ void bin_add(uint32_t* hist, uint32_t bin, bool valid) {
  const uint32_t active = __ballot_sync(0xffffffffu, valid);
  if (active == 0) return;
  const int first = __ffs(active) - 1;
  const uint32_t first_bin = __shfl_sync(0xffffffffu, bin, first);
  const bool uniform = __all_sync(0xffffffffu, !valid || bin == first_bin);
  if (uniform) {
    if (static_cast<int>(lane_id()) == first) atomicAdd(&hist[first_bin], __popc(active));
    return;
  }
  const uint32_t next_bin = __shfl_down_sync(0xffffffffu, bin, 1);
  const bool clustered = __any_sync(0xffffffffu, valid && lane_id() < 31 && next_bin == bin);
  if (clustered) {
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? bin : 0xffffffffu) & active;
    if (valid && (peers & lanemask_lt()) == 0) atomicAdd(&hist[bin], __popc(peers));
  } else if (valid) {
    atomicAdd(&hist[bin], 1u);
  }
}

// Exclusive scan of one value per thread over a block of up to 1024 threads;
// `warp_sum` is 32 words of shared memory, *total receives the block's sum.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_sum,
                                                         uint32_t* total) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t w = lane < static_cast<int>((blockDim.x + 31) >> 5) ? warp_sum[lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_sum[lane] = wi - w;
    if (lane == 31) *total = wi;
  }
  __syncthreads();
  return warp_sum[warp] + incl - v;
}

// Streaming (read-once / write-once) accesses: keep them from displacing data
// that is reused out of L2.
__device__ __forceinline__ float4 ldcs4(const float* p) {
  return __ldcs(reinterpret_cast<const float4*>(p));
}

// ---- measurement hooks (api.cu) ----
enum Stage {
  kStageKeygen = 0, kStagePass0, kStagePass1, kStagePass2, kStagePass3, kStageCellTables,
  kStageGather, kStageBucketCount, kStageBucketScan, kStageBucketScatter, kStageBucketFinish,
  kStageSlabPartition, kStagePush, kStageSlabExchange, kStageCollide, kNumStages
};
// Multiprocessors of the current device (queried once per device).
int sm_count();
void stage_begin(Stage s, cudaStream_t stream);
void stage_end(Stage s, cudaStream_t stream);
void stage_reset();
void count_launches(int kernels);

// Chained launches.  The kernels of one sort call run one after the other on one stream, two
// dozen of them, and the gaps between them (the next kernel's launch begins when the previous
// grid has drained) are most of what a small call costs.  A kernel launched with
// launch_chained may be set up while its predecessor still runs: every kernel of the chain
// begins with chain_begin(), which lets the kernel behind it start its launch
// (griddepcontrol.launch_dependents) and then waits until the grids before it are complete
// and their memory visible (griddepcontrol.wait).  Nothing of a kernel's work moves ahead of
// that wait, so the order of the work is that of the stream.  Launched in the ordinary way
// the same kernels find nothing to wait for.  Measured per sort, ordinary launches / short
// kernels chained / all chained: 1 M particles 0.161 / 0.137 / 0.141 ms, 16 M 0.641 / 0.601 /
// 0.613, 64 M 2.312 / 2.273 / 2.378, 128 M (steady state) 3.745 / 3.706 / 3.724.
__device__ __forceinline__ void chain_begin() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

int chained_launches();            // process-wide: 0 none, 1 the short kernels, 2 all
void set_chained_launches(int mode);

// `heavy`: a kernel that fills the multiprocessors for a long time (scatter, finish); chained
// only in mode 2.
template <bool HEAVY = false, class... Params, class... Args>
cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes,
                           cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = chained_launches() >= (HEAVY ? 2 : 1) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// ---- host-side launchers of the kernels (one translation unit each) ----

// Optional move stage fused into the sort: the sort sees every particle at
// c + v*dt with specular reflection at lo/hi, and the sorted payload carries
// the moved positions and the reflected velocities; the inputs stay as they are.
struct PushSpec {
  int enabled;
  float dt;
  float lo[3], hi[3];
};

// x += v*dt and reflection at the two walls of one axis, in float32 with a rounded
// multiply and a rounded add (fused_particle_push.py:36-44, reference_push :95-108).
// Both wall tests look at the moved coordinate before any reflection.
__device__ __forceinline__ void push_axis(float& c, float& v, float dt, float lo, float hi) {
  c = __fadd_rn(c, __fmul_rn(v, dt));
  const bool below = c < lo, above = c > hi;
  if (below) c = __fsub_rn(__fmul_rn(2.0f, lo), c);
  if (above) c = __fsub_rn(__fmul_rn(2.0f, hi), c);
  if (below || above) v = -v;
}

struct SortArgs {
  const float *x, *y, *z, *velocity;
  int64_t padded, n;
  AetherGrid grid;
  uint64_t seed;
  uint32_t* keys_out;
  int32_t* index_out;
  int32_t *cell_counts, *cell_start;
  float *xs, *ys, *zs, *vs;
  int64_t padded_sorted;
  int64_t num_cells;
  int key_bits;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
  PushSpec push;
};

size_t standard_workspace_bytes(int64_t n, int64_t num_cells);
size_t standard_workspace_bytes_with_records(int64_t n, int64_t num_cells);
// `run_if`: device flag; when not null the kernels do nothing unless it is
// nonzero (the hand-over from the bucketed path), and the first 8 bytes of the
// workspace header (error code and that flag) are left as they are.
cudaError_t standard_sort(const SortArgs& a, const int32_t* run_if);

// One digit pass over three tiles of zero keys with the ticket dispenser started at 1: the
// tile that would publish first is never processed, so every look-back runs out of polls,
// records kErrLookbackTimeout in the workspace header and returns.  For tests of the give-up
// path; `workspace` needs lookback_probe_workspace_bytes() bytes.
cudaError_t lookback_give_up_probe(void* workspace, size_t workspace_bytes, uint32_t poll_limit,
                                   cudaStream_t stream);
int64_t lookback_probe_particles();
size_t lookback_probe_workspace_bytes();

struct BucketPlan {
  int shift;          // a bucket is 2^shift consecutive cell ids
  int64_t buckets;
  bool usable;        // false when even single-cell buckets would be too full on average
  bool small_blocks;  // finish kernel shape: two small blocks per multiprocessor, or one large
};
BucketPlan plan_buckets(int64_t n, int64_t num_cells);
// Most buckets for which the small finish shape is planned (at most 32,768; 0: never).
void set_small_shape_buckets(int64_t buckets);
// Most records of a group of buckets (what one block of the finish kernel sorts at a time).
uint32_t bucket_group_capacity(int64_t n, const BucketPlan& p);
size_t bucketed_workspace_bytes(int64_t n, int64_t num_cells);
cudaError_t bucketed_sort(const SortArgs& a, const BucketPlan& p);

// The bucketed sort of a segmented input, slice by slice (the local sort of the sliced
// multi-GPU exchange): a.n is the CAPACITY of the input arrays, the particle count and the
// segments are read on the device; the bucket plan is made for plan_n particles.
// begin: clears the tables.  slice k: counts, scans and scatters the particles of slice k
// (every source's segment) into chunk k.  finish: bucket starts, groups, and the finish
// kernels; uses a.keys_out ... a.vs.
size_t sliced_sort_workspace_bytes(int64_t capacity, int64_t plan_n, int64_t num_cells, int slices);
cudaError_t sliced_sort_begin(const SortArgs& a, int64_t plan_n, int slices);
cudaError_t sliced_sort_slice(const SortArgs& a, int64_t plan_n, const SliceSegments* segments,
                              int slices, int slice);
cudaError_t sliced_sort_finish(const SortArgs& a, int64_t plan_n, const SliceSegments* segments,
                               int slices);

size_t slab_partition_workspace_bytes(int64_t n, int world);
cudaError_t slab_partition(const float* x, const float* y, const float* z, const float* v,
                           int64_t padded, int64_t n, const AetherGrid& g, int world, float* ox,
                           float* oy, float* oz, float* ovx, float* ovy, float* ovz,
                           int64_t* totals, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream);
cudaError_t launch_make_keys(const float* x, const float* y, const float* z, int64_t n,
                             const AetherGrid& g, uint64_t seed, uint32_t* keys,
                             cudaStream_t stream);
cudaError_t launch_gather(const int32_t* index, int64_t n, const float* x, const float* y,
                          const float* z, const float* velocity, int64_t padded, float* xs,
                          float* ys, float* zs, float* vs, int64_t padded_sorted,
                          cudaStream_t stream, const int32_t* run_if = nullptr);
cudaError_t launch_cell_tables(const uint32_t* sorted_keys, int64_t n, int64_t num_cells,
                               int32_t* cell_counts, int32_t* cell_start, cudaStream_t stream,
                               const int32_t* run_if = nullptr);

cudaError_t slab_exchange_count(const float* x, const float* vx, const PushSpec& push, int64_t n,
                                const AetherGrid& g, int world, int64_t* totals, void* workspace,
                                size_t workspace_bytes, cudaStream_t stream);
// Sliced exchange: one call stores the tiles of one slice and then tells every destination.
struct SliceSignal {
  int slices;
  int slice;
  uint32_t epoch;
  uint32_t* const* peer_flags;    // [world] host array: rank d's flag array [world * slices]
};
cudaError_t slab_exchange_scatter(const float* x, const float* y, const float* z, const float* v,
                                  int64_t padded, int64_t n, const AetherGrid& g, int world,
                                  int rank, float* const* peer_buffers, int64_t capacity,
                                  const int64_t* count_matrix, int32_t* error,
                                  const PushSpec& push, void* workspace, size_t workspace_bytes,
                                  cudaStream_t stream, const SliceSignal* signal = nullptr);
// From the gathered counts matrix[s][k][d] (particles of source s, slice k, for destination d):
// this rank's segment table and the totals totals2d[s][d] the exchange kernel reads.
cudaError_t slab_exchange_prepare(const int64_t* matrix, int world, int slices, int rank,
                                  int64_t* totals2d, SliceSegments* segments, cudaStream_t stream);
void slab_exchange_set_blocks_per_sm(int blocks);
cudaError_t slab_exchange_slice_counts(int64_t n, int world, int slices, int64_t* slice_counts,
                                       void* workspace, size_t workspace_bytes,
                                       cudaStream_t stream);
cudaError_t slab_signal_slice(int world, int rank, int slices, int slice, uint32_t epoch,
                              uint32_t* const* peer_flags, cudaStream_t stream);
cudaError_t slab_wait_slice(const uint32_t* flags, int world, int slices, int slice, uint32_t epoch,
                            uint32_t poll_limit, int32_t* error, cudaStream_t stream);
cudaError_t particle_push(float* x, float* y, float* z, float* vx, float* vy, float* vz, int64_t n,
                          float dt, const float* lo, const float* hi, cudaStream_t stream);
cudaError_t collide_cells(float* velocity, const int* cell_start, float* sigma_g_max,
                          int* collisions, int num_particles, int padded, int num_cells,
                          float selection_factor, float coefficient, float exponent,
                          uint64_t seed, uint64_t step, cudaStream_t stream);

}  // namespace aether
