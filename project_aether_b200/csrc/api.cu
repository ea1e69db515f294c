// extern "C" entry points of libaether_sort.so (declared in include/aether_sort.h).
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace aether {
namespace {

int bit_length(int64_t v) {
  int b = 0;
  while (v > 0) { ++b; v >>= 1; }
  return b;
}

// Bits of (cell << 7 | shuffle); radix_sort_reference.py:62.  The reference
// stops at 31 bits because its keys are signed; keys here are unsigned, so 32
// bits are allowed.
int key_bits_of(int64_t num_cells) {
  const int cb = bit_length(num_cells - 1);
  return (cb < 1 ? 1 : cb) + kShuffleBits;
}

bool grid_ok(const AetherGrid* g) {
  if (!g) return false;
  if (g->nx <= 0 || g->ny <= 0 || g->nz <= 0) return false;
  if (g->nx_local <= 0 || g->ix_offset < 0 || g->ix_offset + g->nx_local > g->nx) return false;
  const int64_t cells = static_cast<int64_t>(g->nx_local) * g->ny * g->nz;
  return cells > 0 && key_bits_of(cells) <= 32;
}

bool count_ok(int64_t n) { return n >= 0 && n < (int64_t{1} << 30); }

int run_sort(SortArgs& a, int path) {
  if (!count_ok(a.n) || !grid_ok(&a.grid)) return cudaErrorInvalidValue;
  if (!a.cell_counts || !a.cell_start || !a.workspace) return cudaErrorInvalidValue;
  if (a.n > 0 && (!a.x || !a.y || !a.z || !a.keys_out || !a.index_out))
    return cudaErrorInvalidValue;
  if (reinterpret_cast<uintptr_t>(a.workspace) & 255) return cudaErrorInvalidValue;
  a.num_cells = static_cast<int64_t>(a.grid.nx_local) * a.grid.ny * a.grid.nz;
  a.key_bits = key_bits_of(a.num_cells);
  stage_reset();
  // path 1 asks for the digit passes; otherwise the bucketed path runs whenever its plan fits
  // (with or without payload outputs) and the workspace is large enough for its records.  A
  // caller with a smaller workspace (the static-scratch entry point above a few hundred
  // thousand particles, or a workspace sized for the digit passes only) gets the digit passes.
  const BucketPlan plan = plan_buckets(a.n, a.num_cells);
  const bool roomy = a.workspace_bytes >= bucketed_workspace_bytes(a.n, a.num_cells);
  const bool bucketed = plan.usable && path != 1 && (roomy || path == 2);
  if (path == 2 && (!plan.usable || !roomy)) return cudaErrorInvalidValue;
  if (!bucketed) return standard_sort(a, nullptr);
  cudaError_t e = bucketed_sort(a, plan);
  if (e != cudaSuccess) return e;
  // Runs only if the device found a bucket the finish kernel cannot hold.
  const Header* hdr = static_cast<const Header*>(a.workspace);
  return standard_sort(a, &hdr->use_standard);
}

}  // namespace
}  // namespace aether

namespace aether {
namespace {
// Stage timing keeps one event pair per stage for each of the last kTimedCalls
// sort calls, so that a benchmark can run its timed calls back to back and read
// the per-stage averages afterwards without a synchronisation in between.
//
// The state below is process-wide and belongs to ONE device: the device that is current when
// AetherSortSetStageTiming(1) is called.  Sort calls on other devices are not timed.  A mutex
// serialises the bookkeeping, so that calls from several host threads stay consistent; the
// figures themselves only mean something when the timed calls come from one thread.
constexpr int kTimedCalls = 32;
std::mutex g_mutex;
int g_timing_device = -1;
bool g_timing = false;
bool g_events_ready = false;
cudaEvent_t g_begin[kTimedCalls][kNumStages], g_end[kTimedCalls][kNumStages];
bool g_ran[kTimedCalls][kNumStages];
int64_t g_call = -1;
uint64_t g_launches = 0;
const char* const kStageNames[kNumStages] = {
    "keygen_upsweep", "digit_pass_0", "digit_pass_1", "digit_pass_2", "digit_pass_3",
    "cell_tables", "payload_gather", "bucket_count", "bucket_scan", "bucket_scatter",
    "bucket_finish", "slab_partition", "particle_push", "slab_exchange", "collide"};
}  // namespace

namespace {
bool timed_here() {
  if (!g_timing) return false;
  int device = -1;
  return cudaGetDevice(&device) == cudaSuccess && device == g_timing_device;
}
}  // namespace

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 148;
  if (cached[device] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        sms <= 0)
      sms = 148;
    cached[device] = sms;
  }
  return cached[device];
}

void stage_reset() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!timed_here()) return;
  ++g_call;
  for (int i = 0; i < kNumStages; ++i) g_ran[g_call % kTimedCalls][i] = false;
}
void stage_begin(Stage s, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!timed_here() || g_call < 0) return;
  if (!g_events_ready) {
    for (int c = 0; c < kTimedCalls; ++c)
      for (int i = 0; i < kNumStages; ++i) {
        cudaEventCreate(&g_begin[c][i]);
        cudaEventCreate(&g_end[c][i]);
      }
    g_events_ready = true;
  }
  cudaEventRecord(g_begin[g_call % kTimedCalls][s], stream);
}
void stage_end(Stage s, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!timed_here() || g_call < 0) return;
  cudaEventRecord(g_end[g_call % kTimedCalls][s], stream);
  g_ran[g_call % kTimedCalls][s] = true;
}
void count_launches(int kernels) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_launches += kernels;
}
}  // namespace aether

using namespace aether;

extern "C" int AetherSortSetStageTiming(int enabled) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (enabled) {
    // The events are created on, and belong to, the device that is current now.
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (g_events_ready && device != g_timing_device) {
      for (int c = 0; c < kTimedCalls; ++c)
        for (int i = 0; i < kNumStages; ++i) {
          cudaEventDestroy(g_begin[c][i]);
          cudaEventDestroy(g_end[c][i]);
        }
      g_events_ready = false;
    }
    g_timing_device = device;
  }
  g_timing = enabled != 0;
  g_call = -1;
  for (int c = 0; c < kTimedCalls; ++c)
    for (int i = 0; i < kNumStages; ++i) g_ran[c][i] = false;
  return 0;
}
extern "C" int AetherSortStageCount(void) { return kNumStages; }
extern "C" const char* AetherSortStageName(int stage) {
  return stage >= 0 && stage < kNumStages ? kStageNames[stage] : "";
}
extern "C" int AetherSortReadStageTimes(float* ms_out, int capacity) {
  if (!ms_out || capacity < kNumStages) return cudaErrorInvalidValue;
  std::lock_guard<std::mutex> lock(g_mutex);
  for (int i = 0; i < kNumStages; ++i) {
    ms_out[i] = -1.f;
    if (!g_events_ready) continue;
    double sum = 0;
    int calls = 0;
    for (int c = 0; c < kTimedCalls; ++c) {
      if (!g_ran[c][i]) continue;
      cudaError_t e = cudaEventSynchronize(g_end[c][i]);
      if (e != cudaSuccess) return e;
      float ms = 0;
      e = cudaEventElapsedTime(&ms, g_begin[c][i], g_end[c][i]);
      if (e != cudaSuccess) return e;
      sum += ms;
      ++calls;
    }
    if (calls) ms_out[i] = static_cast<float>(sum / calls);
  }
  return 0;
}
extern "C" uint64_t AetherSortKernelLaunches(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return g_launches;
}

extern "C" size_t AetherSortProbeLookbackWorkspaceBytes(void) {
  return lookback_probe_workspace_bytes();
}

extern "C" int AetherSortProbeLookbackGiveUp(void* workspace, size_t workspace_bytes,
                                             uint32_t poll_limit, void* stream) {
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255)) return cudaErrorInvalidValue;
  return lookback_give_up_probe(workspace, workspace_bytes, poll_limit,
                                static_cast<cudaStream_t>(stream));
}

extern "C" int AetherSortAbiVersion(void) { return 1; }

extern "C" size_t AetherSortWorkspaceBytes(int64_t n, int64_t num_cells, int with_payload) {
  if (!count_ok(n) || num_cells <= 0 || key_bits_of(num_cells) > 32) return 0;
  // The digit passes gather the payload through 32-byte records when there is room for them.
  const size_t standard = with_payload ? standard_workspace_bytes_with_records(n, num_cells)
                                       : standard_workspace_bytes(n, num_cells);
  return std::max(standard, bucketed_workspace_bytes(n, num_cells));
}

extern "C" int AetherSortBucketPlan(int64_t n, int64_t num_cells, int32_t* cells_per_bucket_log2,
                                    int64_t* buckets, int32_t* group_capacity) {
  if (!count_ok(n) || num_cells <= 0 || key_bits_of(num_cells) > 32) return cudaErrorInvalidValue;
  const BucketPlan plan = plan_buckets(n, num_cells);
  if (cells_per_bucket_log2) *cells_per_bucket_log2 = plan.shift;
  if (buckets) *buckets = plan.buckets;
  if (group_capacity) *group_capacity = static_cast<int32_t>(bucket_group_capacity(n, plan));
  return plan.usable ? 0 : cudaErrorInvalidValue;
}

namespace aether {
namespace {
int g_chained_launches = 1;
}
int chained_launches() { return g_chained_launches; }
void set_chained_launches(int mode) { g_chained_launches = mode; }
}  // namespace aether

extern "C" int AetherSortSetChainedLaunches(int32_t mode) {
  if (mode < 0 || mode > 2) return cudaErrorInvalidValue;
  aether::set_chained_launches(mode);
  return 0;
}

extern "C" int AetherSortSetSmallShapeBucketLimit(int64_t buckets) {
  if (buckets < 0) return cudaErrorInvalidValue;
  set_small_shape_buckets(buckets);
  return 0;
}

extern "C" int AetherSortParticlesByCell(const float* x, const float* y, const float* z,
                                         int64_t n, const AetherGrid* grid, uint64_t seed,
                                         uint32_t* keys_out, int32_t* index_out,
                                         int32_t* cell_counts, int32_t* cell_start,
                                         void* workspace, size_t workspace_bytes, void* stream) {
  if (!grid) return cudaErrorInvalidValue;
  SortArgs a{};
  a.x = x; a.y = y; a.z = z; a.n = n; a.grid = *grid; a.seed = seed;
  a.keys_out = keys_out; a.index_out = index_out;
  a.cell_counts = cell_counts; a.cell_start = cell_start;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return run_sort(a, 0);
}

namespace aether {
namespace {
int sort_and_gather(const float* x, const float* y, const float* z, const float* velocity,
                    int64_t padded, int64_t n, const AetherGrid* grid, uint64_t seed,
                    uint32_t* keys_out, int32_t* index_out, int32_t* cell_counts,
                    int32_t* cell_start, float* x_sorted, float* y_sorted, float* z_sorted,
                    float* velocity_sorted, int64_t padded_sorted, int path, void* workspace,
                    size_t workspace_bytes, void* stream, const PushSpec& push) {
  if (!grid) return cudaErrorInvalidValue;
  if (n > 0 && (!x_sorted || !y_sorted || !z_sorted)) return cudaErrorInvalidValue;
  if ((velocity == nullptr) != (velocity_sorted == nullptr)) return cudaErrorInvalidValue;
  if (velocity && (padded < n || padded_sorted < n)) return cudaErrorInvalidValue;
  if (path < 0 || path > 2) return cudaErrorInvalidValue;
  if (push.enabled && !velocity) return cudaErrorInvalidValue;
  SortArgs a{};
  a.x = x; a.y = y; a.z = z; a.velocity = velocity; a.padded = padded; a.n = n;
  a.grid = *grid; a.seed = seed;
  a.keys_out = keys_out; a.index_out = index_out;
  a.cell_counts = cell_counts; a.cell_start = cell_start;
  a.xs = x_sorted; a.ys = y_sorted; a.zs = z_sorted; a.vs = velocity_sorted;
  a.padded_sorted = padded_sorted;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  a.push = push;
  return run_sort(a, path);
}
}  // namespace
}  // namespace aether

extern "C" int AetherSortAndGatherParticles(
    const float* x, const float* y, const float* z, const float* velocity, int64_t padded,
    int64_t n, const AetherGrid* grid, uint64_t seed, uint32_t* keys_out, int32_t* index_out,
    int32_t* cell_counts, int32_t* cell_start, float* x_sorted, float* y_sorted, float* z_sorted,
    float* velocity_sorted, int64_t padded_sorted, int path, void* workspace,
    size_t workspace_bytes, void* stream) {
  return sort_and_gather(x, y, z, velocity, padded, n, grid, seed, keys_out, index_out,
                         cell_counts, cell_start, x_sorted, y_sorted, z_sorted, velocity_sorted,
                         padded_sorted, path, workspace, workspace_bytes, stream, PushSpec{});
}

extern "C" int AetherPushSortAndGatherParticles(
    const float* x, const float* y, const float* z, const float* velocity, int64_t padded,
    int64_t n, float dt, const float* lo, const float* hi, const AetherGrid* grid, uint64_t seed,
    uint32_t* keys_out, int32_t* index_out, int32_t* cell_counts, int32_t* cell_start,
    float* x_sorted, float* y_sorted, float* z_sorted, float* velocity_sorted,
    int64_t padded_sorted, int path, void* workspace, size_t workspace_bytes, void* stream) {
  if (!lo || !hi) return cudaErrorInvalidValue;
  PushSpec push{};
  push.enabled = 1;
  push.dt = dt;
  for (int c = 0; c < 3; ++c) {
    push.lo[c] = lo[c];
    push.hi[c] = hi[c];
  }
  return sort_and_gather(x, y, z, velocity, padded, n, grid, seed, keys_out, index_out,
                         cell_counts, cell_start, x_sorted, y_sorted, z_sorted, velocity_sorted,
                         padded_sorted, path, workspace, workspace_bytes, stream, push);
}

extern "C" int AetherGatherParticles(const int32_t* index, int64_t n, const float* x,
                                     const float* y, const float* z, const float* velocity,
                                     int64_t padded, float* x_sorted, float* y_sorted,
                                     float* z_sorted, float* velocity_sorted,
                                     int64_t padded_sorted, void* stream) {
  if (!count_ok(n)) return cudaErrorInvalidValue;
  if (n > 0 && (!index || !x || !y || !z || !x_sorted || !y_sorted || !z_sorted))
    return cudaErrorInvalidValue;
  if ((velocity == nullptr) != (velocity_sorted == nullptr)) return cudaErrorInvalidValue;
  if (velocity && (padded < n || padded_sorted < n)) return cudaErrorInvalidValue;
  return launch_gather(index, n, x, y, z, velocity, padded, x_sorted, y_sorted, z_sorted,
                       velocity_sorted, padded_sorted, static_cast<cudaStream_t>(stream));
}

extern "C" int AetherMakeKeys(const float* x, const float* y, const float* z, int64_t n,
                              const AetherGrid* grid, uint64_t seed, uint32_t* keys_out,
                              void* stream) {
  if (!count_ok(n) || !grid_ok(grid)) return cudaErrorInvalidValue;
  if (n > 0 && (!x || !y || !z || !keys_out)) return cudaErrorInvalidValue;
  return launch_make_keys(x, y, z, n, *grid, seed, keys_out, static_cast<cudaStream_t>(stream));
}

extern "C" int AetherSortReadStatus(const void* workspace, void* stream, int32_t* status) {
  if (!workspace || !status) return cudaErrorInvalidValue;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const Header* hdr = static_cast<const Header*>(workspace);
  cudaError_t e = cudaMemcpyAsync(status, &hdr->error, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(s);
}

extern "C" int AetherSortReadUsedDigitPasses(const void* workspace, void* stream, int32_t* used) {
  if (!workspace || !used) return cudaErrorInvalidValue;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const Header* hdr = static_cast<const Header*>(workspace);
  cudaError_t e = cudaMemcpyAsync(used, &hdr->use_standard, sizeof(int32_t),
                                  cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(s);
}

extern "C" size_t AetherSlabPartitionWorkspaceBytes(int64_t n, int world) {
  if (!count_ok(n) || world < 1 || world > 8) return 0;
  return slab_partition_workspace_bytes(n, world);
}

extern "C" int AetherSlabPartition(const float* x, const float* y, const float* z,
                                   const float* velocity, int64_t padded, int64_t n,
                                   const AetherGrid* grid, int world, float* x_out, float* y_out,
                                   float* z_out, float* vx_out, float* vy_out, float* vz_out,
                                   int64_t* counts_out, void* workspace, size_t workspace_bytes,
                                   void* stream) {
  if (!count_ok(n) || !grid_ok(grid) || !counts_out || !workspace) return cudaErrorInvalidValue;
  if (world < 1 || world > 8 || grid->nx % world != 0) return cudaErrorInvalidValue;
  if (n > 0 && (!x || !y || !z || !velocity || !x_out || !y_out || !z_out || !vx_out || !vy_out ||
                !vz_out || padded < n))
    return cudaErrorInvalidValue;
  return slab_partition(x, y, z, velocity, padded, n, *grid, world, x_out, y_out, z_out, vx_out,
                        vy_out, vz_out, counts_out, workspace, workspace_bytes,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int AetherParticlePush(float* x, float* y, float* z, float* vx, float* vy, float* vz,
                                  int64_t n, float dt, const float* lo, const float* hi,
                                  void* stream) {
  if (!count_ok(n) || !lo || !hi) return cudaErrorInvalidValue;
  if (n > 0 && (!x || !y || !z || !vx || !vy || !vz)) return cudaErrorInvalidValue;
  return particle_push(x, y, z, vx, vy, vz, n, dt, lo, hi, static_cast<cudaStream_t>(stream));
}

extern "C" int AetherDsmcCollideTma(float* velocity, const int* cell_start, float* sigma_g_max,
                                    int* collisions, int num_particles, int padded_particles,
                                    int num_cells, float selection_factor, float vhs_coefficient,
                                    float vhs_speed_exponent, uint64_t seed, uint64_t step,
                                    void* stream) {
  return collide_cells(velocity, cell_start, sigma_g_max, collisions, num_particles,
                       padded_particles, num_cells, selection_factor, vhs_coefficient,
                       vhs_speed_exponent, seed, step, static_cast<cudaStream_t>(stream));
}

namespace aether {
namespace {
PushSpec push_spec(float dt, const float* lo, const float* hi) {
  PushSpec push{};
  push.enabled = 1;
  push.dt = dt;
  for (int c = 0; c < 3; ++c) {
    push.lo[c] = lo[c];
    push.hi[c] = hi[c];
  }
  return push;
}

int exchange_count(const float* x, const float* vx, const PushSpec& push, int64_t n,
                   const AetherGrid* grid, int world, int64_t* counts_out, void* workspace,
                   size_t workspace_bytes, void* stream) {
  if (!count_ok(n) || !grid_ok(grid) || !counts_out || !workspace) return cudaErrorInvalidValue;
  if (n > 0 && !x) return cudaErrorInvalidValue;
  return slab_exchange_count(x, vx, push, n, *grid, world, counts_out, workspace, workspace_bytes,
                             static_cast<cudaStream_t>(stream));
}

int exchange_scatter(const float* x, const float* y, const float* z, const float* velocity,
                     int64_t padded, int64_t n, const AetherGrid* grid, int world, int rank,
                     float* const* peer_buffers, int64_t capacity, const int64_t* count_matrix,
                     int32_t* error_out, const PushSpec& push, void* workspace,
                     size_t workspace_bytes, void* stream, const SliceSignal* signal = nullptr) {
  if (!count_ok(n) || !grid_ok(grid) || !peer_buffers || !count_matrix || !error_out || !workspace)
    return cudaErrorInvalidValue;
  if (capacity <= 0 || capacity % 4 != 0 || world < 1 || world > 8) return cudaErrorInvalidValue;
  if (n > 0 && (!x || !y || !z || !velocity || padded < n)) return cudaErrorInvalidValue;
  return slab_exchange_scatter(x, y, z, velocity, padded, n, *grid, world, rank, peer_buffers,
                               capacity, count_matrix, error_out, push, workspace,
                               workspace_bytes, static_cast<cudaStream_t>(stream), signal);
}
}  // namespace
}  // namespace aether

extern "C" int AetherSlabExchangeCount(const float* x, int64_t n, const AetherGrid* grid, int world,
                                       int64_t* counts_out, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  return exchange_count(x, nullptr, PushSpec{}, n, grid, world, counts_out, workspace,
                        workspace_bytes, stream);
}

extern "C" int AetherSlabExchangeScatter(const float* x, const float* y, const float* z,
                                         const float* velocity, int64_t padded, int64_t n,
                                         const AetherGrid* grid, int world, int rank,
                                         float* const* peer_buffers, int64_t capacity,
                                         const int64_t* count_matrix, int32_t* error_out,
                                         void* workspace, size_t workspace_bytes, void* stream) {
  return exchange_scatter(x, y, z, velocity, padded, n, grid, world, rank, peer_buffers, capacity,
                          count_matrix, error_out, PushSpec{}, workspace, workspace_bytes, stream);
}

extern "C" int AetherSlabExchangeCountMoved(const float* x, const float* vx, int64_t n, float dt,
                                            const float* lo, const float* hi,
                                            const AetherGrid* grid, int world,
                                            int64_t* counts_out, void* workspace,
                                            size_t workspace_bytes, void* stream) {
  if (!lo || !hi || (n > 0 && !vx)) return cudaErrorInvalidValue;
  return exchange_count(x, vx, push_spec(dt, lo, hi), n, grid, world, counts_out, workspace,
                        workspace_bytes, stream);
}

extern "C" int AetherSlabExchangeScatterMoved(
    const float* x, const float* y, const float* z, const float* velocity, int64_t padded,
    int64_t n, float dt, const float* lo, const float* hi, const AetherGrid* grid, int world,
    int rank, float* const* peer_buffers, int64_t capacity, const int64_t* count_matrix,
    int32_t* error_out, void* workspace, size_t workspace_bytes, void* stream) {
  if (!lo || !hi) return cudaErrorInvalidValue;
  return exchange_scatter(x, y, z, velocity, padded, n, grid, world, rank, peer_buffers, capacity,
                          count_matrix, error_out, push_spec(dt, lo, hi), workspace,
                          workspace_bytes, stream);
}

// ---- the sliced exchange and the sort of its segmented result ----

extern "C" int AetherSlabExchangeSliceCounts(int64_t n, int world, int slices,
                                             int64_t* slice_counts_out, void* workspace,
                                             size_t workspace_bytes, void* stream) {
  if (!count_ok(n) || !workspace) return cudaErrorInvalidValue;
  return slab_exchange_slice_counts(n, world, slices, slice_counts_out, workspace, workspace_bytes,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" size_t AetherSlabSegmentsBytes(void) { return sizeof(SliceSegments); }

extern "C" int AetherSlabExchangeSetResidentBlocks(int blocks_per_multiprocessor) {
  if (blocks_per_multiprocessor < 0 || blocks_per_multiprocessor > 4) return cudaErrorInvalidValue;
  slab_exchange_set_blocks_per_sm(blocks_per_multiprocessor);
  return 0;
}

extern "C" int AetherSlabExchangePrepare(const int64_t* count_matrix, int world, int slices,
                                         int rank, int64_t* totals_out, void* segments_out,
                                         void* stream) {
  return slab_exchange_prepare(count_matrix, world, slices, rank, totals_out,
                               static_cast<SliceSegments*>(segments_out),
                               static_cast<cudaStream_t>(stream));
}

extern "C" int AetherSlabExchangeScatterSliced(
    const float* x, const float* y, const float* z, const float* velocity, int64_t padded,
    int64_t n, float dt, const float* lo, const float* hi, const AetherGrid* grid, int world,
    int rank, float* const* peer_buffers, int64_t capacity, const int64_t* totals,
    int32_t* error_out, int slices, int slice, uint32_t epoch, uint32_t* const* peer_flags,
    void* workspace, size_t workspace_bytes, void* stream) {
  if ((lo == nullptr) != (hi == nullptr)) return cudaErrorInvalidValue;
  const SliceSignal signal{slices, slice, epoch, peer_flags};
  return exchange_scatter(x, y, z, velocity, padded, n, grid, world, rank, peer_buffers, capacity,
                          totals, error_out, lo ? push_spec(dt, lo, hi) : PushSpec{}, workspace,
                          workspace_bytes, stream, &signal);
}

extern "C" int AetherSlabExchangeSignal(int world, int rank, int slices, int slice,
                                        uint32_t epoch, uint32_t* const* peer_flags,
                                        void* stream) {
  return slab_signal_slice(world, rank, slices, slice, epoch, peer_flags,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int AetherSlabExchangeCopy(void* destination, const void* source, size_t row_bytes,
                                      int rows, size_t pitch_bytes, void* stream) {
  if (row_bytes == 0 || rows == 0) return cudaSuccess;
  if (!destination || !source || rows < 0 || pitch_bytes < row_bytes) return cudaErrorInvalidValue;
  if (rows == 1)
    return cudaMemcpyAsync(destination, source, row_bytes, cudaMemcpyDeviceToDevice,
                           static_cast<cudaStream_t>(stream));
  return cudaMemcpy2DAsync(destination, pitch_bytes, source, pitch_bytes, row_bytes,
                           static_cast<size_t>(rows), cudaMemcpyDeviceToDevice,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int AetherSlabExchangeWait(const uint32_t* flags, int world, int slices, int slice,
                                      uint32_t epoch, uint32_t poll_limit, int32_t* error_out,
                                      void* stream) {
  return slab_wait_slice(flags, world, slices, slice, epoch, poll_limit, error_out,
                         static_cast<cudaStream_t>(stream));
}

extern "C" size_t AetherSortSlicedWorkspaceBytes(int64_t capacity, int64_t plan_n,
                                                 int64_t num_cells, int slices) {
  if (!count_ok(capacity) || !count_ok(plan_n) || plan_n <= 0 || num_cells <= 0 ||
      key_bits_of(num_cells) > 32 || slices < 1 || slices > kMaxSlices)
    return 0;
  return sliced_sort_workspace_bytes(capacity, plan_n, num_cells, slices);
}

namespace aether {
namespace {
bool sliced_args(SortArgs& a, int64_t capacity, int64_t plan_n, const AetherGrid* grid,
                 void* workspace, size_t workspace_bytes, void* stream) {
  if (!count_ok(capacity) || !count_ok(plan_n) || plan_n <= 0 || !grid_ok(grid) || !workspace)
    return false;
  a.n = capacity;
  a.grid = *grid;
  a.num_cells = static_cast<int64_t>(grid->nx_local) * grid->ny * grid->nz;
  a.key_bits = key_bits_of(a.num_cells);
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.stream = static_cast<cudaStream_t>(stream);
  return true;
}
}  // namespace
}  // namespace aether

extern "C" int AetherSortSlicedBegin(int64_t capacity, int64_t plan_n, const AetherGrid* grid,
                                     int slices, void* workspace, size_t workspace_bytes,
                                     void* stream) {
  SortArgs a{};
  if (!sliced_args(a, capacity, plan_n, grid, workspace, workspace_bytes, stream))
    return cudaErrorInvalidValue;
  return sliced_sort_begin(a, plan_n, slices);
}

extern "C" int AetherSortSlicedSlice(const float* x, const float* y, const float* z,
                                     const float* velocity, int64_t padded, int64_t capacity,
                                     int64_t plan_n, const AetherGrid* grid, uint64_t seed,
                                     const void* segments, int slices, int slice, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  SortArgs a{};
  if (!sliced_args(a, capacity, plan_n, grid, workspace, workspace_bytes, stream))
    return cudaErrorInvalidValue;
  a.x = x; a.y = y; a.z = z; a.velocity = velocity; a.padded = padded; a.seed = seed;
  return sliced_sort_slice(a, plan_n, static_cast<const SliceSegments*>(segments), slices, slice);
}

extern "C" int AetherSortSlicedFinish(int64_t capacity, int64_t plan_n, const AetherGrid* grid,
                                      const void* segments, int slices, uint32_t* keys_out,
                                      int32_t* index_out, int32_t* cell_counts,
                                      int32_t* cell_start, float* x_sorted, float* y_sorted,
                                      float* z_sorted, float* velocity_sorted,
                                      int64_t padded_sorted, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  SortArgs a{};
  if (!sliced_args(a, capacity, plan_n, grid, workspace, workspace_bytes, stream))
    return cudaErrorInvalidValue;
  if (!x_sorted || !y_sorted || !z_sorted || !velocity_sorted || padded_sorted < 4)
    return cudaErrorInvalidValue;
  a.keys_out = keys_out; a.index_out = index_out;
  a.cell_counts = cell_counts; a.cell_start = cell_start;
  a.xs = x_sorted; a.ys = y_sorted; a.zs = z_sorted; a.vs = velocity_sorted;
  a.padded_sorted = padded_sorted;
  return sliced_sort_finish(a, plan_n, static_cast<const SliceSegments*>(segments), slices);
}
