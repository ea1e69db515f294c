/* C ABI of libaether_sort.so: the DSMC particle sort for NVIDIA B200 (sm_100a).
 *
 * Conventions (the ones the reference's native library uses for its ctypes
 * boundary, project_aether/src/custom_kernels/cuda/dsmc_collide_tma.h:121-129
 * and dsmc_collide_tma.cu:224-299):
 *   - every pointer is a raw device pointer owned by the caller; `stream` is a
 *     cudaStream_t passed as void*; the call only enqueues work on it;
 *   - the return value is a cudaError_t as int, 0 on success;
 *     cudaErrorInvalidValue (1) is returned for bad arguments before anything
 *     is launched;
 *   - the library allocates nothing: scratch memory is a caller-provided
 *     workspace whose size comes from AetherSortWorkspaceBytes.
 *
 * Keys are UNSIGNED 32-bit: key = (cell << 7) | shuffle, cell id x-fastest
 * (project_aether/src/custom_kernels/triton/fused_radix_sort.py:93-103).
 */
#ifndef AETHER_SORT_H_
#define AETHER_SORT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Geometry of one sort call.  `inv_d*` = cells / (hi - lo) computed in double
 * and rounded to float by the host, as the reference's driver does
 * (fused_radix_sort.py:250).  `nx, ny, nz` is the GLOBAL grid used to compute
 * (ix, iy, iz); the cell id is linearised over the x-slab
 * [ix_offset, ix_offset + nx_local): cell = (iz*ny + iy)*nx_local + ix - ix_offset.
 * A single-GPU sort passes ix_offset = 0, nx_local = nx.  The reference has no
 * slab form; it is the multi-GPU extension of fused_radix_sort.py:99.
 * Precondition of the slab form: every particle's column ix lies inside the
 * slab (the exchange step guarantees it).  A particle outside it is binned into
 * the slab's nearest column, ix - ix_offset clamped to [0, nx_local - 1], so
 * that no table is ever indexed out of range; its cell is then not its own. */
typedef struct AetherGrid {
  float x0, y0, z0;
  float inv_dx, inv_dy, inv_dz;
  int32_t nx, ny, nz;
  int32_t ix_offset, nx_local;
} AetherGrid;

/* Library / ABI version (bumped when a signature changes). */
int AetherSortAbiVersion(void);

/* Bytes of workspace needed by the sort entry points for `n` particles and
 * `num_cells` (slab-local) cells; `with_payload` != 0 when positions and
 * velocities are to be carried (about 40 bytes per particle, 32 without).
 * Replaces the per-call tensor allocations of the reference driver
 * (fused_radix_sort.py:245-248,257-263).  A smaller workspace is accepted as
 * long as the digit passes fit (8 bytes per particle plus status words): with
 * `path` 0 the call then runs the digit passes, the slower of its paths, and
 * `path` 2 is refused.  Returns 0 if the arguments are out of range (n < 0,
 * n >= 2^30, key wider than 32 bits). */
size_t AetherSortWorkspaceBytes(int64_t n, int64_t num_cells, int with_payload);

/* How the bucketed path would lay a call out, for diagnostics and tests (no
 * counterpart in the reference): a bucket is 2^*cells_per_bucket_log2
 * consecutive cell ids, there are *buckets of them, and the finish kernel sorts
 * groups of consecutive buckets of at most *group_capacity records at a time
 * (fuller buckets are cut by cells).  Needs a current CUDA device (the group
 * capacity depends on its multiprocessor count).  Returns cudaErrorInvalidValue
 * when the bucketed path cannot take such a call (the digit passes then run). */
int AetherSortBucketPlan(int64_t n, int64_t num_cells, int32_t* cells_per_bucket_log2,
                         int64_t* buckets, int32_t* group_capacity);

/* Process-wide switch (no counterpart in the reference).  The two dozen kernels of one sort
 * call run one after the other, and the gaps between them are most of what a small call
 * costs.  mode 1 (default): the short kernels (scans, tables, the digit passes that return at
 * once when the bucketed path has done the call) are launched so that each may be set up
 * while the one before it still runs (programmatic dependent launch); mode 2: the scatter and
 * finish kernels too (measured slower on large inputs); mode 0: ordinary launches.  Every
 * kernel waits for the grids before it to complete before it touches anything, so the work
 * runs in stream order in every mode and results do not depend on it. */
int AetherSortSetChainedLaunches(int32_t mode);

/* Tuning knob of the bucketed path (process-wide; no counterpart in the reference): the
 * finish kernel runs in its small shape (two 512-thread blocks per multiprocessor, 2560
 * records each) while the plan needs at most `buckets` buckets of about a thousand records,
 * and in its large shape (one 1024-thread block, 5120 records) beyond.  Default and maximum
 * 32,768; 0 plans the large shape always.  Results do not depend on it. */
int AetherSortSetSmallShapeBucketLimit(int64_t buckets);

/* sort_particles_by_cell (fused_radix_sort.py:221-280): sorted keys,
 * permutation (original index of every sorted particle), per-cell counts (C)
 * and exclusive starts (C+1).  Inputs are not modified. */
int AetherSortParticlesByCell(const float* x, const float* y, const float* z, int64_t n,
                              const AetherGrid* grid, uint64_t seed, uint32_t* keys_out,
                              int32_t* index_out, int32_t* cell_counts, int32_t* cell_start,
                              void* workspace, size_t workspace_bytes, void* stream);

/* The sort plus the payload gather that follows it in the DSMC step
 * (project_aether/src/physics_engine/dsmc_gpu_pipeline.py:105-109): also
 * writes positions and velocities in sorted order.  `velocity` and
 * `velocity_sorted` are (3, padded) row-major with rows vx, vy, vz
 * (dsmc_gpu_pipeline.py:55,69-71); only columns [0, n) are written.
 * `path`: 0 = choose, 1 = digit passes + gather, 2 = bucketed path. */
int AetherSortAndGatherParticles(const float* x, const float* y, const float* z,
                                 const float* velocity, int64_t padded, int64_t n,
                                 const AetherGrid* grid, uint64_t seed, uint32_t* keys_out,
                                 int32_t* index_out, int32_t* cell_counts, int32_t* cell_start,
                                 float* x_sorted, float* y_sorted, float* z_sorted,
                                 float* velocity_sorted, int64_t padded_sorted, int path,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* The payload gather alone (dsmc_gpu_pipeline.py:107-109): out[r] = in[index[r]]. */
int AetherGatherParticles(const int32_t* index, int64_t n, const float* x, const float* y,
                          const float* z, const float* velocity, int64_t padded,
                          float* x_sorted, float* y_sorted, float* z_sorted,
                          float* velocity_sorted, int64_t padded_sorted, void* stream);

/* Key generation alone (the first half of _bin_keys_kernel,
 * fused_radix_sort.py:87-105): keys[i] for the particles as given. */
int AetherMakeKeys(const float* x, const float* y, const float* z, int64_t n,
                   const AetherGrid* grid, uint64_t seed, uint32_t* keys_out, void* stream);

/* Device waits in the digit passes are bounded; a wait that gives up records a
 * code in the workspace instead of spinning (the reference's look-back spins
 * without limit, fused_radix_sort.py:160-171).  This call synchronises
 * `stream`, reads the code back and stores it in *status (0 = clean). */
int AetherSortReadStatus(const void* workspace, void* stream, int32_t* status);

/* Which path produced the last result in this workspace: synchronises `stream`
 * and stores 1 in *used if the device handed the call from the bucketed path to
 * the digit passes (a cell or a counter too full for shared memory), else 0.
 * The results are the same either way; the digit passes are slower.  (New: the
 * reference has a single path.) */
int AetherSortReadUsedDigitPasses(const void* workspace, void* stream, int32_t* used);

/* Multi-GPU step 1: stable partition of this rank's particles by destination
 * x-slab.  With `world` ranks (1..8, nx divisible by world) rank r owns global
 * ix in [r*nx/world, (r+1)*nx/world); ix is computed with the global grid as in
 * fused_radix_sort.py:93.  Writes six contiguous arrays (x, y, z, vx, vy, vz),
 * each ordered by destination rank and, inside one destination, in the input
 * order; counts_out[d] (device, int64) receives the number of particles bound
 * for rank d.  The reference has no multi-GPU particle path; the ordering rule
 * matches its all-to-all convention "row s holds what rank s sent"
 * (project_aether/src/distributed_infra/sccl_synthesizer.py:468-485). */
size_t AetherSlabPartitionWorkspaceBytes(int64_t n, int world);
int AetherSlabPartition(const float* x, const float* y, const float* z, const float* velocity,
                        int64_t padded, int64_t n, const AetherGrid* grid, int world,
                        float* x_out, float* y_out, float* z_out, float* vx_out, float* vy_out,
                        float* vz_out, int64_t* counts_out, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Multi-GPU step 1 fused with the exchange: instead of partitioning locally and
 * handing the arrays to an all-to-all, the scatter writes every particle straight
 * into the receive buffer of its destination GPU over NVLink (plain peer stores,
 * coalesced runs).  Two calls, with the ranks' count exchange in between:
 *   AetherSlabExchangeCount    counts_out[d] (device) = particles bound for rank d;
 *                              leaves the tile offsets in the workspace;
 *   AetherSlabExchangeScatter  peer_buffers[d] (host array of device pointers) is
 *                              rank d's receive buffer of 6 * capacity floats laid
 *                              out [x | y | z | vx | vy | vz], each `capacity` long
 *                              (a multiple of 4); count_matrix (device, int64
 *                              [world][world], [s][d] = particles s sends to d) is
 *                              the all-gathered counts, read on the device so that
 *                              the host need not wait for it; if some rank would
 *                              receive more than `capacity`, nothing is stored for
 *                              it and *error_out (device) is set.  Same ordering
 *                              rule as AetherSlabPartition + all-to-all.
 * The caller must make sure that the peers have finished reading their buffers
 * before the scatter, and that all ranks' scatters are complete before a buffer
 * is read (stream-ordered collectives do both).  No counterpart in the reference. */
int AetherSlabExchangeCount(const float* x, int64_t n, const AetherGrid* grid, int world,
                            int64_t* counts_out, void* workspace, size_t workspace_bytes,
                            void* stream);
int AetherSlabExchangeScatter(const float* x, const float* y, const float* z,
                              const float* velocity, int64_t padded, int64_t n,
                              const AetherGrid* grid, int world, int rank,
                              float* const* peer_buffers, int64_t capacity,
                              const int64_t* count_matrix, int32_t* error_out, void* workspace,
                              size_t workspace_bytes, void* stream);

/* The two exchange calls with the move stage fused in: particles are counted
 * and sent as they are after x += v*dt with specular reflection at lo/hi (the
 * arithmetic of AetherParticlePush; `vx` is the first row of the velocity
 * array, `lo`, `hi` host pointers to three floats).  The receiving rank's sort
 * then needs no move.  The input arrays are not modified.  (New, like the
 * exchange itself.) */
int AetherSlabExchangeCountMoved(const float* x, const float* vx, int64_t n, float dt,
                                 const float* lo, const float* hi, const AetherGrid* grid,
                                 int world, int64_t* counts_out, void* workspace,
                                 size_t workspace_bytes, void* stream);
int AetherSlabExchangeScatterMoved(const float* x, const float* y, const float* z,
                                   const float* velocity, int64_t padded, int64_t n, float dt,
                                   const float* lo, const float* hi, const AetherGrid* grid,
                                   int world, int rank, float* const* peer_buffers,
                                   int64_t capacity, const int64_t* count_matrix,
                                   int32_t* error_out, void* workspace, size_t workspace_bytes,
                                   void* stream);

/* The sliced form of the exchange and of the local sort behind it, which lets
 * the two overlap (no counterpart in the reference).  Every rank cuts its input
 * into `slices` (1..32) runs of consecutive tiles; the exchange tells the
 * destinations when a slice has been stored, and the destination counts and
 * scatters slice k of all sources into the records of its sort while later
 * slices are still on their way; only the finish kernels wait for everything.
 * The ordering rule, hence every result, is that of the unsliced form.
 *
 *   AetherSlabExchangeSliceCounts   after AetherSlabExchangeCount[Moved] on the same
 *       workspace: slice_counts_out[k * world + d] (device) = particles of slice k for
 *       rank d.  The ranks all-gather these into count_matrix[s][k][d].
 *   AetherSlabExchangePrepare       from the gathered matrix: totals_out[s][d] (device,
 *       what AetherSlabExchangeScatterSliced reads) and this rank's segment table
 *       (segments_out, AetherSlabSegmentsBytes() bytes of device memory): where every
 *       source's slice lies in the received arrays.
 *   AetherSlabExchangeScatterSliced AetherSlabExchangeScatter (with the move fused in when
 *       lo/hi are not NULL) for the tiles of slice `slice` only, followed in the stream by a
 *       one-warp kernel that writes `epoch` to word [rank * slices + slice] of every
 *       peer_flags[d] (host array of device pointers into the ranks' flag arrays of
 *       world * slices words).  A kernel is complete only when its stores are performed, so
 *       the flag cannot overtake the data.  Called once per slice, in order; epochs must
 *       grow from step to step.
 *   AetherSlabExchangeSignal        the one-warp kernel alone, and
 *   AetherSlabExchangeCopy          one device-to-device copy of `rows` rows of row_bytes
 *       bytes, pitch_bytes apart on both sides (cudaMemcpy2DAsync; cudaMemcpyAsync for one
 *       row): the transport of the exchange by copy engine.  There
 *       AetherSlabExchangeScatterSliced partitions slice `slice` into staging buffers in this
 *       GPU's own memory (peer_buffers[d] = the staging buffer for destination d, laid out
 *       like d's receive buffer; peer_flags[d] = a scratch flag array), one copy per
 *       destination (six rows: the six arrays, `capacity` floats apart) then carries the
 *       slice's share into the destination's receive buffer without occupying a
 *       multiprocessor, and the signal follows the copies in stream order.
 *   AetherSlabExchangeWait          enqueues a one-warp kernel that polls this rank's flag
 *       array until every source has signalled `slice` of `epoch`.  The wait is bounded:
 *       after poll_limit polls (256 ns apart) it stores 6 in *error_out (device) and
 *       returns, and the step must be discarded.
 *
 *   AetherSortSliced{Begin,Slice,Finish}  the bucketed sort of the received arrays with one
 *       chunk of records per slice: Begin clears the tables, Slice k counts, scans and
 *       scatters the particles of slice k, Finish sorts the buckets and writes all outputs.
 *       `capacity` is the length of the input arrays; the particle count is read from the
 *       segment table on the device; `plan_n` (host) is the particle count the bucket
 *       widths are planned for, e.g. the previous step's.  Workspace from
 *       AetherSortSlicedWorkspaceBytes.  Results as AetherSortAndGatherParticles.
 *   AetherSlabExchangeSetResidentBlocks  tuning knob: thread blocks of the sliced exchange
 *       kernel per multiprocessor (1..4, default 2; 0 = one block per tile).  Fewer leave
 *       more of the GPU to the local sort's kernels that run beside it; more keep more
 *       NVLink stores in flight.
 */
int AetherSlabExchangeSetResidentBlocks(int blocks_per_multiprocessor);
int AetherSlabExchangeSliceCounts(int64_t n, int world, int slices, int64_t* slice_counts_out,
                                  void* workspace, size_t workspace_bytes, void* stream);
size_t AetherSlabSegmentsBytes(void);
int AetherSlabExchangePrepare(const int64_t* count_matrix, int world, int slices, int rank,
                              int64_t* totals_out, void* segments_out, void* stream);
int AetherSlabExchangeScatterSliced(const float* x, const float* y, const float* z,
                                    const float* velocity, int64_t padded, int64_t n, float dt,
                                    const float* lo, const float* hi, const AetherGrid* grid,
                                    int world, int rank, float* const* peer_buffers,
                                    int64_t capacity, const int64_t* totals, int32_t* error_out,
                                    int slices, int slice, uint32_t epoch,
                                    uint32_t* const* peer_flags, void* workspace,
                                    size_t workspace_bytes, void* stream);
int AetherSlabExchangeSignal(int world, int rank, int slices, int slice, uint32_t epoch,
                             uint32_t* const* peer_flags, void* stream);
int AetherSlabExchangeCopy(void* destination, const void* source, size_t row_bytes, int rows,
                           size_t pitch_bytes, void* stream);
int AetherSlabExchangeWait(const uint32_t* flags, int world, int slices, int slice,
                           uint32_t epoch, uint32_t poll_limit, int32_t* error_out, void* stream);
size_t AetherSortSlicedWorkspaceBytes(int64_t capacity, int64_t plan_n, int64_t num_cells,
                                      int slices);
int AetherSortSlicedBegin(int64_t capacity, int64_t plan_n, const AetherGrid* grid, int slices,
                          void* workspace, size_t workspace_bytes, void* stream);
int AetherSortSlicedSlice(const float* x, const float* y, const float* z, const float* velocity,
                          int64_t padded, int64_t capacity, int64_t plan_n,
                          const AetherGrid* grid, uint64_t seed, const void* segments, int slices,
                          int slice, void* workspace, size_t workspace_bytes, void* stream);
int AetherSortSlicedFinish(int64_t capacity, int64_t plan_n, const AetherGrid* grid,
                           const void* segments, int slices, uint32_t* keys_out,
                           int32_t* index_out, int32_t* cell_counts, int32_t* cell_start,
                           float* x_sorted, float* y_sorted, float* z_sorted,
                           float* velocity_sorted, int64_t padded_sorted, void* workspace,
                           size_t workspace_bytes, void* stream);

/* The move stage that precedes the sort in the DSMC step: x += v*dt, specular
 * reflection at the six walls, in place (fused_particle_push,
 * project_aether/src/custom_kernels/triton/fused_particle_push.py:75-92; arithmetic
 * of its unfused statement reference_push, :95-108).  `lo`, `hi` are host
 * pointers to three floats each. */
int AetherParticlePush(float* x, float* y, float* z, float* vx, float* vy, float* vz, int64_t n,
                       float dt, const float* lo, const float* hi, void* stream);

/* The move stage and the sort in one call: every particle is taken at
 * x + v*dt with specular reflection at lo/hi (the arithmetic of AetherParticlePush),
 * sorted by the cell of that moved position, and the sorted payload carries the
 * moved positions and the reflected velocities.  The input arrays are not
 * modified.  Replaces lines 101-109 of the reference's step
 * (project_aether/src/physics_engine/dsmc_gpu_pipeline.py: fused_particle_push,
 * sort_particles_by_cell and the four index_select gathers) and saves the move
 * stage's own pass over positions and velocities (48 bytes per particle).
 * Arguments as AetherSortAndGatherParticles plus dt and host pointers lo, hi to
 * three floats each; velocity is required; the workspace must have the size
 * AetherSortWorkspaceBytes(n, num_cells, 1) reports. */
int AetherPushSortAndGatherParticles(
    const float* x, const float* y, const float* z, const float* velocity, int64_t padded,
    int64_t n, float dt, const float* lo, const float* hi, const AetherGrid* grid, uint64_t seed,
    uint32_t* keys_out, int32_t* index_out, int32_t* cell_counts, int32_t* cell_start,
    float* x_sorted, float* y_sorted, float* z_sorted, float* velocity_sorted,
    int64_t padded_sorted, int path, void* workspace, size_t workspace_bytes, void* stream);

/* The stage that follows the sort in the DSMC step: No-Time-Counter collisions
 * on the cell-sorted velocities, in place.  Name, arguments and return value are
 * those of the reference's entry point, so its ctypes binding loads this library
 * unchanged (project_aether/src/custom_kernels/cuda/dsmc_collide_tma.h:121-129,
 * bound in project_aether/src/custom_kernels/cuda/tma_collide.py:67-78); the
 * kernel behind it is written for sm_100a and uses no tensor map.
 *   velocity     (3, padded_particles) floats, rows vx, vy, vz, cell-sorted, updated in place;
 *                padded_particles is a multiple of 4
 *   cell_start   (num_cells + 1) exclusive prefix of the cell counts
 *   sigma_g_max  (num_cells) majorant of sigma_T * g per cell, raised to the largest value seen
 *   collisions   (num_cells) receives the accepted pairs of every cell
 * The candidate pairs of a cell are (start + 2j, start + 1 + 2j): the sort's shuffle
 * bits have already randomised the order inside a cell.  Pair arithmetic follows
 * dsmc_collide_tma.h:59-113. */
int AetherDsmcCollideTma(float* velocity, const int* cell_start, float* sigma_g_max,
                         int* collisions, int num_particles, int padded_particles, int num_cells,
                         float selection_factor, float vhs_coefficient, float vhs_speed_exponent,
                         uint64_t seed, uint64_t step, void* stream);

/* The same sort for callers that cannot allocate device memory: a plugin that
 * runs inside a host application which has already handed all of the GPU's
 * memory to its own pool, or a step of a real-time loop in which cudaMalloc
 * (which synchronises the whole device) is forbidden.  Such a caller has no
 * workspace to pass, so this entry point keeps the sort's scratch in a fixed
 * array inside the library image (9 MiB, reserved on every GPU
 * that loads the library until the process exits) and allocates nothing: no
 * cudaMalloc, no cudaFree, no allocating library routine.  It has no
 * counterpart in the reference, whose driver allocates about ten tensors per
 * call (fused_radix_sort.py:245-263).
 *   - Limit: n <= AetherSortStaticMaxParticles() (2^20); larger counts, or a
 *     grid whose scratch would not fit, return cudaErrorInvalidValue before
 *     anything is launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) with that device current; make that first call
 *     outside any stream capture.
 *   - All calls share the one array.  It keeps the previous call's contents; the
 *     call clears the part that must start at zero itself.  Two calls whose
 *     work overlaps on the GPU (different streams, no dependency) race on it:
 *     serialise them.
 *   - Which of the two sort paths runs follows from the size: calls whose
 *     bucketed record layout fits the array (up to a few hundred thousand
 *     particles) take the bucketed path, larger ones the digit passes.
 *   - The device status of a call (a bounded wait that gave up) lives in that
 *     array too: read it with AetherSortStaticReadStatus, and the path that
 *     produced the result with AetherSortStaticReadUsedDigitPasses; both
 *     synchronise `stream` like their workspace twins and allocate nothing.
 * Inputs, outputs and results are those of AetherSortParticlesByCell. */
int64_t AetherSortStaticMaxParticles(void);
int AetherSortParticlesByCellStatic(const float* x, const float* y, const float* z, int64_t n,
                                    const AetherGrid* grid, uint64_t seed, uint32_t* keys_out,
                                    int32_t* index_out, int32_t* cell_counts, int32_t* cell_start,
                                    void* stream);
int AetherSortStaticReadStatus(void* stream, int32_t* status);
int AetherSortStaticReadUsedDigitPasses(void* stream, int32_t* used);

/* Test hook for the bounded device waits (no counterpart in the reference, whose
 * look-back spins without limit, fused_radix_sort.py:160-171).  Runs one digit
 * pass over three tiles of zero keys with the ticket dispenser started at 1, so
 * that the tile every look-back ends at is never processed and never publishes:
 * the waiting blocks poll `poll_limit` times, record the give-up code in the
 * workspace header and return.  Nothing traps or spins without limit.  Afterwards
 * AetherSortReadStatus(workspace, ...) reports 1 (look-back timeout).  The
 * workspace must hold AetherSortProbeLookbackWorkspaceBytes() bytes. */
size_t AetherSortProbeLookbackWorkspaceBytes(void);
int AetherSortProbeLookbackGiveUp(void* workspace, size_t workspace_bytes, uint32_t poll_limit,
                                  void* stream);

/* Measurement hooks.  The reference times whole calls with CUDA events around
 * the Python entry point (project_aether/scripts/phase2_triton_sort_benchmark.py:
 * 73-84); these give the same kind of event timing per stage of one call.
 * With stage timing enabled every sort call brackets its stages with events on
 * the caller's stream.  AetherSortReadStageTimes synchronises on them and
 * writes the elapsed milliseconds of each stage, averaged over the sort calls
 * made since timing was enabled (the most recent 32 at most; -1 for a stage
 * that did not run), into ms_out[0 .. AetherSortStageCount()).  The timing
 * state is process-wide and bound to the device that is current when timing is
 * enabled: calls on other devices are not timed, and the figures only mean
 * something when the timed calls come from one host thread.
 * AetherSortKernelLaunches returns how many kernels this library has launched
 * in this process so far. */
int AetherSortSetStageTiming(int enabled);
int AetherSortStageCount(void);
const char* AetherSortStageName(int stage);
int AetherSortReadStageTimes(float* ms_out, int capacity);
uint64_t AetherSortKernelLaunches(void);

#ifdef __cplusplus
}
#endif

#endif /* AETHER_SORT_H_ */
