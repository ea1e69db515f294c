// Bucketed path of the particle sort: every byte of particle payload moves
// through HBM twice, both times in full 32-byte sectors or long runs.
//
//   bucket_count_kernel    reads x,y,z once and counts particles per bucket, a
//                          bucket being 2^s consecutive cell ids (the upsweep;
//                          replaces the histogram half of _bin_keys_kernel,
//                          fused_radix_sort.py:106-113)
//   bucket_scan_kernel     exclusive scan of the bucket counts -> bucket starts
//                          and write cursors; decides whether every bucket fits
//                          one thread block's shared memory
//   bucket_scatter_kernel  reads x,y,z,v once, builds the key (cell id + Philox
//                          shuffle bits, fused_radix_sort.py:93-103) and writes
//                          one 32-byte record {key, index, x, y, z, vx, vy, vz}
//                          into the particle's bucket
//   bucket_finish_kernel   a thread block takes a GROUP of consecutive buckets
//                          that fits its shared memory (cut on the device from
//                          the bucket totals, so dense and thin regions both
//                          fill a block): a counting sort on the low key bits
//                          in shared memory, ties put in index order, then
//                          coalesced SoA output of keys, indices, positions,
//                          velocities and the group's rows of cell_counts /
//                          cell_start (replaces the digit passes, the last-pass
//                          count atomics, torch.cumsum and the payload gather:
//                          fused_radix_sort.py:116-203,277-279,
//                          dsmc_gpu_pipeline.py:107-109)
//
// The result equals the stable sort by key: the records of a bucket arrive in
// no particular order, and the finish kernel orders them by (low key bits,
// original index), which is the order a stable sort produces.
//
// Record layout in HBM: chunk-major.  The particles are taken in chunks of 2^22
// consecutive indices; the records of chunk c and bucket b form one run, and the
// runs are laid out [chunk][bucket].  While chunk c is being scattered all
// stores fall into its 128 MB region instead of the whole record array: B200
// serves scattered 32-byte stores about 1.6 times faster that way (measured).
// Consecutive buckets are neighbours inside a chunk's region, so a group of
// buckets is still one contiguous run per chunk: the finish kernel collects a
// group with one bulk copy per chunk.
#include <algorithm>

#include "common.cuh"

namespace aether {

namespace {

constexpr int kRecordWords = 8;  // 32-byte record

// ------------------------------------------------------------------------
// Upsweep: particles per bucket.
// ------------------------------------------------------------------------
constexpr int kCountThreads = 512;       // blocks that share an SM (table up to 96 KB)
constexpr int kCountThreadsWide = 1024;  // one block per SM (table up to 200 KB)

#ifndef AETHER_TUNE_CHUNK_LOG
#define AETHER_TUNE_CHUNK_LOG 22
#endif
constexpr int kChunkLog = AETHER_TUNE_CHUNK_LOG;  // particles per chunk of the record layout at 64 M
                                                  // particles; see chunk_log_for

// Where a block keeps its counts while it works through a slice.
enum CountTable {
  kTableGlobal = 0,    // no table: adds go straight to the chunk's row of counts
  kTableShared32 = 1,  // 32-bit counters in shared memory (up to 200 KB: 51,200 buckets)
  kTableShared16 = 2,  // 16-bit counters, two per word (up to 102,400 buckets); a slice holds
                       // fewer than 65,536 particles, so no counter can carry into its neighbour
};
constexpr int kSlice16 = 61440;  // particles per slice with 16-bit counters (15 rounds of 4096)

template <int TABLE>
__device__ __forceinline__ void table_add(uint32_t* table, uint32_t bin, uint32_t count) {
  if (TABLE == kTableShared16) atomicAdd(&table[bin >> 1], count << (16 * (bin & 1)));
  else atomicAdd(&table[bin], count);
}

// One count per lane into `table`; lanes that hit the same bin share one add when the whole
// warp agrees or (through match.any) when neighbouring lanes do.
// Returns whether lanes shared an add (the same for all lanes): on input in random order
// they never do, and the caller then skips the votes for the rest of its round.
template <int TABLE>
__device__ __forceinline__ bool count_add(uint32_t* table, uint32_t bin, bool valid) {
  const uint32_t active = __ballot_sync(0xffffffffu, valid);
  if (active == 0) return true;
  const int first = __ffs(active) - 1;
  const uint32_t first_bin = __shfl_sync(0xffffffffu, bin, first);
  const bool uniform = __all_sync(0xffffffffu, !valid || bin == first_bin);
  if (uniform) {
    if (static_cast<int>(lane_id()) == first) table_add<TABLE>(table, first_bin, __popc(active));
    return true;
  }
  const uint32_t next_bin = __shfl_down_sync(0xffffffffu, bin, 1);
  const bool clustered = __any_sync(0xffffffffu, valid && lane_id() < 31 && next_bin == bin);
  if (clustered) {
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? bin : 0xffffffffu) & active;
    if (valid && (peers & lanemask_lt()) == 0) table_add<TABLE>(table, bin, __popc(peers));
  } else if (valid) {
    table_add<TABLE>(table, bin, 1u);
  }
  return clustered;
}

// Work unit = one slice of one chunk; a block counts the slice into its table and adds the
// table to the chunk's row of counts, count[chunk * buckets + b].
template <int TABLE, bool VEC, int THREADS>
__global__ void __launch_bounds__(THREADS)
bucket_count_kernel(const float* __restrict__ x, const float* __restrict__ y,
                    const float* __restrict__ z, const float* __restrict__ v, int64_t padded,
                    PushSpec push, int64_t n, AetherGrid g, int shift,
                    int buckets, int chunks, int chunk_log, int parts, int64_t slice,
                    uint32_t* __restrict__ bucket_count) {
  chain_begin();
  extern __shared__ uint32_t hist[];
  const int table_words = TABLE == kTableShared16 ? (buckets + 1) / 2 : buckets;
  for (int unit = blockIdx.x; unit < chunks * parts; unit += gridDim.x) {
    const int chunk = unit / parts, part = unit % parts;
    uint32_t* row = bucket_count + static_cast<size_t>(chunk) * buckets;
    if (TABLE != kTableGlobal) {
      for (int i = threadIdx.x; i < table_words; i += THREADS) hist[i] = 0;
      __syncthreads();
    }
    uint32_t* target = TABLE != kTableGlobal ? hist : row;
    const int64_t chunk_first = static_cast<int64_t>(chunk) << chunk_log;
    const int64_t chunk_last = min(static_cast<long long>(n),
                                   static_cast<long long>(chunk_first + (int64_t{1} << chunk_log)));
    const int64_t first = chunk_first + part * slice;
    const int64_t last = min(static_cast<long long>(chunk_last), static_cast<long long>(first + slice));
    const int64_t rounds = first < last ? (last - first + THREADS * 4 - 1) / (THREADS * 4) : 0;
    for (int64_t r = 0; r < rounds; ++r) {
      const int64_t i0 = first + (r * THREADS + threadIdx.x) * 4;
      float px[4], py[4], pz[4];
      if (VEC && i0 + 4 <= last) {
        const float4 a = ldcs4(x + i0), b = ldcs4(y + i0), c = ldcs4(z + i0);
        px[0] = a.x; px[1] = a.y; px[2] = a.z; px[3] = a.w;
        py[0] = b.x; py[1] = b.y; py[2] = b.z; py[3] = b.w;
        pz[0] = c.x; pz[1] = c.y; pz[2] = c.z; pz[3] = c.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const bool ok = i0 + k < last;
          px[k] = ok ? x[i0 + k] : 0.f;
          py[k] = ok ? y[i0 + k] : 0.f;
          pz[k] = ok ? z[i0 + k] : 0.f;
        }
      }
      if (push.enabled) {  // count the particles where the fused move stage puts them
        float w[3][4];
        if (VEC && i0 + 4 <= last) {
          const float4 a = ldcs4(v + i0), b = ldcs4(v + padded + i0), c = ldcs4(v + 2 * padded + i0);
          w[0][0] = a.x; w[0][1] = a.y; w[0][2] = a.z; w[0][3] = a.w;
          w[1][0] = b.x; w[1][1] = b.y; w[1][2] = b.z; w[1][3] = b.w;
          w[2][0] = c.x; w[2][1] = c.y; w[2][2] = c.z; w[2][3] = c.w;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const bool ok = i0 + k < last;
            w[0][k] = ok ? v[i0 + k] : 0.f;
            w[1][k] = ok ? v[padded + i0 + k] : 0.f;
            w[2][k] = ok ? v[2 * padded + i0 + k] : 0.f;
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          push_axis(px[k], w[0][k], push.dt, push.lo[0], push.hi[0]);
          push_axis(py[k], w[1][k], push.dt, push.lo[1], push.hi[1]);
          push_axis(pz[k], w[2][k], push.dt, push.lo[2], push.hi[2]);
        }
      }
      bool sharing = true;  // the round's first particle tells whether votes are worth it
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t bin = cell_of(px[k], py[k], pz[k], g) >> shift;
        if (sharing) sharing = count_add<TABLE>(target, bin, i0 + k < last);
        else if (i0 + k < last) table_add<TABLE>(target, bin, 1u);
      }
    }
    if (TABLE != kTableGlobal) {
      __syncthreads();
      for (int i = threadIdx.x; i < table_words; i += THREADS) {
        const uint32_t w = hist[i];
        if (TABLE == kTableShared16) {
          if (w & 0xffffu) atomicAdd(&row[2 * i], w & 0xffffu);
          if (w >> 16) atomicAdd(&row[2 * i + 1], w >> 16);
        } else if (w) {
          atomicAdd(&row[i], w);
        }
      }
      __syncthreads();
    }
  }
}

// Per bucket: particles in all chunks.
__global__ void __launch_bounds__(256)
bucket_total_kernel(const uint32_t* __restrict__ bucket_count, int buckets, int chunks,
                    uint32_t* __restrict__ total) {
  chain_begin();
  const int b = blockIdx.x * 256 + threadIdx.x;
  if (b >= buckets) return;
  uint32_t sum = 0;
  for (int c = 0; c < chunks; ++c) sum += bucket_count[static_cast<size_t>(c) * buckets + b];
  total[b] = sum;
}

// Exclusive scan of the [chunk][bucket] counts in memory order: where every run
// starts in the record array.  Two levels (1024 entries per block, then the
// block totals), then one pass that writes the run starts twice: as the scatter's
// cursors, which the scatter advances, and as the table run_begin[chunk * buckets + b]
// (with the total behind its last entry) from which the finish kernel takes the run
// of any range of buckets [b0, b1) in chunk c: run_begin[c*B + b0] .. run_begin[c*B + b1].
constexpr int kFlatScanBlock = 1024;

__global__ void __launch_bounds__(kFlatScanBlock)
run_scan_local_kernel(const uint32_t* __restrict__ count, int64_t entries,
                      uint32_t* __restrict__ local, uint32_t* __restrict__ block_sum) {
  chain_begin();
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t total;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kFlatScanBlock + threadIdx.x;
  const uint32_t v = i < entries ? count[i] : 0u;
  const uint32_t excl = block_exclusive_scan(v, warp_sum, &total);
  if (i < entries) local[i] = excl;
  if (threadIdx.x == 0) block_sum[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kFlatScanBlock)
run_scan_blocks_kernel(uint32_t* __restrict__ block_sum, int blocks) {
  chain_begin();
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t total, carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < blocks; base += kFlatScanBlock) {
    const int i = base + threadIdx.x;
    const uint32_t v = i < blocks ? block_sum[i] : 0u;
    const uint32_t excl = block_exclusive_scan(v, warp_sum, &total);
    if (i < blocks) block_sum[i] = carry + excl;
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
run_table_kernel(const uint32_t* __restrict__ local, const uint32_t* __restrict__ block_sum,
                 int64_t entries, uint32_t n, uint32_t* __restrict__ cursor,
                 uint32_t* __restrict__ run_begin) {
  chain_begin();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i > entries) return;
  const uint32_t start = i < entries ? local[i] + block_sum[i / kFlatScanBlock] : n;
  run_begin[i] = start;
  if (i < entries) cursor[i] = start;
}

// ------------------------------------------------------------------------
// Bucket starts.
// ------------------------------------------------------------------------
constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads)
bucket_scan_kernel(const uint32_t* __restrict__ bucket_count, int buckets, int64_t n,
                   const uint32_t* __restrict__ n_on_device, uint32_t capacity,
                   uint32_t* __restrict__ bucket_start, uint32_t* __restrict__ cursor,
                   Header* __restrict__ hdr) {
  chain_begin();
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t biggest;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) biggest = 0;
  __syncthreads();
  const int per = (buckets + kScanThreads - 1) / kScanThreads;
  const int first = min(buckets, tid * per), last = min(buckets, first + per);
  uint32_t sum = 0, big = 0;
  for (int b = first; b < last; ++b) {
    const uint32_t c = bucket_count[b];
    sum += c;
    big = max(big, c);
  }
  uint32_t incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sum[warp] = incl;
  if (big) atomicMax(&biggest, big);
  __syncthreads();
  if (warp == 0) {
    uint32_t w = warp_sum[lane], wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_sum[lane] = wi - w;
  }
  __syncthreads();
  uint32_t run = warp_sum[warp] + incl - sum;
  for (int b = first; b < last; ++b) {
    bucket_start[b] = run;
    if (cursor) cursor[b] = run;
    run += bucket_count[b];
  }
  if (tid == 0) {
    bucket_start[buckets] = n_on_device ? *n_on_device : static_cast<uint32_t>(n);
    hdr->max_bucket = biggest;
    // A bucket above `capacity` cannot be finished at all: hand over before the scatter runs.
    if (biggest > capacity) hdr->use_standard = 1;
  }
}

// ------------------------------------------------------------------------
// Scatter of 32-byte records into buckets.
// ------------------------------------------------------------------------
constexpr int kScatterThreads = 512;

__device__ __forceinline__ void store_record(uint32_t* dst, uint32_t key, uint32_t index, float x,
                                             float y, float z, float vx, float vy, float vz) {
  // One full 32-byte sector per record.
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(key),
               "r"(index), "r"(__float_as_uint(x)), "r"(__float_as_uint(y)),
               "r"(__float_as_uint(z)), "r"(__float_as_uint(vx)), "r"(__float_as_uint(vy)),
               "r"(__float_as_uint(vz))
               : "memory");
}

// Reserves one slot in bucket `b`.  Lanes that target the same bucket share one
// atomic: always when the whole warp agrees (cell-sorted input), and through
// match.any when at least two neighbouring lanes agree (nearly sorted input).
// Random input, where no neighbours agree, goes straight to one atomic per lane.
__device__ __forceinline__ uint32_t reserve_slot(uint32_t* cursor, uint32_t b, bool valid) {
  const uint32_t active = __ballot_sync(0xffffffffu, valid);
  if (active == 0) return 0;
  const int first = __ffs(active) - 1;
  const uint32_t first_b = __shfl_sync(0xffffffffu, b, first);
  const bool uniform = __all_sync(0xffffffffu, !valid || b == first_b);
  uint32_t slot = 0;
  if (uniform) {
    if (static_cast<int>(lane_id()) == first) slot = atomicAdd(&cursor[first_b], __popc(active));
    return __shfl_sync(0xffffffffu, slot, first) + __popc(active & lanemask_lt());
  }
  const uint32_t next_b = __shfl_down_sync(0xffffffffu, b, 1);
  const bool clustered = __any_sync(0xffffffffu, valid && lane_id() < 31 && next_b == b);
  if (clustered) {
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? b : 0xffffffffu) & active;
    const int leader = __ffs(peers) - 1;
    if (valid && static_cast<int>(lane_id()) == leader) slot = atomicAdd(&cursor[b], __popc(peers));
    slot = __shfl_sync(0xffffffffu, slot, leader < 0 ? 0 : leader) + __popc(peers & lanemask_lt());
    return slot;
  }
  if (valid) slot = atomicAdd(&cursor[b], 1u);
  return slot;
}

// ITEMS consecutive particles per thread and round (4: 128-bit loads, 2: 64-bit
// loads with twice the resident threads to keep more slot reservations in flight).
template <int ITEMS>
__device__ __forceinline__ void load_items(const float* p, float* out) {
  if (ITEMS == 4) {
    const float4 a = ldcs4(p);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  } else {
    const float2 a = __ldcs(reinterpret_cast<const float2*>(p));
    out[0] = a.x; out[1] = a.y;
  }
}

template <bool VEC, int ITEMS>
__global__ void __launch_bounds__(kScatterThreads, 8 / ITEMS)
bucket_scatter_kernel(const float* __restrict__ x, const float* __restrict__ y,
                      const float* __restrict__ z, const float* __restrict__ v, int64_t padded,
                      PushSpec push, int64_t n, AetherGrid g, uint32_t k0, uint32_t k1, int shift,
                      int buckets, int chunk_log, uint32_t* __restrict__ cursor,
                      uint32_t* __restrict__ records, const Header* __restrict__ hdr) {
  chain_begin();
  if (hdr->use_standard) return;
  const int64_t groups = (n + ITEMS - 1) / ITEMS;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kScatterThreads;
  const int64_t rounds = (groups + stride - 1) / stride;
  for (int64_t r = 0; r < rounds; ++r) {
    const int64_t i0 = (r * stride + static_cast<int64_t>(blockIdx.x) * kScatterThreads +
                        threadIdx.x) * ITEMS;
    float f[6][ITEMS];
    if (VEC && i0 + ITEMS <= n) {
      load_items<ITEMS>(x + i0, f[0]);
      load_items<ITEMS>(y + i0, f[1]);
      load_items<ITEMS>(z + i0, f[2]);
      if (v) {
        load_items<ITEMS>(v + i0, f[3]);
        load_items<ITEMS>(v + padded + i0, f[4]);
        load_items<ITEMS>(v + 2 * padded + i0, f[5]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        const bool ok = i0 + k < n;
        f[0][k] = ok ? x[i0 + k] : 0.f;
        f[1][k] = ok ? y[i0 + k] : 0.f;
        f[2][k] = ok ? z[i0 + k] : 0.f;
        f[3][k] = ok && v ? v[i0 + k] : 0.f;
        f[4][k] = ok && v ? v[padded + i0 + k] : 0.f;
        f[5][k] = ok && v ? v[2 * padded + i0 + k] : 0.f;
      }
    }
    if (!v) {
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) f[3][k] = f[4][k] = f[5][k] = 0.f;
    }
    if (push.enabled) {  // the fused move stage: the record carries the moved particle
#pragma unroll
      for (int k = 0; k < ITEMS; ++k) {
        push_axis(f[0][k], f[3][k], push.dt, push.lo[0], push.hi[0]);
        push_axis(f[1][k], f[4][k], push.dt, push.lo[1], push.hi[1]);
        push_axis(f[2][k], f[5][k], push.dt, push.lo[2], push.hi[2]);
      }
    }
    uint32_t key[ITEMS], slot[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const uint32_t cell = cell_of(f[0][k], f[1][k], f[2][k], g);
      const uint32_t run = static_cast<uint32_t>((i0 + k) >> chunk_log) * buckets + (cell >> shift);
      slot[k] = reserve_slot(cursor, run, i0 + k < n);
      key[k] = make_key(cell, static_cast<uint32_t>(i0 + k), k0, k1);
    }
#pragma unroll
    for (int k = 0; k < ITEMS; ++k)
      if (i0 + k < n)
        store_record(records + static_cast<size_t>(slot[k]) * kRecordWords, key[k],
                     static_cast<uint32_t>(i0 + k), f[0][k], f[1][k], f[2][k], f[3][k], f[4][k],
                     f[5][k]);
  }
}

// ------------------------------------------------------------------------
// Segmented input (the local sort of the sliced multi-GPU exchange): the particles of one
// slice are up to kMaxWorld index ranges of the input arrays, known on the device only.
// ------------------------------------------------------------------------
constexpr int kSegmentUnit = 16384;  // particles per work unit of the segment kernels

// Work unit `unit` of slice `k`: the units of source 0's segment, then source 1's, ...  Each
// segment is cut from its 4-aligned start in pieces of kSegmentUnit, so that the 16-byte loads
// stay aligned.  Returns false past the last unit; else [first, last) is the piece (first a
// multiple of 4) and `lo` the first index in it that belongs to the segment.
__device__ __forceinline__ bool segment_unit(const SliceSegments* __restrict__ seg, int k, int unit,
                                             int64_t* first, int64_t* last, int64_t* lo) {
  const int sources = static_cast<int>(seg->sources);
  for (int s = 0; s < sources; ++s) {
    const int64_t begin = seg->first[k][s], length = seg->length[k][s];
    if (length == 0) continue;
    const int64_t base = begin & ~int64_t{3};
    const int units = static_cast<int>((begin + length - base + kSegmentUnit - 1) / kSegmentUnit);
    if (unit < units) {
      *first = base + static_cast<int64_t>(unit) * kSegmentUnit;
      *last = min(static_cast<long long>(begin + length), static_cast<long long>(*first + kSegmentUnit));
      *lo = max(static_cast<long long>(begin), static_cast<long long>(*first));
      return true;
    }
    unit -= units;
  }
  return false;
}

// Particles per bucket of one slice, added to the slice's row of counts.  `capacity` is the
// length of the input arrays (vector loads must not pass it).
template <int TABLE, int THREADS>
__global__ void __launch_bounds__(THREADS)
bucket_count_segments_kernel(const float* __restrict__ x, const float* __restrict__ y,
                             const float* __restrict__ z, int64_t capacity, bool vec,
                             const SliceSegments* __restrict__ seg, int k, AetherGrid g, int shift,
                             int buckets, uint32_t* __restrict__ row) {
  extern __shared__ uint32_t hist[];
  if (TABLE != kTableGlobal) {
    for (int i = threadIdx.x; i < buckets; i += THREADS) hist[i] = 0;
    __syncthreads();
  }
  uint32_t* target = TABLE != kTableGlobal ? hist : row;
  int64_t first, last, lo;
  for (int unit = blockIdx.x; segment_unit(seg, k, unit, &first, &last, &lo); unit += gridDim.x) {
    // Every thread of the block makes the same number of rounds: the adds below use
    // warp-wide votes, which all 32 lanes must reach.
    for (int64_t round = first; round < last; round += THREADS * 4) {
      const int64_t i0 = round + static_cast<int64_t>(threadIdx.x) * 4;
      float px[4], py[4], pz[4];
      if (vec && i0 + 4 <= capacity) {
        const float4 a = ldcs4(x + i0), b = ldcs4(y + i0), c = ldcs4(z + i0);
        px[0] = a.x; px[1] = a.y; px[2] = a.z; px[3] = a.w;
        py[0] = b.x; py[1] = b.y; py[2] = b.z; py[3] = b.w;
        pz[0] = c.x; pz[1] = c.y; pz[2] = c.z; pz[3] = c.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool ok = i0 + j >= lo && i0 + j < last;
          px[j] = ok ? x[i0 + j] : 0.f;
          py[j] = ok ? y[i0 + j] : 0.f;
          pz[j] = ok ? z[i0 + j] : 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        count_add<TABLE>(target, cell_of(px[j], py[j], pz[j], g) >> shift,
                         i0 + j >= lo && i0 + j < last);
    }
  }
  if (TABLE != kTableGlobal) {
    __syncthreads();
    for (int i = threadIdx.x; i < buckets; i += THREADS)
      if (hist[i]) atomicAdd(&row[i], hist[i]);
  }
}

// Exclusive scan of one slice's row of counts, offset by the records of the slices before it:
// the scatter's cursors and the finish kernel's run_begin row of that chunk.  One block.
// STAGED: the row fits shared memory (padded against bank conflicts); it is read and written
// once, coalesced, and every thread scans a contiguous piece of it.  Otherwise 1024 entries
// at a time.
constexpr int kStagedScanMax = 48 * 1024;  // buckets whose row (plus padding) fits 200 KB

template <bool STAGED>
__global__ void __launch_bounds__(kFlatScanBlock)
chunk_scan_kernel(const uint32_t* __restrict__ row, int buckets,
                  const SliceSegments* __restrict__ seg, int k, uint32_t* __restrict__ cursor_row,
                  uint32_t* __restrict__ run_begin_row) {
  extern __shared__ uint32_t staged[];
  __shared__ uint32_t warp_sum[32];
  __shared__ uint32_t total, carry;
  if (STAGED) {
    const int per = (buckets + kFlatScanBlock - 1) / kFlatScanBlock;
    const int pad = 1 + (per & 1);  // pieces an odd number of words apart: no bank conflicts
    auto at = [per, pad](int i) { return i + i / per * pad; };
    for (int i = threadIdx.x; i < buckets; i += kFlatScanBlock) staged[at(i)] = row[i];
    __syncthreads();
    const int first = min(buckets, static_cast<int>(threadIdx.x) * per);
    const int last = min(buckets, first + per);
    uint32_t sum = 0;
    for (int b = first; b < last; ++b) sum += staged[at(b)];
    uint32_t run = seg->chunk_base[k] + block_exclusive_scan(sum, warp_sum, &total);
    for (int b = first; b < last; ++b) {
      const uint32_t here = staged[at(b)];
      staged[at(b)] = run;
      run += here;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < buckets; i += kFlatScanBlock) {
      const uint32_t start = staged[at(i)];
      cursor_row[i] = start;
      run_begin_row[i] = start;
    }
  } else {
    if (threadIdx.x == 0) carry = seg->chunk_base[k];
    __syncthreads();
    for (int base = 0; base < buckets; base += kFlatScanBlock) {
      const int i = base + threadIdx.x;
      const uint32_t v = i < buckets ? row[i] : 0u;
      const uint32_t excl = block_exclusive_scan(v, warp_sum, &total);
      if (i < buckets) {
        cursor_row[i] = carry + excl;
        run_begin_row[i] = carry + excl;
      }
      __syncthreads();
      if (threadIdx.x == 0) carry += total;
      __syncthreads();
    }
  }
  // Behind the last chunk's row: the end of the last run.
  if (k + 1 == static_cast<int>(seg->slices) && threadIdx.x == 0) run_begin_row[buckets] = seg->n;
}

// Records of one slice into the runs of chunk k.
template <int ITEMS>
__global__ void __launch_bounds__(kScatterThreads, 8 / ITEMS)
bucket_scatter_segments_kernel(const float* __restrict__ x, const float* __restrict__ y,
                               const float* __restrict__ z, const float* __restrict__ v,
                               int64_t padded, int64_t capacity, bool vec,
                               const SliceSegments* __restrict__ seg, int k, AetherGrid g,
                               uint32_t k0, uint32_t k1, int shift, int buckets,
                               uint32_t* __restrict__ cursor_row, uint32_t* __restrict__ records) {
  int64_t first, last, lo;
  for (int unit = blockIdx.x; segment_unit(seg, k, unit, &first, &last, &lo); unit += gridDim.x) {
    // Every thread of the block makes the same number of rounds: the slot reservation uses
    // warp-wide votes, which all 32 lanes must reach.
    for (int64_t round = first; round < last; round += kScatterThreads * ITEMS) {
      const int64_t i0 = round + static_cast<int64_t>(threadIdx.x) * ITEMS;
      float f[6][ITEMS];
      if (vec && i0 + ITEMS <= capacity) {
        load_items<ITEMS>(x + i0, f[0]);
        load_items<ITEMS>(y + i0, f[1]);
        load_items<ITEMS>(z + i0, f[2]);
        load_items<ITEMS>(v + i0, f[3]);
        load_items<ITEMS>(v + padded + i0, f[4]);
        load_items<ITEMS>(v + 2 * padded + i0, f[5]);
      } else {
#pragma unroll
        for (int j = 0; j < ITEMS; ++j) {
          const bool ok = i0 + j >= lo && i0 + j < last;
          f[0][j] = ok ? x[i0 + j] : 0.f;
          f[1][j] = ok ? y[i0 + j] : 0.f;
          f[2][j] = ok ? z[i0 + j] : 0.f;
          f[3][j] = ok ? v[i0 + j] : 0.f;
          f[4][j] = ok ? v[padded + i0 + j] : 0.f;
          f[5][j] = ok ? v[2 * padded + i0 + j] : 0.f;
        }
      }
      uint32_t key[ITEMS], slot[ITEMS];
#pragma unroll
      for (int j = 0; j < ITEMS; ++j) {
        const bool ok = i0 + j >= lo && i0 + j < last;
        const uint32_t cell = cell_of(f[0][j], f[1][j], f[2][j], g);
        slot[j] = reserve_slot(cursor_row, cell >> shift, ok);
        key[j] = make_key(cell, static_cast<uint32_t>(i0 + j), k0, k1);
      }
#pragma unroll
      for (int j = 0; j < ITEMS; ++j)
        if (i0 + j >= lo && i0 + j < last)
          store_record(records + static_cast<size_t>(slot[j]) * kRecordWords, key[j],
                       static_cast<uint32_t>(i0 + j), f[0][j], f[1][j], f[2][j], f[3][j], f[4][j],
                       f[5][j]);
    }
  }
}

// ------------------------------------------------------------------------
// Groups: consecutive buckets that one block finishes together.
// ------------------------------------------------------------------------
// One thread per aligned block of 2^group_shift buckets cuts it, greedily from the bucket
// totals, into groups of consecutive buckets with at most `capacity` records, and appends
// them (first bucket, end bucket) to the group list; their order in the list is of no
// consequence.  A bucket that exceeds the capacity on its own is not listed:
// bucket_finish_large_kernel takes it.
__global__ void __launch_bounds__(256)
group_cut_kernel(const uint32_t* __restrict__ bucket_start, int buckets, int group_shift,
                 uint32_t capacity, uint2* __restrict__ groups, uint32_t* __restrict__ group_count) {
  chain_begin();
  const int block_of_buckets = blockIdx.x * 256 + threadIdx.x;
  const int b_first = block_of_buckets << group_shift;
  if (b_first >= buckets) return;
  const int b_last = min(buckets, b_first + (1 << group_shift));
  uint32_t base = 0;
  for (int pass = 0; pass < 2; ++pass) {
    uint32_t found = 0;
    int b0 = b_first;
    uint32_t begin = bucket_start[b0];
    while (b0 < b_last) {
      int b1 = b0 + 1;
      uint32_t end = bucket_start[b1];
      const bool fits = end - begin <= capacity;
      if (fits) {
        while (b1 < b_last) {
          const uint32_t further = bucket_start[b1 + 1];
          if (further - begin > capacity) break;
          end = further;
          ++b1;
        }
        if (pass == 1) groups[base + found] = make_uint2(static_cast<uint32_t>(b0), static_cast<uint32_t>(b1));
        ++found;
      }
      b0 = b1;
      begin = end;
    }
    if (pass == 0) {
      if (found == 0) return;
      base = atomicAdd(group_count, found);
    }
  }
}

// Words of one row of a group's table: one entry per chunk and three more, rounded up to
// whole 16-byte pieces (the finish kernel fetches the tables with 16-byte copies).
__host__ __device__ inline int table_row_words(int chunks) { return (chunks + 3 + 3) / 4 * 4; }

// Where the records of every group lie: per group two rows of table_row_words(chunks) words,
//   row 0: [c] first record of the group's run in chunk c; [chunks] first output slot of the
//          group; [chunks + 1], [chunks + 2] its buckets b0, b1
//   row 1: [c] records of the group in chunks before c; [chunks] records of the group.
// One warp per group, a lane per chunk.
__global__ void __launch_bounds__(256)
group_table_kernel(const uint2* __restrict__ groups, const uint32_t* __restrict__ group_count,
                   const uint32_t* __restrict__ bucket_start, const uint32_t* __restrict__ run_begin,
                   int chunks, int buckets, uint32_t* __restrict__ tables) {
  chain_begin();
  const int lane = threadIdx.x & 31;
  const uint32_t total = *group_count;
  const int row_words = table_row_words(chunks);
  for (uint32_t g = blockIdx.x * 8 + (threadIdx.x >> 5); g < total; g += gridDim.x * 8) {
    const uint2 group = groups[g];
    uint32_t* row0 = tables + static_cast<size_t>(g) * 2 * row_words;
    uint32_t* row1 = row0 + row_words;
    uint32_t offset = 0;
    for (int c0 = 0; c0 < chunks; c0 += 32) {
      const int c = c0 + lane;
      uint32_t length = 0, start = 0;
      if (c < chunks) {
        const size_t row = static_cast<size_t>(c) * buckets;
        start = run_begin[row + group.x];
        length = run_begin[row + group.y] - start;
      }
      uint32_t incl = length;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (c < chunks) {
        row0[c] = start;
        row1[c] = offset + incl - length;
      }
      offset += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      row0[chunks] = bucket_start[group.x];
      row0[chunks + 1] = group.x;
      row0[chunks + 2] = group.y;
      row1[chunks] = offset;
    }
  }
}

// ------------------------------------------------------------------------
// Finish: a block sorts one group of buckets in shared memory and writes the output.
// ------------------------------------------------------------------------
constexpr uint32_t kBulkChunkBytes = 32768;  // bytes per bulk copy
constexpr uint32_t kBulkWaitLimit = 1u << 24;  // polls of the copy barrier
constexpr int kMaxSegments = 32;  // runs of cells an oversized bucket is cut into
constexpr int kMaxGroupBuckets = 512;  // buckets in the aligned block a group may not leave
constexpr int kMaxChunks = 256;        // 2^30 particles in chunks of 2^22
constexpr int kTableRowWords = (kMaxChunks + 3 + 3) / 4 * 4;

// Two shapes of the finish kernel.  The small one runs two blocks per multiprocessor, so that
// one block's bulk copy and output stores overlap the other's ranking; it wants buckets of
// about a thousand records, which the count kernel's table can only offer up to about a
// hundred million particles.  Above that the large shape (one block per multiprocessor) runs.
template <int THREADS, int CAPACITY, int LOW_BITS>
struct FinishShape {
  static constexpr int kThreads = THREADS;
  static constexpr int kCapacity = CAPACITY;                // records a block holds
  static constexpr int kItems = (CAPACITY + THREADS - 1) / THREADS;
  static constexpr int kLowBits = LOW_BITS;                 // key bits the counters resolve
  static constexpr int kHistWords = (1 << LOW_BITS) / 4;    // byte counters, 4 per word
  static constexpr int kWordsPerThread = kHistWords / THREADS;
  // A group spans at most this many cells: its low key (cell in group, shuffle bits) then has
  // at most LOW_BITS + 2 bits, two of which the tie step may take.
  static constexpr int kMaxCells = 1 << (LOW_BITS + 2 - kShuffleBits);
  static constexpr uint32_t kLargestBucket = static_cast<uint32_t>(kMaxSegments) * CAPACITY;
  static_assert(kWordsPerThread == 8, "the counter scan reads eight words per thread");
  static_assert(kHistWords >= CAPACITY, "the tie step lays one word per record over the counters");
};
using FinishSmall = FinishShape<512, 2560, 14>;
using FinishLarge = FinishShape<1024, 5120, 15>;

template <class Shape>
struct __align__(128) FinishSmem {
  uint32_t raw[Shape::kCapacity * kRecordWords];  // the group's records as they lie in HBM
  uint32_t hist[Shape::kHistWords];     // byte counter per low-key value
  uint16_t word_prefix[Shape::kHistWords];  // exclusive prefix of each counter word
  uint16_t order[Shape::kCapacity];     // record held by each sorted slot
  uint32_t warp_sum[32];
  uint32_t total;
  uint32_t gave_up;
  unsigned long long barrier;    // mbarrier of the bulk copy
  uint32_t seg_begin[kMaxSegments + 1];  // oversized bucket: records before each run of cells
  uint16_t seg_first[kMaxSegments + 1];  // ... and the first cell of each run
  uint32_t fill;                         // ... and the records picked so far for the run at hand
};
// Behind the structure, in the same dynamic allocation: the tables of three consecutive
// groups, 2 * row_words words each (at most kTableRowWords per row).
constexpr size_t kSmallShapeTableBytes = 3 * 2 * 16 * sizeof(uint32_t);  // up to 13 chunks
static_assert(sizeof(FinishSmem<FinishLarge>) + 3 * 2 * kTableRowWords * sizeof(uint32_t) <=
                  227 * 1024, "finish kernel shared memory");
static_assert(2 * (sizeof(FinishSmem<FinishSmall>) + kSmallShapeTableBytes + 1024) <= 228 * 1024,
              "two small finish blocks must share a multiprocessor");

template <class Shape>
__device__ __forceinline__ uint32_t* group_table(FinishSmem<Shape>& s, int q, int row_words) {
  return reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(&s) + sizeof(FinishSmem<Shape>)) +
         q * 2 * row_words;
}

__device__ __forceinline__ uint32_t byte_sum(uint32_t w) { return __dp4a(w, 0x01010101u, 0u); }

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Copies `bytes` (a multiple of 16, both addresses 16-byte aligned) from global
// to shared memory with the bulk-copy engine, in pieces of at most 32 KB; the
// bytes are counted on the mbarrier, which must already expect them.
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes,
                                          unsigned long long* barrier) {
  const uint32_t bar = smem_addr(barrier);
  for (uint32_t done = 0; done < bytes; done += kBulkChunkBytes) {
    const uint32_t part = min(kBulkChunkBytes, bytes - done);
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_addr(static_cast<unsigned char*>(dst) + done)),
          "l"(static_cast<const unsigned char*>(src) + done), "r"(part), "r"(bar)
        : "memory");
  }
}

// Waits (bounded) for the phase `parity` of the copy barrier; false if it gave up: after
// kBulkWaitLimit polls, or after about two seconds on the global timer (a single poll may
// itself wait a while inside the hardware), whichever comes first.
__device__ __forceinline__ bool bulk_load_wait(unsigned long long* barrier, uint32_t parity) {
  const uint32_t bar = smem_addr(barrier);
  unsigned long long started = 0;
  for (uint32_t polls = 0; polls < kBulkWaitLimit; ++polls) {
    uint32_t ready;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ready) : "r"(bar), "r"(parity) : "memory");
    if (ready) return true;
    if ((polls & 1023u) == 1023u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (started == 0) started = now;
      else if (now - started > 2000000000ull) return false;
    }
  }
  return false;
}

// Output arrays of the finish kernel.
struct FinishOut {
  uint32_t* keys;
  int32_t* index;
  int32_t* cell_counts;
  int32_t* cell_start;
  float* xs;
  float* ys;
  float* zs;
  float* vs;
  int64_t padded_sorted;
};

// Key bits the byte counters must leave to the tie step for a set of `cells` cells.
template <class Shape>
__device__ __forceinline__ int drop_for(int cells) {
  const int low_bits = (cells <= 1 ? 0 : 32 - __clz(cells - 1)) + kShuffleBits;
  return max(0, low_bits - Shape::kLowBits);
}

// Sorts the `count` records staged in s.raw (any order) and writes them to the
// output from slot `begin` on.  The records belong to the cells first_cell ..
// first_cell + cells_here - 1 (at most Shape::kMaxCells).  The low key of a record is
// its key minus the key of the first cell's first shuffle value; the counters resolve
// all but its `drop` lowest bits, which the tie step orders together with the index.
// s.hist must be zero over the counters used; the call leaves it overwritten.
// Returns false if a byte counter wrapped (more than 255 records on one counter).
template <class Shape>
__device__ __forceinline__ bool sort_staged(FinishSmem<Shape>& s, const FinishOut& out, int count,
                                            uint32_t begin, int64_t first_cell, int cells_here,
                                            int drop) {
  constexpr int kThreads = Shape::kThreads, kItems = Shape::kItems;
  constexpr int kWordsPerThread = Shape::kWordsPerThread;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t key_base = static_cast<uint32_t>(first_cell) << kShuffleBits;
  const uint32_t drop_mask = (1u << drop) - 1;
  const int cell_words = 32 >> drop;  // counter words per cell
  const int hist_words = max(8, cells_here * cell_words);

  // Count the low key bits with byte-wide counters; the value an add returns
  // is the record's rank among the records of its counter.
  uint32_t packed[kItems];  // counter id | rank << 16
  uint32_t mine[kItems];    // what orders the records of one counter: dropped key bits, index
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    const int r = tid + k * kThreads;
    packed[k] = 0;
    mine[k] = 0;
    if (r < count) {
      // Key and index in one access: it costs the same bank conflicts as the key alone.
      const uint2 key_index = *reinterpret_cast<const uint2*>(&s.raw[r * kRecordWords]);
      const uint32_t low = (key_index.x - key_base) >> drop;
      const int sh = 8 * (low & 3);
      const uint32_t old = atomicAdd(&s.hist[low >> 2], 1u << sh);
      packed[k] = low | (((old >> sh) & 0xffu) << 16);
      mine[k] = ((key_index.x & drop_mask) << 30) | key_index.y;
    }
  }
  __syncthreads();

  // Exclusive scan of the counters (8 words = 32 counters per thread, fetched
  // as two 128-bit loads so that neighbouring threads do not collide on banks).
  uint32_t local[kWordsPerThread];
  uint32_t sum = 0;
  {
    uint32_t w[kWordsPerThread];
    const uint4 a = *reinterpret_cast<const uint4*>(&s.hist[tid * kWordsPerThread]);
    const uint4 c = *reinterpret_cast<const uint4*>(&s.hist[tid * kWordsPerThread + 4]);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    w[4] = c.x; w[5] = c.y; w[6] = c.z; w[7] = c.w;
#pragma unroll
    for (int j = 0; j < kWordsPerThread; ++j) {
      local[j] = sum;
      sum += tid * kWordsPerThread + j < hist_words ? byte_sum(w[j]) : 0u;
    }
  }
  uint32_t incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s.warp_sum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t w = lane < kThreads / 32 ? s.warp_sum[lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    s.warp_sum[lane] = wi - w;
    if (lane == 31) s.total = wi;
  }
  __syncthreads();
  const uint32_t thread_base = s.warp_sum[warp] + incl - sum;
  if (tid * kWordsPerThread < hist_words) {  // hist_words is a multiple of 8
    uint4 packed_prefix;
    packed_prefix.x = (thread_base + local[0]) | ((thread_base + local[1]) << 16);
    packed_prefix.y = (thread_base + local[2]) | ((thread_base + local[3]) << 16);
    packed_prefix.z = (thread_base + local[4]) | ((thread_base + local[5]) << 16);
    packed_prefix.w = (thread_base + local[6]) | ((thread_base + local[7]) << 16);
    *reinterpret_cast<uint4*>(&s.word_prefix[tid * kWordsPerThread]) = packed_prefix;
  }
  // A byte counter that wrapped loses 256 from the total.
  const bool wrapped = s.total != static_cast<uint32_t>(count);
  __syncthreads();
  if (wrapped) return false;

  // Cell tables: every cell is 128 >> drop consecutive counters.
  for (int c = tid; c < cells_here; c += kThreads) {
    const uint32_t lo = s.word_prefix[c * cell_words];
    const uint32_t hi = (c + 1) * cell_words < hist_words ? s.word_prefix[(c + 1) * cell_words]
                                                           : static_cast<uint32_t>(count);
    out.cell_start[first_cell + c] = static_cast<int32_t>(begin + lo);
    out.cell_counts[first_cell + c] = static_cast<int32_t>(hi - lo);
  }

  // Sorted slot of every record: start of its counter's run + arrival rank.  A
  // counter held by one record only (the usual case) is final at once.
  uint32_t run[kItems];  // run start | run length << 16, for records that share a counter
#pragma unroll
  for (int k = 0; k < kItems; ++k) {
    const int r = tid + k * kThreads;
    run[k] = 0;
    if (r < count) {
      const uint32_t low = packed[k] & 0xffffu, rank = packed[k] >> 16;
      const uint32_t word = s.hist[low >> 2];
      const int sh = 8 * (low & 3);
      const uint32_t start = s.word_prefix[low >> 2] + byte_sum(word & ((1u << sh) - 1u));
      const uint32_t length = (word >> sh) & 0xffu;
      if (length > 1) run[k] = start | (length << 16);
      else s.order[start] = static_cast<uint16_t>(r);
    }
  }
  __syncthreads();

  // Records that share a counter must appear in ascending (dropped key bits,
  // original index): a record inside such a run goes to (run start + number of
  // smaller records in the run).  Indices stay below 2^30, so the dropped bits
  // ride above them in one word.  The words to compare are laid out run by run
  // over the counters, which nobody reads any more: a run is then a few
  // neighbouring words instead of as many records scattered over s.raw.
  uint32_t* tie = s.hist;
#pragma unroll
  for (int k = 0; k < kItems; ++k)
    if (run[k]) tie[(run[k] & 0xffffu) + (packed[k] >> 16)] = mine[k];
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kItems; ++k)
    if (run[k]) {
      const uint32_t start = run[k] & 0xffffu, length = run[k] >> 16;
      uint32_t smaller = 0;
      // Most runs are two or three records: four independent loads, then the rare rest.
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j)
        if (j < length) smaller += tie[start + j] < mine[k];
      for (uint32_t j = 4; j < length; ++j) smaller += tie[start + j] < mine[k];
      s.order[start + smaller] = static_cast<uint16_t>(tid + k * kThreads);
    }
  __syncthreads();

  // Coalesced output.  Two neighbouring lanes pull one record out of shared memory, a half
  // each (a quarter warp then reads four whole records: fewer bank conflicts than eight
  // halves of eight records), and write their four words to four of the eight output arrays.
  {
    const int half = tid & 1;
    uint32_t* const o0 = half ? reinterpret_cast<uint32_t*>(out.zs) : out.keys;
    uint32_t* const o1 = half ? reinterpret_cast<uint32_t*>(out.vs)
                              : reinterpret_cast<uint32_t*>(out.index);
    uint32_t* const o2 = half ? (out.vs ? reinterpret_cast<uint32_t*>(out.vs + out.padded_sorted) : nullptr)
                              : reinterpret_cast<uint32_t*>(out.xs);
    uint32_t* const o3 = half ? (out.vs ? reinterpret_cast<uint32_t*>(out.vs + 2 * out.padded_sorted) : nullptr)
                              : reinterpret_cast<uint32_t*>(out.ys);
    int next = tid >> 1 < count ? s.order[tid >> 1] : 0;  // one round ahead of its use
    for (int d = tid >> 1; d < count; d += kThreads / 2) {
      const int rec = next;
      if (d + kThreads / 2 < count) next = s.order[d + kThreads / 2];
      const uint4 a = *reinterpret_cast<const uint4*>(&s.raw[rec * kRecordWords + 4 * half]);
      const size_t o = static_cast<size_t>(begin) + d;
      if (o0) __stcs(o0 + o, a.x);  // keys-only calls leave the payload out
      if (o1) __stcs(o1 + o, a.y);
      if (o2) __stcs(o2 + o, a.z);
      if (o3) __stcs(o3 + o, a.w);
    }
  }
  __syncthreads();
  return true;
}

// What the finish kernels need to find the records of a range of buckets.
struct RunTable {
  const uint32_t* records;
  const uint32_t* bucket_start;  // [buckets + 1]: records before each bucket, all chunks
  const uint32_t* run_begin;     // [chunks * buckets + 1]: first record of run (chunk, bucket)
  const uint32_t* tables;        // two rows of row_words words per group (group_table_kernel)
  const uint32_t* group_count;
  int row_words;
  int chunks;
  int buckets;
  int shift;                     // a bucket is 2^shift cells
};

// A bucket with more records than shared memory holds (a dense region: the
// bucket width is planned from the average load).  The block counts the
// bucket's records per cell, cuts the cells into up to kMaxSegments runs that
// fit, and for every run picks the run's records out of the bucket (which it
// reads from global memory once per run) and sorts them like a small group.
// Returns false if it cannot (a single cell larger than shared memory, too many
// runs, or a wrapped byte counter): the call then goes to the digit passes.
template <class Shape>
__device__ bool finish_large_bucket(FinishSmem<Shape>& s, const FinishOut& out, const RunTable& t,
                                    int b, uint32_t begin, int count, int64_t first_cell,
                                    int cells_here) {
  constexpr int kThreads = Shape::kThreads, kCapacity = Shape::kCapacity;
  const int tid = threadIdx.x;
  uint32_t* cell_count = s.hist;  // one word per cell; s.hist is free until a run is sorted
  for (int c = tid; c < cells_here; c += kThreads) cell_count[c] = 0;
  __syncthreads();
  // Per-cell counts: one pass over the keys of the bucket's records.
  for (int c = 0; c < t.chunks; ++c) {
    const size_t entry = static_cast<size_t>(c) * t.buckets + b;
    const uint32_t start = t.run_begin[entry], length = t.run_begin[entry + 1] - start;
    for (uint32_t i = tid; i < length; i += kThreads) {
      const uint32_t key = __ldg(t.records + static_cast<size_t>(start + i) * kRecordWords);
      atomicAdd(&cell_count[(key >> kShuffleBits) - static_cast<uint32_t>(first_cell)], 1u);
    }
  }
  __syncthreads();
  // Cut into runs of cells that fit (one thread; at most Shape::kMaxCells cells).
  if (tid == 0) {
    int segments = 0;
    uint32_t load = 0, before = 0;
    bool ok = true;
    s.seg_first[0] = 0;
    s.seg_begin[0] = 0;
    for (int c = 0; c < cells_here && ok; ++c) {
      const uint32_t here = cell_count[c];
      if (here > static_cast<uint32_t>(kCapacity)) ok = false;
      if (load + here > static_cast<uint32_t>(kCapacity)) {  // close the run before cell c
        before += load;
        load = 0;
        ++segments;
        if (segments >= kMaxSegments) { ok = false; break; }
        s.seg_first[segments] = static_cast<uint16_t>(c);
        s.seg_begin[segments] = before;
      }
      load += here;
    }
    if (ok) {
      ++segments;
      s.seg_first[segments] = static_cast<uint16_t>(cells_here);
      s.seg_begin[segments] = before + load;
    }
    s.total = ok ? static_cast<uint32_t>(segments) : 0u;
  }
  __syncthreads();
  const int segments = static_cast<int>(s.total);
  __syncthreads();
  if (segments == 0) return false;
  for (int k = 0; k < segments; ++k) {
    const int c0 = s.seg_first[k], c1 = s.seg_first[k + 1];
    const uint32_t seg_begin = s.seg_begin[k];
    const int seg_count = static_cast<int>(s.seg_begin[k + 1] - seg_begin);
    const int drop = drop_for<Shape>(c1 - c0);
    // Zero the counters of this run and the fill cursor (cell_count is overwritten
    // from here on; the cuts above are already in seg_first / seg_begin).
    const int words = max(8, (c1 - c0) * (32 >> drop));
    for (int i = tid; i < words; i += kThreads) s.hist[i] = 0;
    if (tid == 0) s.fill = 0;
    __syncthreads();
    for (int c = 0; c < t.chunks; ++c) {
      const size_t entry = static_cast<size_t>(c) * t.buckets + b;
      const uint32_t start = t.run_begin[entry], length = t.run_begin[entry + 1] - start;
      for (uint32_t i = tid; i < length; i += kThreads) {
        const uint4* rec = reinterpret_cast<const uint4*>(t.records +
                                                          static_cast<size_t>(start + i) * kRecordWords);
        const uint4 lo = __ldg(rec);
        const int cell = static_cast<int>((lo.x >> kShuffleBits) - static_cast<uint32_t>(first_cell));
        if (cell >= c0 && cell < c1) {
          const uint32_t slot = atomicAdd(&s.fill, 1u);
          if (slot < static_cast<uint32_t>(kCapacity)) {
            *reinterpret_cast<uint4*>(&s.raw[slot * kRecordWords]) = lo;
            *reinterpret_cast<uint4*>(&s.raw[slot * kRecordWords + 4]) = __ldg(rec + 1);
          }
        }
      }
    }
    __syncthreads();
    const bool consistent = s.fill == static_cast<uint32_t>(seg_count);
    __syncthreads();
    if (!consistent) return false;
    if (!sort_staged<Shape>(s, out, seg_count, begin + seg_begin, first_cell + c0, c1 - c0, drop))
      return false;
  }
  return true;
}

__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Starts the asynchronous copy of the table of group `g` (if there is one) into set `q`.
template <class Shape>
__device__ __forceinline__ void fetch_table(FinishSmem<Shape>& s, int q, const RunTable& t,
                                            uint32_t g, uint32_t groups) {
  const int pieces = 2 * t.row_words / 4;  // 16-byte pieces of the two rows
  if (g >= groups || static_cast<int>(threadIdx.x) >= pieces) return;
  const uint32_t* src = t.tables + static_cast<size_t>(g) * 2 * t.row_words + threadIdx.x * 4;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   smem_addr(group_table(s, q, t.row_words) + threadIdx.x * 4)), "l"(src) : "memory");
}

// Warp 0: the runs of the group whose table is in set `q`, one per chunk.  FETCH: bulk copies
// back to back into s.raw, counted on the barrier (lane 0 tells it first how many bytes to
// expect); otherwise only a request to bring the runs into L2, for the group after.
template <class Shape, bool FETCH>
__device__ __forceinline__ void touch_runs(FinishSmem<Shape>& s, int q, const RunTable& t) {
  const int lane = threadIdx.x & 31;
  const uint32_t* run_first = group_table(s, q, t.row_words);
  const uint32_t* run_offset = run_first + t.row_words;
  const uint32_t count = run_offset[t.chunks];
  if (count == 0) return;
  if (FETCH) {
    if (lane == 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                       smem_addr(&s.barrier)), "r"(count * kRecordWords * 4u) : "memory");
    }
    __syncwarp();
  }
  for (int c = lane; c < t.chunks; c += 32) {
    const uint32_t length = run_offset[c + 1] - run_offset[c];
    if (length == 0) continue;
    const uint32_t* src = t.records + static_cast<size_t>(run_first[c]) * kRecordWords;
    if (FETCH) {
      if (run_offset[c + 1] <= static_cast<uint32_t>(Shape::kCapacity))
        bulk_copy(s.raw + static_cast<size_t>(run_offset[c]) * kRecordWords, src,
                  length * kRecordWords * 4u, &s.barrier);
    } else {
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src),
                   "r"(length * kRecordWords * 4u) : "memory");
    }
  }
}

// A block works through groups blockIdx.x, blockIdx.x + gridDim.x, ... of the group list.
// What it needs to know about a group (where its runs lie) arrives two groups ahead by
// asynchronous copies; a group's records are asked into L2 while the group before it is
// sorted, and copied into shared memory as soon as that one's output is written.
template <class Shape>
__global__ void __launch_bounds__(Shape::kThreads, Shape::kThreads <= 512 ? 2 : 1)
bucket_finish_kernel(RunTable t, int64_t n, const uint32_t* __restrict__ n_on_device,
                     int64_t num_cells, FinishOut out, Header* __restrict__ hdr) {
  chain_begin();
  if (hdr->use_standard) return;
  constexpr int kThreads = Shape::kThreads;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FinishSmem<Shape>& s = *reinterpret_cast<FinishSmem<Shape>*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t groups = *t.group_count;
  if (blockIdx.x == 0 && tid == 0)
    out.cell_start[num_cells] = n_on_device ? static_cast<int32_t>(*n_on_device) : static_cast<int32_t>(n);
  const uint32_t stride = gridDim.x;
  uint32_t g = blockIdx.x;
  if (g >= groups) return;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&s.barrier)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s.gave_up = 0;
  }
  fetch_table<Shape>(s, 0, t, g, groups);
  fetch_table<Shape>(s, 1, t, g + stride, groups);
  copy_commit();
  copy_wait_all();
  __syncthreads();
  if (warp == 0) {
    touch_runs<Shape, true>(s, 0, t);
    if (g + stride < groups) touch_runs<Shape, false>(s, 1, t);
  }
  uint32_t parity = 0;

  for (int q = 0; g < groups; g += stride, q = q == 2 ? 0 : q + 1) {
    const int q1 = q == 2 ? 0 : q + 1, q2 = q1 == 2 ? 0 : q1 + 1;
    fetch_table<Shape>(s, q2, t, g + 2 * stride, groups);
    copy_commit();
    const uint32_t* row0 = group_table(s, q, t.row_words);
    const int count = static_cast<int>(row0[t.row_words + t.chunks]);
    const uint32_t begin = row0[t.chunks];
    const int b0 = static_cast<int>(row0[t.chunks + 1]), b1 = static_cast<int>(row0[t.chunks + 2]);
    const int64_t first_cell = static_cast<int64_t>(b0) << t.shift;
    const int cells_here = static_cast<int>(
        min(static_cast<long long>(b1 - b0) << t.shift, static_cast<long long>(num_cells - first_cell)));
    const int drop = drop_for<Shape>(cells_here);
    const int hist_words = max(8, cells_here * (32 >> drop));
    for (int i = tid; i < hist_words; i += kThreads) s.hist[i] = 0;
    if (count > 0) {
      if (!bulk_load_wait(&s.barrier, parity)) s.gave_up = 1;
      parity ^= 1;
    }
    __syncthreads();
    if (s.gave_up) {  // the copy never landed: report and stop without touching the output
      if (tid == 0) atomicCAS(&hdr->error, 0, kErrBulkCopyTimeout);
      copy_wait_all();
      return;
    }
    if (!sort_staged<Shape>(s, out, count, begin, first_cell, cells_here, drop)) {
      if (tid == 0) hdr->use_standard = 1;
    }
    // s.raw is free (sort_staged ended with a barrier): the next group's records, which L2
    // holds by now, can come in, and the group after it is asked into L2.
    copy_wait_all();
    __syncthreads();  // the table of group g + 2 * stride is visible
    if (warp == 0) {
      if (g + stride < groups) touch_runs<Shape, true>(s, q1, t);
      if (g + 2 * stride < groups) touch_runs<Shape, false>(s, q2, t);
    }
  }
}

// The buckets the kernel above skipped: those with more records than its shared
// memory holds.  Usually there are none and every block returns after a look at
// the largest bucket count.
template <class Shape>
__global__ void __launch_bounds__(Shape::kThreads, 1)
bucket_finish_large_kernel(RunTable t, int64_t num_cells, FinishOut out,
                           Header* __restrict__ hdr, uint32_t capacity) {
  chain_begin();
  if (hdr->use_standard || hdr->max_bucket <= capacity) return;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FinishSmem<Shape>& s = *reinterpret_cast<FinishSmem<Shape>*>(smem_raw);
  for (int b = blockIdx.x; b < t.buckets; b += gridDim.x) {
    const uint32_t begin = t.bucket_start[b], end = t.bucket_start[b + 1];
    const int count = static_cast<int>(end - begin);
    if (static_cast<uint32_t>(count) <= capacity) continue;
    const int64_t first_cell = static_cast<int64_t>(b) << t.shift;
    const int cells_here = static_cast<int>(
        min(static_cast<long long>(1) << t.shift, static_cast<long long>(num_cells - first_cell)));
    if (!finish_large_bucket<Shape>(s, out, t, b, begin, count, first_cell, cells_here)) {
      if (threadIdx.x == 0) hdr->use_standard = 1;
      return;
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The chunk-major record layout: while a chunk is scattered its stores stay inside the
// chunk's region, which L2 serves faster than the whole record array; but every bucket gets
// one run per chunk, and short runs cost the scatter (partial lines) and the finish kernel
// (many small copies) more than the window saves.  Measured optimum on random input: runs of
// about 256 records, i.e. 2^22 particles per chunk with 16 K buckets (64 M particles: 2.50 ms
// against 2.63 at 2^23), 2^23 with 32 K buckets (128 M: 5.15 against 5.66 at 2^22 and 5.50 at
// 2^24), 2^24 with 64 K buckets (256 M: 11.8 against 14.7 at 2^22, 12.8 at 2^23, 12.0 at
// 2^25).  Smaller inputs take smaller chunks (fewer particles contend for a slot counter):
// best 2^20 at 4 M particles, 2^21 at 16 M.
inline int chunk_log_for(int64_t buckets, int64_t n) {
  if (n <= (int64_t{1} << 22)) return kChunkLog - 2;
  if (n <= (int64_t{1} << 24)) return kChunkLog - 1;
  int bucket_log = 0;
  while ((int64_t{1} << bucket_log) < buckets) ++bucket_log;
  return std::min(kChunkLog + 2, std::max(kChunkLog, bucket_log + 8));
}

struct BucketLayout {
  int chunk_log;
  int chunks;
  int64_t entries;  // chunks * buckets runs
  int scan_blocks;
  size_t count_off, total_off, start_off, cursor_off, local_off, block_sum_off, run_begin_off,
      groups_off, tables_off, records_off, total;
};

// Tables and records for `n` particles (or room for that many) in `chunks` chunks.
BucketLayout bucket_layout_of(int64_t n, int64_t buckets, int chunk_log, int chunks) {
  BucketLayout l;
  l.chunk_log = chunk_log;
  l.chunks = chunks;
  l.entries = static_cast<int64_t>(l.chunks) * buckets;
  l.scan_blocks = static_cast<int>((l.entries + kFlatScanBlock - 1) / kFlatScanBlock);
  const size_t words = sizeof(uint32_t);
  l.count_off = sizeof(Header);  // zeroed per call together with the header
  l.total_off = align_up(l.count_off + l.entries * words, 256);
  l.start_off = align_up(l.total_off + buckets * words, 256);
  l.cursor_off = align_up(l.start_off + (buckets + 1) * words, 256);
  l.local_off = align_up(l.cursor_off + l.entries * words, 256);
  l.block_sum_off = align_up(l.local_off + l.entries * words, 256);
  l.run_begin_off = align_up(l.block_sum_off + l.scan_blocks * words, 256);
  l.groups_off = align_up(l.run_begin_off + (l.entries + 1) * words, 256);
  l.tables_off = align_up(l.groups_off + buckets * 2 * words, 256);
  l.records_off = align_up(l.tables_off + buckets * 2 * table_row_words(l.chunks) * words, 256);
  l.total = align_up(l.records_off + static_cast<size_t>(n) * kRecordWords * words, 256);
  return l;
}

BucketLayout bucket_layout(int64_t n, int64_t buckets) {
  const int chunk_log = chunk_log_for(buckets, n);
  const int chunks = static_cast<int>(
      std::max<int64_t>(1, (n + (int64_t{1} << chunk_log) - 1) >> chunk_log));
  return bucket_layout_of(n, buckets, chunk_log, chunks);
}

// Most buckets the small finish shape is planned for: beyond, the count kernel's table, the
// scans and the scatter pay more for the many small buckets than the finish kernel gains
// (measured at 64 M particles: 65,536 buckets of 1,024 against 16,384 of 4,096).
constexpr int64_t kMaxSmallShapeBuckets = 32 * 1024;
int64_t g_small_shape_buckets = kMaxSmallShapeBuckets;  // tuning knob, see set_small_shape_buckets

// Largest bucket width 2^s, s <= max_shift, whose average load stays at or below `target`,
// with at least 2048 buckets (fewer make the slot counters of the scatter contend: measured
// at 1 M and 4 M particles, 2048 beats 1024, 4096 and 8192).
int shift_for(int64_t n, int64_t num_cells, int64_t target, int max_shift) {
  for (int s = max_shift; s > 0; --s) {
    const int64_t buckets = (num_cells + (int64_t{1} << s) - 1) >> s;
    if (n <= target * buckets && buckets >= 2048) return s;
  }
  return 0;
}

int log2_floor(int v) {
  int l = 0;
  while ((2 << l) <= v) ++l;
  return l;
}

}  // namespace

namespace {
BucketPlan plan_buckets_shape(int64_t n, int64_t num_cells, bool allow_small) {
  BucketPlan p;
  // The small finish shape (two blocks per multiprocessor) wants buckets well below its
  // capacity, so that the groups cut from them fill a block whatever the density does
  // inside a row of cells.
  p.small_blocks = true;
  p.shift = shift_for(n, num_cells, 1100, log2_floor(FinishSmall::kMaxCells));
  p.buckets = (num_cells + (int64_t{1} << p.shift) - 1) >> p.shift;
  p.usable = allow_small && n > 0 && n <= 1100 * p.buckets && p.buckets <= g_small_shape_buckets;
  if (p.usable) return p;
  p.small_blocks = false;
  p.shift = shift_for(n, num_cells, 4160, log2_floor(FinishLarge::kMaxCells));
  p.buckets = (num_cells + (int64_t{1} << p.shift) - 1) >> p.shift;
  p.usable = n > 0 && n <= 4160 * p.buckets && p.buckets <= (int64_t{1} << 24);
  return p;
}
}  // namespace

BucketPlan plan_buckets(int64_t n, int64_t num_cells) {
  return plan_buckets_shape(n, num_cells, true);
}

void set_small_shape_buckets(int64_t buckets) {
  g_small_shape_buckets = std::max<int64_t>(0, std::min<int64_t>(buckets, kMaxSmallShapeBuckets));
}

uint32_t bucket_group_capacity(int64_t n, const BucketPlan& p) {
  // A block's capacity, or less on small inputs so that every multiprocessor gets several groups.
  const int capacity = p.small_blocks ? FinishSmall::kCapacity : FinishLarge::kCapacity;
  return static_cast<uint32_t>(std::min<int64_t>(
      capacity, std::max<int64_t>(1024, n / (4 * static_cast<int64_t>(sm_count())))));
}

size_t bucketed_workspace_bytes(int64_t n, int64_t num_cells) {
  const BucketPlan p = plan_buckets(n, num_cells);
  return bucket_layout(n, p.buckets).total;
}

namespace {

template <class Shape>
cudaError_t launch_finish(const RunTable& t, const SortArgs& a, const FinishOut& out, Header* hdr,
                          uint32_t group_capacity, const uint32_t* n_on_device = nullptr) {
  const size_t table_bytes = 3 * 2 * static_cast<size_t>(t.row_words) * sizeof(uint32_t);
  if (Shape::kThreads <= 512 && table_bytes > kSmallShapeTableBytes) return cudaErrorInvalidValue;
  const int smem = static_cast<int>(sizeof(FinishSmem<Shape>) + table_bytes);
  cudaError_t e = cudaFuncSetAttribute(bucket_finish_kernel<Shape>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  // Buckets in no group (more records than a group may hold) go to the large shape whatever
  // the shape of the groups: a single cell may then hold up to its 5120 records.
  const int smem_large = static_cast<int>(sizeof(FinishSmem<FinishLarge>));
  e = cudaFuncSetAttribute(bucket_finish_large_kernel<FinishLarge>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem_large);
  if (e != cudaSuccess) return e;
  const int per_sm = Shape::kThreads <= 512 ? 2 : 1;
  e = launch_chained<true>(bucket_finish_kernel<Shape>, std::min(t.buckets, sm_count() * per_sm),
                     Shape::kThreads, smem, a.stream, t, a.n, n_on_device, a.num_cells, out, hdr);
  if (e != cudaSuccess) return e;
  e = launch_chained<true>(bucket_finish_large_kernel<FinishLarge>, std::min(t.buckets, sm_count()),
                     FinishLarge::kThreads, smem_large, a.stream, t, a.num_cells, out, hdr,
                     group_capacity);
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

// Enqueues the bucketed path.  When a bucket turns out too large for the finish
// kernel the device sets Header::use_standard and the remaining kernels return
// at once; the caller then enqueues the digit-pass path predicated on that flag.
cudaError_t bucketed_sort(const SortArgs& a, const BucketPlan& p) {
  const BucketLayout l = bucket_layout(a.n, p.buckets);
  if (a.workspace_bytes < l.total || l.chunks > kMaxChunks) return cudaErrorInvalidValue;
  auto* base = static_cast<unsigned char*>(a.workspace);
  auto words_at = [&](size_t off) { return reinterpret_cast<uint32_t*>(base + off); };
  Header* hdr = reinterpret_cast<Header*>(base);
  uint32_t* count = words_at(l.count_off);
  uint32_t* total = words_at(l.total_off);
  uint32_t* start = words_at(l.start_off);
  uint32_t* cursor = words_at(l.cursor_off);
  uint32_t* local = words_at(l.local_off);
  uint32_t* block_sum = words_at(l.block_sum_off);
  uint32_t* run_begin = words_at(l.run_begin_off);
  uint2* groups = reinterpret_cast<uint2*>(base + l.groups_off);
  uint32_t* tables = words_at(l.tables_off);
  uint32_t* records = words_at(l.records_off);
  cudaError_t e = cudaMemsetAsync(base, 0, l.total_off, a.stream);  // header and run counts
  if (e != cudaSuccess) return e;
  const int buckets = static_cast<int>(p.buckets);
  const uint32_t k0 = static_cast<uint32_t>(a.seed), k1 = static_cast<uint32_t>(a.seed >> 32);
  const bool vec = aligned16(a.x) && aligned16(a.y) && aligned16(a.z) &&
                   (!a.velocity || (aligned16(a.velocity) && a.padded % 4 == 0));

  stage_begin(kStageBucketCount, a.stream);
  {
    const size_t bytes32 = static_cast<size_t>(buckets) * sizeof(uint32_t);
    const size_t bytes16 = (static_cast<size_t>(buckets) + 1) / 2 * sizeof(uint32_t);
    const int table = bytes32 <= 200 * 1024 ? kTableShared32
                      : bytes16 <= 200 * 1024 ? kTableShared16 : kTableGlobal;
    const size_t table_bytes = table == kTableShared32 ? bytes32 : table == kTableShared16 ? bytes16 : 0;
    const bool wide = table_bytes > 96 * 1024;  // one 1024-thread block per SM holds the table
    const int threads = wide ? kCountThreadsWide : kCountThreads;
    const int blocks_per_sm = table == kTableGlobal ? 4 : wide ? 1 : table_bytes <= 48 * 1024 ? 4 : 2;
    const int64_t chunk_size = int64_t{1} << l.chunk_log;
    const int64_t covered = std::min<int64_t>(a.n, chunk_size);
    // Slices of a chunk: enough units to fill the GPU twice over, each a multiple of one
    // block round (4 particles per thread) so that the 16-byte loads stay aligned.
    const int want = std::max(1, sm_count() * blocks_per_sm * 2 / l.chunks);
    const int64_t round = threads * 4;
    int64_t slice = std::max<int64_t>(round, ((covered + want - 1) / want + round - 1) / round * round);
    if (table == kTableShared16) slice = std::min<int64_t>(slice, kSlice16 / round * round);
    const int parts = static_cast<int>((covered + slice - 1) / slice);
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>(static_cast<int64_t>(l.chunks) * parts, sm_count() * blocks_per_sm)));
#define AETHER_COUNT_LAUNCH(TABLE, THREADS)                                                      \
  do {                                                                                            \
    auto kernel = vec ? bucket_count_kernel<TABLE, true, THREADS>                                 \
                      : bucket_count_kernel<TABLE, false, THREADS>;                               \
    if (table_bytes > 48 * 1024) {                                                                \
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,               \
                               static_cast<int>(table_bytes));                                    \
      if (e != cudaSuccess) return e;                                                             \
    }                                                                                             \
    kernel<<<grid, THREADS, table_bytes, a.stream>>>(a.x, a.y, a.z, a.velocity, a.padded, a.push, \
                                                     a.n, a.grid, p.shift, buckets, l.chunks,     \
                                                     l.chunk_log, parts, slice, count);           \
  } while (0)
    if (table == kTableGlobal) AETHER_COUNT_LAUNCH(kTableGlobal, kCountThreads);
    else if (table == kTableShared16) AETHER_COUNT_LAUNCH(kTableShared16, kCountThreadsWide);
    else if (wide) AETHER_COUNT_LAUNCH(kTableShared32, kCountThreadsWide);
    else AETHER_COUNT_LAUNCH(kTableShared32, kCountThreads);
#undef AETHER_COUNT_LAUNCH
  }
  stage_end(kStageBucketCount, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  stage_begin(kStageBucketScan, a.stream);
  const uint32_t largest = FinishLarge::kLargestBucket;
  const int max_cells = p.small_blocks ? FinishSmall::kMaxCells : FinishLarge::kMaxCells;
  const uint32_t group_capacity = bucket_group_capacity(a.n, p);
  const int group_shift = std::min(log2_floor(kMaxGroupBuckets),
                                   std::max(0, log2_floor(max_cells) - p.shift));
  const int blocks_of_buckets = (buckets + (1 << group_shift) - 1) >> group_shift;
  e = launch_chained(bucket_total_kernel, (buckets + 255) / 256, 256, 0, a.stream, count, buckets,
                     l.chunks, total);
  if (e == cudaSuccess)
    e = launch_chained(bucket_scan_kernel, 1, kScanThreads, 0, a.stream, total, buckets, a.n,
                       nullptr, largest, start, nullptr, hdr);
  if (e == cudaSuccess)
    e = launch_chained(group_cut_kernel, (blocks_of_buckets + 255) / 256, 256, 0, a.stream, start,
                       buckets, group_shift, group_capacity, groups, &hdr->aux_counter[1]);
  if (e == cudaSuccess)
    e = launch_chained(run_scan_local_kernel, l.scan_blocks, kFlatScanBlock, 0, a.stream, count,
                       l.entries, local, block_sum);
  if (e == cudaSuccess)
    e = launch_chained(run_scan_blocks_kernel, 1, kFlatScanBlock, 0, a.stream, block_sum,
                       l.scan_blocks);
  if (e == cudaSuccess)
    e = launch_chained(run_table_kernel, static_cast<int>((l.entries + 1 + 255) / 256), 256, 0,
                       a.stream, local, block_sum, l.entries, static_cast<uint32_t>(a.n), cursor,
                       run_begin);
  if (e == cudaSuccess)
    e = launch_chained(group_table_kernel,
                       std::max(1, std::min((buckets + 7) / 8, sm_count() * 8)), 256, 0, a.stream,
                       groups, &hdr->aux_counter[1], start, run_begin, l.chunks, buckets, tables);
  if (e != cudaSuccess) return e;
  count_launches(7);
  stage_end(kStageBucketScan, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  stage_begin(kStageBucketScatter, a.stream);
  {
    constexpr int kItems = 2;
    const int64_t groups = (a.n + kItems - 1) / kItems;
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>((groups + kScatterThreads - 1) / kScatterThreads,
                             sm_count() * (8 / kItems) * 4)));
    auto kernel = vec ? bucket_scatter_kernel<true, kItems> : bucket_scatter_kernel<false, kItems>;
    e = launch_chained<true>(kernel, grid, kScatterThreads, 0, a.stream, a.x, a.y, a.z, a.velocity,
                       a.padded, a.push, a.n, a.grid, k0, k1, p.shift, buckets, l.chunk_log, cursor,
                       records, hdr);
    if (e != cudaSuccess) return e;
  }
  stage_end(kStageBucketScatter, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  count_launches(2);

  stage_begin(kStageBucketFinish, a.stream);
  const FinishOut out{a.keys_out, a.index_out, a.cell_counts, a.cell_start, a.xs, a.ys, a.zs,
                      a.vs, a.padded_sorted};
  const RunTable t{records, start, run_begin, tables, &hdr->aux_counter[1],
                   table_row_words(l.chunks), l.chunks, buckets, p.shift};
  e = p.small_blocks ? launch_finish<FinishSmall>(t, a, out, hdr, group_capacity)
                     : launch_finish<FinishLarge>(t, a, out, hdr, group_capacity);
  stage_end(kStageBucketFinish, a.stream);
  count_launches(2);
  return e;
}

// ---- the segmented form: one chunk per slice of the sliced exchange ----

namespace {
// The small shape's shared memory has room for the tables of a dozen chunks only.
BucketPlan sliced_plan(int64_t plan_n, int64_t num_cells, int slices) {
  const bool tables_fit =
      3 * 2 * static_cast<size_t>(table_row_words(slices)) * sizeof(uint32_t) <= kSmallShapeTableBytes;
  return plan_buckets_shape(plan_n, num_cells, tables_fit);
}
}  // namespace

size_t sliced_sort_workspace_bytes(int64_t capacity, int64_t plan_n, int64_t num_cells, int slices) {
  const BucketPlan p = sliced_plan(plan_n, num_cells, slices);
  return bucket_layout_of(capacity, p.buckets, 0, slices).total;
}

namespace {
struct SlicedState {
  BucketPlan plan;
  BucketLayout layout;
  unsigned char* base;
  bool ok;
};
SlicedState sliced_state(const SortArgs& a, int64_t plan_n, int slices) {
  SlicedState st{};
  st.plan = sliced_plan(plan_n, a.num_cells, slices);
  st.layout = bucket_layout_of(a.n, st.plan.buckets, 0, slices);
  st.base = static_cast<unsigned char*>(a.workspace);
  st.ok = st.plan.usable && slices >= 1 && slices <= kMaxSlices && a.workspace &&
          a.workspace_bytes >= st.layout.total &&
          (reinterpret_cast<uintptr_t>(a.workspace) & 255) == 0;
  return st;
}
}  // namespace

cudaError_t sliced_sort_begin(const SortArgs& a, int64_t plan_n, int slices) {
  const SlicedState st = sliced_state(a, plan_n, slices);
  if (!st.ok) return cudaErrorInvalidValue;
  stage_reset();
  return cudaMemsetAsync(st.base, 0, st.layout.total_off, a.stream);  // header and run counts
}

cudaError_t sliced_sort_slice(const SortArgs& a, int64_t plan_n, const SliceSegments* segments,
                              int slices, int slice) {
  const SlicedState st = sliced_state(a, plan_n, slices);
  if (!st.ok || !segments || slice < 0 || slice >= slices) return cudaErrorInvalidValue;
  if (!a.x || !a.y || !a.z || !a.velocity || a.padded < a.n) return cudaErrorInvalidValue;
  const BucketLayout& l = st.layout;
  auto words_at = [&](size_t off) { return reinterpret_cast<uint32_t*>(st.base + off); };
  const int buckets = static_cast<int>(st.plan.buckets);
  uint32_t* row = words_at(l.count_off) + static_cast<size_t>(slice) * buckets;
  uint32_t* cursor_row = words_at(l.cursor_off) + static_cast<size_t>(slice) * buckets;
  uint32_t* run_begin_row = words_at(l.run_begin_off) + static_cast<size_t>(slice) * buckets;
  uint32_t* records = words_at(l.records_off);
  const bool vec = aligned16(a.x) && aligned16(a.y) && aligned16(a.z) && aligned16(a.velocity) &&
                   a.padded % 4 == 0;
  // Work units of a slice: its share of the planned particles, and one partial unit per source.
  const int64_t units = plan_n / slices / kSegmentUnit + kMaxWorld + 1;
  cudaError_t e = cudaSuccess;

  stage_begin(kStageBucketCount, a.stream);
  {
    const size_t table_bytes = static_cast<size_t>(buckets) * sizeof(uint32_t);
    const bool shared = table_bytes <= 200 * 1024;
    const bool wide = shared && table_bytes > 96 * 1024;
    const int per_sm = !shared ? 4 : wide ? 1 : table_bytes <= 48 * 1024 ? 4 : 2;
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(units, sm_count() * per_sm)));
    if (!shared) {
      bucket_count_segments_kernel<kTableGlobal, kCountThreads><<<grid, kCountThreads, 0, a.stream>>>(
          a.x, a.y, a.z, a.n, vec, segments, slice, a.grid, st.plan.shift, buckets, row);
    } else if (wide) {
      auto kernel = bucket_count_segments_kernel<kTableShared32, kCountThreadsWide>;
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(table_bytes));
      if (e != cudaSuccess) return e;
      kernel<<<grid, kCountThreadsWide, table_bytes, a.stream>>>(
          a.x, a.y, a.z, a.n, vec, segments, slice, a.grid, st.plan.shift, buckets, row);
    } else {
      auto kernel = bucket_count_segments_kernel<kTableShared32, kCountThreads>;
      if (table_bytes > 48 * 1024) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(table_bytes));
        if (e != cudaSuccess) return e;
      }
      kernel<<<grid, kCountThreads, table_bytes, a.stream>>>(
          a.x, a.y, a.z, a.n, vec, segments, slice, a.grid, st.plan.shift, buckets, row);
    }
  }
  stage_end(kStageBucketCount, a.stream);
  stage_begin(kStageBucketScan, a.stream);
  if (buckets <= kStagedScanMax) {
    const int per = (buckets + kFlatScanBlock - 1) / kFlatScanBlock;
    const size_t bytes = (static_cast<size_t>(buckets) + 2 * (buckets / per + 1)) * sizeof(uint32_t);
    if (bytes > 48 * 1024) {
      e = cudaFuncSetAttribute(chunk_scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(bytes));
      if (e != cudaSuccess) return e;
    }
    chunk_scan_kernel<true><<<1, kFlatScanBlock, bytes, a.stream>>>(row, buckets, segments, slice,
                                                                    cursor_row, run_begin_row);
  } else {
    chunk_scan_kernel<false><<<1, kFlatScanBlock, 0, a.stream>>>(row, buckets, segments, slice,
                                                                 cursor_row, run_begin_row);
  }
  stage_end(kStageBucketScan, a.stream);
  stage_begin(kStageBucketScatter, a.stream);
  {
    constexpr int kItems = 2;
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>(units, sm_count() * (8 / kItems))));
    const uint32_t k0 = static_cast<uint32_t>(a.seed), k1 = static_cast<uint32_t>(a.seed >> 32);
    bucket_scatter_segments_kernel<kItems><<<grid, kScatterThreads, 0, a.stream>>>(
        a.x, a.y, a.z, a.velocity, a.padded, a.n, vec, segments, slice, a.grid, k0, k1,
        st.plan.shift, buckets, cursor_row, records);
  }
  stage_end(kStageBucketScatter, a.stream);
  count_launches(3);
  return cudaGetLastError();
}

cudaError_t sliced_sort_finish(const SortArgs& a, int64_t plan_n, const SliceSegments* segments,
                               int slices) {
  const SlicedState st = sliced_state(a, plan_n, slices);
  if (!st.ok || !segments) return cudaErrorInvalidValue;
  if (!a.keys_out || !a.index_out || !a.cell_counts || !a.cell_start) return cudaErrorInvalidValue;
  const BucketLayout& l = st.layout;
  const BucketPlan& p = st.plan;
  auto words_at = [&](size_t off) { return reinterpret_cast<uint32_t*>(st.base + off); };
  Header* hdr = reinterpret_cast<Header*>(st.base);
  const int buckets = static_cast<int>(p.buckets);
  uint32_t* count = words_at(l.count_off);
  uint32_t* total = words_at(l.total_off);
  uint32_t* start = words_at(l.start_off);
  uint32_t* run_begin = words_at(l.run_begin_off);
  uint2* groups = reinterpret_cast<uint2*>(st.base + l.groups_off);
  uint32_t* tables = words_at(l.tables_off);
  uint32_t* records = words_at(l.records_off);
  const uint32_t* n_on_device = &segments->n;

  stage_begin(kStageBucketFinish, a.stream);
  const int max_cells = p.small_blocks ? FinishSmall::kMaxCells : FinishLarge::kMaxCells;
  const uint32_t group_capacity = bucket_group_capacity(plan_n, p);
  const int group_shift = std::min(log2_floor(kMaxGroupBuckets),
                                   std::max(0, log2_floor(max_cells) - p.shift));
  const int blocks_of_buckets = (buckets + (1 << group_shift) - 1) >> group_shift;
  bucket_total_kernel<<<(buckets + 255) / 256, 256, 0, a.stream>>>(count, buckets, l.chunks, total);
  bucket_scan_kernel<<<1, kScanThreads, 0, a.stream>>>(total, buckets, a.n, n_on_device,
                                                       FinishLarge::kLargestBucket, start, nullptr,
                                                       hdr);
  group_cut_kernel<<<(blocks_of_buckets + 255) / 256, 256, 0, a.stream>>>(
      start, buckets, group_shift, group_capacity, groups, &hdr->aux_counter[1]);
  group_table_kernel<<<std::max(1, std::min((buckets + 7) / 8, sm_count() * 8)), 256, 0, a.stream>>>(
      groups, &hdr->aux_counter[1], start, run_begin, l.chunks, buckets, tables);
  count_launches(6);
  const FinishOut out{a.keys_out, a.index_out, a.cell_counts, a.cell_start, a.xs, a.ys, a.zs,
                      a.vs, a.padded_sorted};
  const RunTable t{records, start, run_begin, tables, &hdr->aux_counter[1],
                   table_row_words(l.chunks), l.chunks, buckets, p.shift};
  const cudaError_t e = p.small_blocks
                            ? launch_finish<FinishSmall>(t, a, out, hdr, group_capacity, n_on_device)
                            : launch_finish<FinishLarge>(t, a, out, hdr, group_capacity, n_on_device);
  stage_end(kStageBucketFinish, a.stream);
  return e;
}

}  // namespace aether
