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
//   bucket_finish_kernel   one thread block per bucket: a counting sort on the
//                          low key bits in shared memory, ties put in index
//                          order, then coalesced SoA output of keys, indices,
//                          positions, velocities and the bucket's rows of
//                          cell_counts / cell_start (replaces the digit passes,
//                          the last-pass count atomics, torch.cumsum and the
//                          payload gather: fused_radix_sort.py:116-203,277-279,
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
// The finish kernel collects a bucket from its runs, one bulk copy per chunk.
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

constexpr int kChunkLog = 22;      // particles per chunk of the record layout (2^22; 2^21, 2^23
                                   // and 2^24 measured slower end to end) ...
constexpr int kNoChunkLog = 31;    // ... or one chunk for everything

// Work unit = one slice of one chunk; a block counts the slice into a table
// (shared memory, or the global counts directly when the table does not fit)
// and adds the table to the chunk's row of counts, count[chunk * buckets + b].
template <bool SHARED, bool VEC, int THREADS>
__global__ void __launch_bounds__(THREADS)
bucket_count_kernel(const float* __restrict__ x, const float* __restrict__ y,
                    const float* __restrict__ z, const float* __restrict__ v, int64_t padded,
                    PushSpec push, int64_t n, AetherGrid g, int shift,
                    int buckets, int chunks, int chunk_log, int parts, int64_t slice,
                    uint32_t* __restrict__ bucket_count) {
  extern __shared__ uint32_t hist[];
  for (int unit = blockIdx.x; unit < chunks * parts; unit += gridDim.x) {
    const int chunk = unit / parts, part = unit % parts;
    uint32_t* row = bucket_count + static_cast<size_t>(chunk) * buckets;
    if (SHARED) {
      for (int i = threadIdx.x; i < buckets; i += THREADS) hist[i] = 0;
      __syncthreads();
    }
    uint32_t* target = SHARED ? hist : row;
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
#pragma unroll
      for (int k = 0; k < 4; ++k)
        bin_add(target, cell_of(px[k], py[k], pz[k], g) >> shift, i0 + k < last);
    }
    if (SHARED) {
      __syncthreads();
      for (int i = threadIdx.x; i < buckets; i += THREADS)
        if (hist[i]) atomicAdd(&row[i], hist[i]);
      __syncthreads();
    }
  }
}

// Per bucket: particles in all chunks.
__global__ void __launch_bounds__(256)
bucket_total_kernel(const uint32_t* __restrict__ bucket_count, int buckets, int chunks,
                    uint32_t* __restrict__ total) {
  const int b = blockIdx.x * 256 + threadIdx.x;
  if (b >= buckets) return;
  uint32_t sum = 0;
  for (int c = 0; c < chunks; ++c) sum += bucket_count[static_cast<size_t>(c) * buckets + b];
  total[b] = sum;
}

// Exclusive scan of the [chunk][bucket] counts in memory order: where every run
// starts in the record array.  Two levels (1024 entries per block, then the
// block totals), then one pass that writes the run starts as scatter cursors and,
// transposed to [bucket][chunk], as the run table the finish kernel reads.
constexpr int kFlatScanBlock = 1024;

__global__ void __launch_bounds__(kFlatScanBlock)
run_scan_local_kernel(const uint32_t* __restrict__ count, int64_t entries,
                      uint32_t* __restrict__ local, uint32_t* __restrict__ block_sum) {
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
run_table_kernel(const uint32_t* __restrict__ count, const uint32_t* __restrict__ local,
                 const uint32_t* __restrict__ block_sum, int buckets, int chunks,
                 uint32_t* __restrict__ cursor, uint32_t* __restrict__ run_start,
                 uint32_t* __restrict__ run_length) {
  const int64_t entries = static_cast<int64_t>(buckets) * chunks;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= entries) return;
  const uint32_t start = local[i] + block_sum[i / kFlatScanBlock];
  cursor[i] = start;
  const int64_t chunk = i / buckets, b = i % buckets;
  run_start[b * chunks + chunk] = start;
  run_length[b * chunks + chunk] = count[i];
}

// ------------------------------------------------------------------------
// Bucket starts.
// ------------------------------------------------------------------------
constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads)
bucket_scan_kernel(const uint32_t* __restrict__ bucket_count, int buckets, int64_t n,
                   uint32_t capacity, uint32_t* __restrict__ bucket_start,
                   uint32_t* __restrict__ cursor, Header* __restrict__ hdr) {
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
    bucket_start[buckets] = static_cast<uint32_t>(n);
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
// Finish: one block sorts one bucket in shared memory and writes the output.
// ------------------------------------------------------------------------
constexpr int kFinishThreads = 1024;
constexpr int kFinishCapacity = 5376;                      // records per bucket
constexpr int kFinishItems = (kFinishCapacity + kFinishThreads - 1) / kFinishThreads;  // 6
constexpr int kMaxLowBits = 15;                            // bits the counters resolve
constexpr int kMaxShift = 10;                              // bucket = up to 1024 cells
constexpr int kHistWords = (1 << kMaxLowBits) / 4;         // byte counters, 4 per word
constexpr int kWordsPerThread = kHistWords / kFinishThreads;  // 8
constexpr uint32_t kBulkChunkBytes = 32768;                // bytes per bulk copy
constexpr uint32_t kBulkWaitLimit = 1u << 24;              // polls of the copy barrier
constexpr int kMaxSegments = 32;                           // runs of cells an oversized bucket is cut into
constexpr uint32_t kLargestBucket = kMaxSegments * kFinishCapacity;  // beyond this no cut can fit

struct __align__(128) FinishSmem {
  uint32_t raw[kFinishCapacity * kRecordWords];  // the bucket's records as they lie in HBM
  uint32_t hist[kHistWords];     // byte counter per low-key value
  uint16_t word_prefix[kHistWords];  // exclusive prefix of each counter word
  uint16_t order[kFinishCapacity];  // record held by each sorted slot
  uint32_t warp_sum[32];
  uint32_t total;
  uint32_t gave_up;
  unsigned long long barrier;    // mbarrier of the bulk copy
  uint32_t seg_begin[kMaxSegments + 1];  // oversized bucket: records before each run of cells
  uint16_t seg_first[kMaxSegments + 1];  // ... and the first cell of each run
  uint32_t fill;                         // ... and the records picked so far for the run at hand
};
static_assert(sizeof(FinishSmem) <= 227 * 1024, "finish kernel shared memory");

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

// Waits (bounded) for the phase `parity` of the copy barrier; false if it gave up.
__device__ __forceinline__ bool bulk_load_wait(unsigned long long* barrier, uint32_t parity) {
  const uint32_t bar = smem_addr(barrier);
  for (uint32_t polls = 0; polls < kBulkWaitLimit; ++polls) {
    uint32_t ready;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ready) : "r"(bar), "r"(parity) : "memory");
    if (ready) return true;
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

// Sorts the `count` records staged in s.raw (any order) and writes them to the
// output from slot `begin` on.  The records belong to the cells first_cell ..
// first_cell + cells_here - 1; `low_base` is the low key (bits below the bucket
// id) of the first of these cells.  s.hist must be zero over the counters used.
// Returns false if a byte counter wrapped (more than 255 records on one counter).
// DROP: the number of low key bits the counters leave out, fixed at compile time
// (0, 1, 2) or -1 to take it from `drop_at_run_time`.
template <int DROP>
__device__ __forceinline__ bool sort_staged(FinishSmem& s, const FinishOut& out, int count,
                                            uint32_t begin, int64_t first_cell, int cells_here,
                                            uint32_t low_base, uint32_t low_mask,
                                            int drop_at_run_time) {
  const int drop = DROP >= 0 ? DROP : drop_at_run_time;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t drop_mask = (1u << drop) - 1;
  const int cell_words = 32 >> drop;  // counter words per cell
  const int hist_words = max(8, cells_here * cell_words);

  // Count the low key bits with byte-wide counters; the value an add returns
  // is the record's rank among the records of its counter.
  uint32_t packed[kFinishItems];  // counter id | rank << 16
#pragma unroll
  for (int k = 0; k < kFinishItems; ++k) {
    const int r = tid + k * kFinishThreads;
    packed[k] = 0;
    if (r < count) {
      const uint32_t low = ((s.raw[r * kRecordWords] & low_mask) - low_base) >> drop;
      const int sh = 8 * (low & 3);
      const uint32_t old = atomicAdd(&s.hist[low >> 2], 1u << sh);
      packed[k] = low | (((old >> sh) & 0xffu) << 16);
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
    const uint32_t w = s.warp_sum[lane];
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
  for (int c = tid; c < cells_here; c += kFinishThreads) {
    const uint32_t lo = s.word_prefix[c * cell_words];
    const uint32_t hi = (c + 1) * cell_words < hist_words ? s.word_prefix[(c + 1) * cell_words]
                                                           : static_cast<uint32_t>(count);
    out.cell_start[first_cell + c] = static_cast<int32_t>(begin + lo);
    out.cell_counts[first_cell + c] = static_cast<int32_t>(hi - lo);
  }

  // Sorted slot of every record: start of its counter's run + arrival rank.  A
  // counter held by one record only (the usual case) is final at once.
  uint32_t run[kFinishItems];  // run start | run length << 16, for records that share a counter
#pragma unroll
  for (int k = 0; k < kFinishItems; ++k) {
    const int r = tid + k * kFinishThreads;
    run[k] = 0;
    if (r < count) {
      const uint32_t low = packed[k] & 0xffffu, rank = packed[k] >> 16;
      const uint32_t word = s.hist[low >> 2];
      const int sh = 8 * (low & 3);
      const uint32_t start = s.word_prefix[low >> 2] + byte_sum(word & ((1u << sh) - 1u));
      const uint32_t length = (word >> sh) & 0xffu;
      s.order[start + rank] = static_cast<uint16_t>(r);
      if (length > 1) run[k] = start | (length << 16);
    }
  }
  __syncthreads();

  // Records that share a counter must appear in ascending (dropped key bits,
  // original index): a record inside such a run moves to (run start + number of
  // smaller records in the run).  Indices stay below 2^30, so the dropped bits
  // ride above them in one word.
  uint32_t moved[kFinishItems];
#pragma unroll
  for (int k = 0; k < kFinishItems; ++k) {
    moved[k] = 0xffffffffu;
    if (run[k]) {
      const int r = tid + k * kFinishThreads;
      const uint32_t start = run[k] & 0xffffu, length = run[k] >> 16;
      const uint32_t mine = ((s.raw[r * kRecordWords] & drop_mask) << 30) | s.raw[r * kRecordWords + 1];
      uint32_t smaller = 0;
      for (uint32_t j = 0; j < length; ++j) {
        const uint32_t* other = &s.raw[s.order[start + j] * kRecordWords];
        smaller += (((other[0] & drop_mask) << 30) | other[1]) < mine;
      }
      moved[k] = start + smaller;
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kFinishItems; ++k)
    if (moved[k] != 0xffffffffu) s.order[moved[k]] = static_cast<uint16_t>(tid + k * kFinishThreads);
  __syncthreads();

  // Coalesced output: each lane pulls one whole record out of shared memory
  // and writes its eight words to the eight output arrays.  (128-bit stores of
  // four consecutive slots per thread were measured: slower, 1.45 ms against
  // 1.32 ms at 64 M particles.)
  for (int d = tid; d < count; d += kFinishThreads) {
    const int rec = s.order[d];
    const uint4 a = *reinterpret_cast<const uint4*>(&s.raw[rec * kRecordWords]);
    const uint4 c = *reinterpret_cast<const uint4*>(&s.raw[rec * kRecordWords + 4]);
    const size_t o = static_cast<size_t>(begin) + d;
    __stcs(out.keys + o, a.x);
    __stcs(out.index + o, static_cast<int32_t>(a.y));
    if (out.xs) {  // keys-only calls leave the payload out
      __stcs(out.xs + o, __uint_as_float(a.z));
      __stcs(out.ys + o, __uint_as_float(a.w));
      __stcs(out.zs + o, __uint_as_float(c.x));
    }
    if (out.vs) {
      __stcs(out.vs + o, __uint_as_float(c.y));
      __stcs(out.vs + out.padded_sorted + o, __uint_as_float(c.z));
      __stcs(out.vs + 2 * out.padded_sorted + o, __uint_as_float(c.w));
    }
  }
  __syncthreads();
  return true;
}

// A bucket with more records than shared memory holds (a dense region: the
// bucket width is planned from the average load).  The block counts the
// bucket's records per cell, cuts the cells into up to kMaxSegments runs that
// fit, and for every run picks the run's records out of the bucket (which it
// reads from global memory once per run) and sorts them like a small bucket.
// Returns false if it cannot (a single cell larger than shared memory, too many
// runs, or a wrapped byte counter): the call then goes to the digit passes.
__device__ bool finish_large_bucket(FinishSmem& s, const FinishOut& out,
                                    const uint32_t* __restrict__ records,
                                    const uint32_t* __restrict__ run_start,
                                    const uint32_t* __restrict__ run_length, int chunks, int b,
                                    uint32_t begin, int count, int64_t first_cell, int cells_here,
                                    uint32_t low_mask, int drop) {
  const int tid = threadIdx.x;
  uint32_t* cell_count = s.hist;  // up to 1024 cells; s.hist is free until a run is sorted
  for (int c = tid; c < cells_here; c += kFinishThreads) cell_count[c] = 0;
  __syncthreads();
  // Per-cell counts: one pass over the keys of the bucket's records.
  for (int c = 0; c < chunks; ++c) {
    const uint32_t start = chunks == 1 ? begin : run_start[static_cast<size_t>(b) * chunks + c];
    const uint32_t length = chunks == 1 ? static_cast<uint32_t>(count)
                                        : run_length[static_cast<size_t>(b) * chunks + c];
    for (uint32_t i = tid; i < length; i += kFinishThreads) {
      const uint32_t key = __ldg(records + static_cast<size_t>(start + i) * kRecordWords);
      atomicAdd(&cell_count[(key & low_mask) >> kShuffleBits], 1u);
    }
  }
  __syncthreads();
  // Cut into runs of cells that fit (one thread; at most 1024 cells).
  if (tid == 0) {
    int segments = 0;
    uint32_t load = 0, before = 0;
    bool ok = true;
    s.seg_first[0] = 0;
    s.seg_begin[0] = 0;
    for (int c = 0; c < cells_here && ok; ++c) {
      const uint32_t here = cell_count[c];
      if (here > static_cast<uint32_t>(kFinishCapacity)) ok = false;
      if (load + here > static_cast<uint32_t>(kFinishCapacity)) {  // close the run before cell c
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
  const int cell_words = 32 >> drop;
  for (int k = 0; k < segments; ++k) {
    const int c0 = s.seg_first[k], c1 = s.seg_first[k + 1];
    const uint32_t seg_begin = s.seg_begin[k];
    const int seg_count = static_cast<int>(s.seg_begin[k + 1] - seg_begin);
    // Zero the counters of this run and the fill cursor (cell_count is overwritten
    // from here on; the cuts above are already in seg_first / seg_begin).
    const int words = max(8, (c1 - c0) * cell_words);
    for (int i = tid; i < words; i += kFinishThreads) s.hist[i] = 0;
    if (tid == 0) s.fill = 0;
    __syncthreads();
    for (int c = 0; c < chunks; ++c) {
      const uint32_t start = chunks == 1 ? begin : run_start[static_cast<size_t>(b) * chunks + c];
      const uint32_t length = chunks == 1 ? static_cast<uint32_t>(count)
                                          : run_length[static_cast<size_t>(b) * chunks + c];
      for (uint32_t i = tid; i < length; i += kFinishThreads) {
        const uint4* rec = reinterpret_cast<const uint4*>(records +
                                                          static_cast<size_t>(start + i) * kRecordWords);
        const uint4 lo = __ldg(rec);
        const int cell = static_cast<int>((lo.x & low_mask) >> kShuffleBits);
        if (cell >= c0 && cell < c1) {
          const uint32_t slot = atomicAdd(&s.fill, 1u);
          if (slot < static_cast<uint32_t>(kFinishCapacity)) {
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
    if (!sort_staged<-1>(s, out, seg_count, begin + seg_begin, first_cell + c0, c1 - c0,
                         static_cast<uint32_t>(c0) << kShuffleBits, low_mask, drop))
      return false;
  }
  return true;
}

template <int DROP>
__global__ void __launch_bounds__(kFinishThreads, 1)
bucket_finish_kernel(const uint32_t* __restrict__ records, const uint32_t* __restrict__ bucket_start,
                     const uint32_t* __restrict__ run_start, const uint32_t* __restrict__ run_length,
                     int chunks, int buckets, int shift, int64_t n, int64_t num_cells,
                     FinishOut out, Header* __restrict__ hdr) {
  if (hdr->use_standard) return;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FinishSmem& s = *reinterpret_cast<FinishSmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // The key bits below the bucket id: shift cell bits and the 7 shuffle bits.  The
  // counters resolve the upper 15 of them; up to two lowest bits (buckets of 512 or
  // 1024 cells) are left to the tie step, which orders by (those bits, index).
  const int low_bits = shift + kShuffleBits;
  const uint32_t low_mask = (1u << low_bits) - 1;
  constexpr int drop = DROP;  // max(0, low_bits - kMaxLowBits), chosen by the launcher
  const int hist_words = max(8, (1 << (low_bits - drop)) / 4);

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&s.barrier)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s.gave_up = 0;
  }
  __syncthreads();
  uint32_t parity = 0;

  // Bucket bounds and (warp 0, one chunk per lane) the bucket's run table are
  // fetched one bucket ahead, so that their latency is not on the path of the copy.
  const bool lane_runs = chunks > 1 && chunks <= 32;
  uint32_t next_begin = 0, next_end = 0, next_length = 0, next_start = 0;
  if (static_cast<int>(blockIdx.x) < buckets) {
    next_begin = bucket_start[blockIdx.x];
    next_end = bucket_start[blockIdx.x + 1];
    if (warp == 0 && lane_runs && lane < chunks) {
      next_length = run_length[static_cast<size_t>(blockIdx.x) * chunks + lane];
      next_start = run_start[static_cast<size_t>(blockIdx.x) * chunks + lane];
    }
  }

  for (int b = blockIdx.x; b < buckets; b += gridDim.x) {
    const uint32_t begin = next_begin, end = next_end;
    const uint32_t my_length = next_length, my_start = next_start;
    const int count = static_cast<int>(end - begin);
    {
      const int nb = b + gridDim.x;
      if (nb < buckets) {
        next_begin = bucket_start[nb];
        next_end = bucket_start[nb + 1];
        if (warp == 0 && lane_runs && lane < chunks) {
          next_length = run_length[static_cast<size_t>(nb) * chunks + lane];
          next_start = run_start[static_cast<size_t>(nb) * chunks + lane];
        }
      }
    }
    const int64_t first_cell = static_cast<int64_t>(b) << shift;
    const int cells_here = static_cast<int>(
        min(static_cast<long long>(1) << shift, static_cast<long long>(num_cells - first_cell)));
    if (b == buckets - 1 && tid == 0) out.cell_start[num_cells] = static_cast<int32_t>(n);
    if (count > kFinishCapacity) continue;  // bucket_finish_large_kernel's job
    // The bucket lies in HBM as one contiguous run of 32-byte records per chunk
    // (a single run when there is one chunk): fetch the runs back to back into
    // shared memory with bulk copies while the counters are cleared.  Warp 0
    // does it: lane l looks up the runs of chunks l, l+32, ... and issues their
    // copies after lane 0 has told the barrier how many bytes to expect.
    if (warp == 0 && count > 0) {
      if (lane == 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                         smem_addr(&s.barrier)),
                     "r"(static_cast<uint32_t>(count) * kRecordWords * 4u)
                     : "memory");
      }
      __syncwarp();
      uint32_t offset = 0;  // records of this bucket in earlier chunks
      for (int c0 = 0; c0 < chunks; c0 += 32) {
        const int c = c0 + lane;
        uint32_t length = 0, start = begin;
        if (chunks == 1) {
          length = lane == 0 ? static_cast<uint32_t>(count) : 0u;
        } else if (lane_runs) {
          length = my_length;  // zero for lanes past the last chunk
          start = my_start;
        } else if (c < chunks) {
          length = run_length[static_cast<size_t>(b) * chunks + c];
          start = run_start[static_cast<size_t>(b) * chunks + c];
        }
        uint32_t incl = length;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const uint32_t dst_record = offset + incl - length;
        if (length > 0 && dst_record + length <= static_cast<uint32_t>(count))
          bulk_copy(s.raw + static_cast<size_t>(dst_record) * kRecordWords,
                    records + static_cast<size_t>(start) * kRecordWords,
                    length * kRecordWords * 4u, &s.barrier);
        offset += __shfl_sync(0xffffffffu, incl, 31);
      }
    }
    for (int i = tid; i < hist_words; i += kFinishThreads) s.hist[i] = 0;
    if (count > 0) {
      if (!bulk_load_wait(&s.barrier, parity)) s.gave_up = 1;
      parity ^= 1;
    }
    __syncthreads();
    if (s.gave_up) {  // the copy never landed: report and stop without touching the output
      if (tid == 0) atomicCAS(&hdr->error, 0, kErrBulkCopyTimeout);
      return;
    }
    if (!sort_staged<DROP>(s, out, count, begin, first_cell, cells_here, 0u, low_mask, drop)) {
      if (tid == 0) hdr->use_standard = 1;
    }
  }
}

// The buckets the kernel above skipped: those with more records than its shared
// memory holds.  Usually there are none and every block returns after a look at
// its share of the bucket table.
__global__ void __launch_bounds__(kFinishThreads, 1)
bucket_finish_large_kernel(const uint32_t* __restrict__ records,
                           const uint32_t* __restrict__ bucket_start,
                           const uint32_t* __restrict__ run_start,
                           const uint32_t* __restrict__ run_length, int chunks, int buckets,
                           int shift, int64_t num_cells, FinishOut out, Header* __restrict__ hdr) {
  if (hdr->use_standard || hdr->max_bucket <= static_cast<uint32_t>(kFinishCapacity)) return;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  FinishSmem& s = *reinterpret_cast<FinishSmem*>(smem_raw);
  const int low_bits = shift + kShuffleBits;
  const uint32_t low_mask = (1u << low_bits) - 1;
  const int drop = max(0, low_bits - kMaxLowBits);
  for (int b = blockIdx.x; b < buckets; b += gridDim.x) {
    const uint32_t begin = bucket_start[b], end = bucket_start[b + 1];
    const int count = static_cast<int>(end - begin);
    if (count <= kFinishCapacity) continue;
    const int64_t first_cell = static_cast<int64_t>(b) << shift;
    const int cells_here = static_cast<int>(
        min(static_cast<long long>(1) << shift, static_cast<long long>(num_cells - first_cell)));
    if (!finish_large_bucket(s, out, records, run_start, run_length, chunks, b, begin, count,
                             first_cell, cells_here, low_mask, drop)) {
      if (threadIdx.x == 0) hdr->use_standard = 1;
      return;
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The chunk-major record layout pays when the scatter is bound by scattered
// stores and a bucket's runs stay long: up to 32 K buckets.  With more buckets
// (few particles per bucket and chunk) one chunk holds everything.
// Smaller inputs take smaller chunks (fewer particles contend for a slot counter, and the
// chunk's records stay deeper inside L2): measured best 2^20 at 4 M particles, 2^21 at 16 M,
// 2^22 from 32 M on.
inline int chunk_log_for(int64_t buckets, int64_t n) {
  if (buckets > 32768) return kNoChunkLog;
  if (n <= (int64_t{1} << 22)) return kChunkLog - 2;
  if (n <= (int64_t{1} << 24)) return kChunkLog - 1;
  return kChunkLog;
}

struct BucketLayout {
  int chunk_log;
  int chunks;
  int64_t entries;  // chunks * buckets runs
  int scan_blocks;
  size_t count_off, total_off, start_off, cursor_off, local_off, block_sum_off, run_start_off,
      run_length_off, records_off, total;
};

BucketLayout bucket_layout(int64_t n, int64_t buckets) {
  BucketLayout l;
  l.chunk_log = chunk_log_for(buckets, n);
  l.chunks = static_cast<int>(
      std::max<int64_t>(1, (n + (int64_t{1} << l.chunk_log) - 1) >> l.chunk_log));
  l.entries = static_cast<int64_t>(l.chunks) * buckets;
  l.scan_blocks = static_cast<int>((l.entries + kFlatScanBlock - 1) / kFlatScanBlock);
  const bool chunked = l.chunks > 1;
  const size_t words = sizeof(uint32_t);
  l.count_off = sizeof(Header);  // zeroed per call together with the header
  l.total_off = align_up(l.count_off + l.entries * words, 256);
  l.start_off = align_up(l.total_off + (chunked ? buckets * words : 0), 256);
  l.cursor_off = align_up(l.start_off + (buckets + 1) * words, 256);
  l.local_off = align_up(l.cursor_off + l.entries * words, 256);
  l.block_sum_off = align_up(l.local_off + (chunked ? l.entries * words : 0), 256);
  l.run_start_off = align_up(l.block_sum_off + (chunked ? l.scan_blocks * words : 0), 256);
  l.run_length_off = align_up(l.run_start_off + (chunked ? l.entries * words : 0), 256);
  l.records_off = align_up(l.run_length_off + (chunked ? l.entries * words : 0), 256);
  l.total = align_up(l.records_off + static_cast<size_t>(n) * kRecordWords * words, 256);
  return l;
}

}  // namespace

BucketPlan plan_buckets(int64_t n, int64_t num_cells) {
  // Largest bucket width 2^s (s <= 10: the counters of the finish kernel resolve 15
  // low key bits and its tie step two more) whose average load stays at or below the
  // target.
  BucketPlan p;
  p.shift = 0;
  const int64_t target = 4224;
  for (int s = kMaxShift; s >= 0; --s) {
    const int64_t buckets = (num_cells + (int64_t{1} << s) - 1) >> s;
    // Fewer than 2048 buckets make the slot counters of the scatter contend (measured at 1 M
    // and 4 M particles: 2048 beats 1024, 4096 and 8192).
    if ((n <= target * buckets && buckets >= 2048) || s == 0) {
      p.shift = s;
      break;
    }
  }
  p.buckets = (num_cells + (int64_t{1} << p.shift) - 1) >> p.shift;
  p.usable = n > 0 && n <= target * p.buckets && p.buckets <= (int64_t{1} << 24);
  return p;
}

size_t bucketed_workspace_bytes(int64_t n, int64_t num_cells) {
  const BucketPlan p = plan_buckets(n, num_cells);
  return bucket_layout(n, p.buckets).total;
}

// Enqueues the bucketed path.  When a bucket turns out too large for the finish
// kernel the device sets Header::use_standard and the remaining kernels return
// at once; the caller then enqueues the digit-pass path predicated on that flag.
cudaError_t bucketed_sort(const SortArgs& a, const BucketPlan& p) {
  const BucketLayout l = bucket_layout(a.n, p.buckets);
  if (a.workspace_bytes < l.total) return cudaErrorInvalidValue;
  auto* base = static_cast<unsigned char*>(a.workspace);
  auto words_at = [&](size_t off) { return reinterpret_cast<uint32_t*>(base + off); };
  Header* hdr = reinterpret_cast<Header*>(base);
  const bool chunked = l.chunks > 1;
  uint32_t* count = words_at(l.count_off);
  uint32_t* total = chunked ? words_at(l.total_off) : count;
  uint32_t* start = words_at(l.start_off);
  uint32_t* cursor = words_at(l.cursor_off);
  uint32_t* records = words_at(l.records_off);
  cudaError_t e = cudaMemsetAsync(base, 0, l.total_off, a.stream);  // header and run counts
  if (e != cudaSuccess) return e;
  const int buckets = static_cast<int>(p.buckets);
  const uint32_t k0 = static_cast<uint32_t>(a.seed), k1 = static_cast<uint32_t>(a.seed >> 32);
  const bool vec = aligned16(a.x) && aligned16(a.y) && aligned16(a.z) &&
                   (!a.velocity || (aligned16(a.velocity) && a.padded % 4 == 0));
  const size_t table_bytes = static_cast<size_t>(buckets) * sizeof(uint32_t);

  stage_begin(kStageBucketCount, a.stream);
  {
    const bool shared = table_bytes <= 200 * 1024;
    const bool wide = table_bytes > 96 * 1024;  // one 1024-thread block per SM holds the table
    const int threads = shared && wide ? kCountThreadsWide : kCountThreads;
    const int blocks_per_sm = shared ? (wide ? 1 : table_bytes <= 48 * 1024 ? 4 : 2) : 4;
    const int64_t chunk_size = int64_t{1} << l.chunk_log;
    const int64_t covered = std::min<int64_t>(a.n, chunk_size);
    // Slices of a chunk: enough units to fill the GPU twice over, each a multiple of one
    // block round (4 particles per thread) so that the 16-byte loads stay aligned.
    const int want = std::max(1, sm_count() * blocks_per_sm * 2 / l.chunks);
    const int64_t round = threads * 4;
    const int64_t slice = std::max<int64_t>(round, ((covered + want - 1) / want + round - 1) / round * round);
    const int parts = static_cast<int>((covered + slice - 1) / slice);
    const int grid = std::max(1, std::min(l.chunks * parts, sm_count() * blocks_per_sm));
    if (shared) {
      auto kernel = wide ? (vec ? bucket_count_kernel<true, true, kCountThreadsWide>
                                : bucket_count_kernel<true, false, kCountThreadsWide>)
                         : (vec ? bucket_count_kernel<true, true, kCountThreads>
                                : bucket_count_kernel<true, false, kCountThreads>);
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(table_bytes));
      if (e != cudaSuccess) return e;
      kernel<<<grid, threads, table_bytes, a.stream>>>(a.x, a.y, a.z, a.velocity, a.padded, a.push,
                                                       a.n, a.grid, p.shift, buckets, l.chunks,
                                                       l.chunk_log, parts, slice, count);
    } else {
      auto kernel = vec ? bucket_count_kernel<false, true, kCountThreads>
                        : bucket_count_kernel<false, false, kCountThreads>;
      kernel<<<grid, threads, 0, a.stream>>>(a.x, a.y, a.z, a.velocity, a.padded, a.push, a.n,
                                             a.grid, p.shift, buckets, l.chunks, l.chunk_log,
                                             parts, slice, count);
    }
  }
  stage_end(kStageBucketCount, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  stage_begin(kStageBucketScan, a.stream);
  uint32_t* run_start = nullptr;
  uint32_t* run_length = nullptr;
  if (chunked) {
    uint32_t* local = words_at(l.local_off);
    uint32_t* block_sum = words_at(l.block_sum_off);
    run_start = words_at(l.run_start_off);
    run_length = words_at(l.run_length_off);
    bucket_total_kernel<<<(buckets + 255) / 256, 256, 0, a.stream>>>(count, buckets, l.chunks, total);
    bucket_scan_kernel<<<1, kScanThreads, 0, a.stream>>>(total, buckets, a.n, kLargestBucket,
                                                         start, nullptr, hdr);
    run_scan_local_kernel<<<l.scan_blocks, kFlatScanBlock, 0, a.stream>>>(count, l.entries, local,
                                                                          block_sum);
    run_scan_blocks_kernel<<<1, kFlatScanBlock, 0, a.stream>>>(block_sum, l.scan_blocks);
    run_table_kernel<<<static_cast<int>((l.entries + 255) / 256), 256, 0, a.stream>>>(
        count, local, block_sum, buckets, l.chunks, cursor, run_start, run_length);
    count_launches(5);
  } else {
    bucket_scan_kernel<<<1, kScanThreads, 0, a.stream>>>(count, buckets, a.n, kLargestBucket,
                                                         start, cursor, hdr);
    count_launches(1);
  }
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
    kernel<<<grid, kScatterThreads, 0, a.stream>>>(a.x, a.y, a.z, a.velocity, a.padded, a.push,
                                                    a.n, a.grid, k0, k1, p.shift, buckets,
                                                    l.chunk_log, cursor, records, hdr);
  }
  stage_end(kStageBucketScatter, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  count_launches(2);

  stage_begin(kStageBucketFinish, a.stream);
  const FinishOut out{a.keys_out, a.index_out, a.cell_counts, a.cell_start, a.xs, a.ys, a.zs,
                      a.vs, a.padded_sorted};
  {
    const int drop = std::max(0, p.shift + kShuffleBits - kMaxLowBits);
    auto kernel = drop == 0 ? bucket_finish_kernel<0>
                            : drop == 1 ? bucket_finish_kernel<1> : bucket_finish_kernel<2>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(FinishSmem)));
    if (e != cudaSuccess) return e;
    kernel<<<std::min(buckets, sm_count()), kFinishThreads, sizeof(FinishSmem), a.stream>>>(
        records, start, run_start, run_length, l.chunks, buckets, p.shift, a.n, a.num_cells, out,
        hdr);
  }
  e = cudaFuncSetAttribute(bucket_finish_large_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(sizeof(FinishSmem)));
  if (e != cudaSuccess) return e;
  bucket_finish_large_kernel<<<std::min(buckets, sm_count()), kFinishThreads, sizeof(FinishSmem),
                               a.stream>>>(records, start, run_start, run_length, l.chunks,
                                           buckets, p.shift, a.num_cells, out, hdr);
  stage_end(kStageBucketFinish, a.stream);
  count_launches(2);
  return cudaGetLastError();
}

}  // namespace aether
