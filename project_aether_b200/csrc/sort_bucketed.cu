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
#include <algorithm>

#include "common.cuh"

namespace aether {

namespace {

constexpr int kSmCount = 148;
constexpr int kRecordWords = 8;  // 32-byte record

// ------------------------------------------------------------------------
// Upsweep: particles per bucket.
// ------------------------------------------------------------------------
constexpr int kCountThreads = 512;

// Adds one to a histogram bin per lane; a warp whose lanes all hit the same bin
// (every particle in one cell) issues a single add.
template <bool SHARED>
__device__ __forceinline__ void bin_add(uint32_t* hist, uint32_t bin, bool valid) {
  const uint32_t active = __ballot_sync(0xffffffffu, valid);
  if (active == 0) return;
  const int first = __ffs(active) - 1;
  const uint32_t first_bin = __shfl_sync(0xffffffffu, bin, first);
  const bool uniform = __all_sync(0xffffffffu, !valid || bin == first_bin);
  if (uniform) {
    if (static_cast<int>(lane_id()) == first) atomicAdd(&hist[first_bin], __popc(active));
  } else if (valid) {
    atomicAdd(&hist[bin], 1u);
  }
}

template <bool SHARED, bool VEC>
__global__ void __launch_bounds__(kCountThreads)
bucket_count_kernel(const float* __restrict__ x, const float* __restrict__ y,
                    const float* __restrict__ z, int64_t n, AetherGrid g, int shift,
                    int buckets, uint32_t* __restrict__ bucket_count) {
  extern __shared__ uint32_t hist[];
  if (SHARED) {
    for (int i = threadIdx.x; i < buckets; i += kCountThreads) hist[i] = 0;
    __syncthreads();
  }
  uint32_t* target = SHARED ? hist : bucket_count;
  const int64_t groups = (n + 3) / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kCountThreads;
  const int64_t rounds = (groups + stride - 1) / stride;
  for (int64_t r = 0; r < rounds; ++r) {
    const int64_t i0 = (r * stride + static_cast<int64_t>(blockIdx.x) * kCountThreads +
                        threadIdx.x) * 4;
    float px[4], py[4], pz[4];
    if (VEC && i0 + 4 <= n) {
      const float4 a = ldcs4(x + i0), b = ldcs4(y + i0), c = ldcs4(z + i0);
      px[0] = a.x; px[1] = a.y; px[2] = a.z; px[3] = a.w;
      py[0] = b.x; py[1] = b.y; py[2] = b.z; py[3] = b.w;
      pz[0] = c.x; pz[1] = c.y; pz[2] = c.z; pz[3] = c.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool ok = i0 + k < n;
        px[k] = ok ? x[i0 + k] : 0.f;
        py[k] = ok ? y[i0 + k] : 0.f;
        pz[k] = ok ? z[i0 + k] : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      bin_add<SHARED>(target, cell_of(px[k], py[k], pz[k], g) >> shift, i0 + k < n);
  }
  if (SHARED) {
    __syncthreads();
    for (int i = threadIdx.x; i < buckets; i += kCountThreads)
      if (hist[i]) atomicAdd(&bucket_count[i], hist[i]);
  }
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
    cursor[b] = run;
    run += bucket_count[b];
  }
  if (tid == 0) {
    bucket_start[buckets] = static_cast<uint32_t>(n);
    hdr->max_bucket = biggest;
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

// Reserves one slot in bucket `b`; a warp whose lanes all target one bucket
// reserves its slots with a single atomic.
__device__ __forceinline__ uint32_t reserve_slot(uint32_t* cursor, uint32_t b, bool valid) {
  const uint32_t active = __ballot_sync(0xffffffffu, valid);
  if (active == 0) return 0;
  const int first = __ffs(active) - 1;
  const uint32_t first_b = __shfl_sync(0xffffffffu, b, first);
  const bool uniform = __all_sync(0xffffffffu, !valid || b == first_b);
  uint32_t slot = 0;
  if (uniform) {
    if (static_cast<int>(lane_id()) == first) slot = atomicAdd(&cursor[first_b], __popc(active));
    slot = __shfl_sync(0xffffffffu, slot, first) + __popc(active & lanemask_lt());
  } else if (valid) {
    slot = atomicAdd(&cursor[b], 1u);
  }
  return slot;
}

template <bool VEC>
__global__ void __launch_bounds__(kScatterThreads, 2)
bucket_scatter_kernel(const float* __restrict__ x, const float* __restrict__ y,
                      const float* __restrict__ z, const float* __restrict__ v, int64_t padded,
                      int64_t n, AetherGrid g, uint32_t k0, uint32_t k1, int shift,
                      uint32_t* __restrict__ cursor, uint32_t* __restrict__ records,
                      const Header* __restrict__ hdr) {
  if (hdr->use_standard) return;
  const int64_t groups = (n + 3) / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kScatterThreads;
  const int64_t rounds = (groups + stride - 1) / stride;
  for (int64_t r = 0; r < rounds; ++r) {
    const int64_t i0 = (r * stride + static_cast<int64_t>(blockIdx.x) * kScatterThreads +
                        threadIdx.x) * 4;
    float f[6][4];
    if (VEC && i0 + 4 <= n) {
      const float4 a = ldcs4(x + i0), b = ldcs4(y + i0), c = ldcs4(z + i0);
      f[0][0] = a.x; f[0][1] = a.y; f[0][2] = a.z; f[0][3] = a.w;
      f[1][0] = b.x; f[1][1] = b.y; f[1][2] = b.z; f[1][3] = b.w;
      f[2][0] = c.x; f[2][1] = c.y; f[2][2] = c.z; f[2][3] = c.w;
      if (v) {
        const float4 d = ldcs4(v + i0), e = ldcs4(v + padded + i0), h = ldcs4(v + 2 * padded + i0);
        f[3][0] = d.x; f[3][1] = d.y; f[3][2] = d.z; f[3][3] = d.w;
        f[4][0] = e.x; f[4][1] = e.y; f[4][2] = e.z; f[4][3] = e.w;
        f[5][0] = h.x; f[5][1] = h.y; f[5][2] = h.z; f[5][3] = h.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
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
      for (int k = 0; k < 4; ++k) f[3][k] = f[4][k] = f[5][k] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool ok = i0 + k < n;
      const uint32_t cell = cell_of(f[0][k], f[1][k], f[2][k], g);
      const uint32_t index = static_cast<uint32_t>(i0 + k);
      const uint32_t key = make_key(cell, index, k0, k1);
      const uint32_t slot = reserve_slot(cursor, cell >> shift, ok);
      if (ok)
        store_record(records + static_cast<size_t>(slot) * kRecordWords, key, index, f[0][k],
                     f[1][k], f[2][k], f[3][k], f[4][k], f[5][k]);
    }
  }
}

// ------------------------------------------------------------------------
// Finish: one block sorts one bucket in shared memory and writes the output.
// ------------------------------------------------------------------------
constexpr int kFinishThreads = 1024;
constexpr int kFinishCapacity = 5632;                      // records per bucket
constexpr int kFinishItems = (kFinishCapacity + kFinishThreads - 1) / kFinishThreads;  // 6
constexpr int kMaxLowBits = 15;                            // (cell bits in bucket) + 7
constexpr int kHistWords = (1 << kMaxLowBits) / 4;         // byte counters, 4 per word
constexpr int kWordsPerThread = kHistWords / kFinishThreads;  // 8

struct FinishSmem {
  uint32_t hist[kHistWords];     // byte counter per low-key value; later: final order (u16)
  uint16_t word_prefix[kHistWords];  // exclusive prefix of each counter word
  uint16_t slot_of[kFinishCapacity];  // record held by each sorted slot (before the tie pass)
  uint16_t low_key[kFinishCapacity];  // low key bits of each sorted slot
  uint32_t index[kFinishCapacity];
  float field[6][kFinishCapacity];
  uint32_t warp_sum[32];
  uint32_t total;
};
static_assert(sizeof(FinishSmem) <= 227 * 1024, "finish kernel shared memory");

__device__ __forceinline__ uint32_t byte_sum(uint32_t w) { return __dp4a(w, 0x01010101u, 0u); }

__global__ void __launch_bounds__(kFinishThreads, 1)
bucket_finish_kernel(const uint32_t* __restrict__ records, const uint32_t* __restrict__ bucket_start,
                     int buckets, int shift, int64_t n, int64_t num_cells,
                     uint32_t* __restrict__ keys_out, int32_t* __restrict__ index_out,
                     int32_t* __restrict__ cell_counts, int32_t* __restrict__ cell_start,
                     float* __restrict__ xs, float* __restrict__ ys, float* __restrict__ zs,
                     float* __restrict__ vs, int64_t padded_sorted, Header* __restrict__ hdr) {
  if (hdr->use_standard) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  FinishSmem& s = *reinterpret_cast<FinishSmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int low_bits = shift + kShuffleBits;
  const uint32_t low_mask = (1u << low_bits) - 1;
  const int hist_words = max(1, (1 << low_bits) / 4);
  uint16_t* final_slot = reinterpret_cast<uint16_t*>(s.hist);  // reused after the scan is consumed

  for (int b = blockIdx.x; b < buckets; b += gridDim.x) {
    const uint32_t begin = bucket_start[b], end = bucket_start[b + 1];
    const int count = static_cast<int>(end - begin);
    if (count > kFinishCapacity) {  // cannot happen once the scan kernel has checked
      if (tid == 0) hdr->use_standard = 1;
      continue;
    }
    for (int i = tid; i < hist_words; i += kFinishThreads) s.hist[i] = 0;
    __syncthreads();

    // Load the bucket: one 32-byte record per lane and load; keep the payload in
    // shared memory (SoA) and count the low key bits with byte-wide counters.
    uint32_t packed[kFinishItems];  // low key | rank among equal keys << 16
#pragma unroll
    for (int k = 0; k < kFinishItems; ++k) {
      const int r = tid + k * kFinishThreads;
      packed[k] = 0;
      if (r < count) {
        uint32_t w[8];
        const uint32_t* src = records + (static_cast<size_t>(begin) + r) * kRecordWords;
        asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]),
                       "=r"(w[6]), "=r"(w[7])
                     : "l"(src));
        s.index[r] = w[1];
#pragma unroll
        for (int c = 0; c < 6; ++c) s.field[c][r] = __uint_as_float(w[2 + c]);
        const uint32_t low = w[0] & low_mask;
        const int sh = 8 * (low & 3);
        const uint32_t old = atomicAdd(&s.hist[low >> 2], 1u << sh);
        packed[k] = low | (((old >> sh) & 0xffu) << 16);
      }
    }
    __syncthreads();

    // Exclusive scan of the counters (8 words = 32 counters per thread).
    uint32_t local[kWordsPerThread];
    uint32_t sum = 0;
#pragma unroll
    for (int j = 0; j < kWordsPerThread; ++j) {
      const int w = tid * kWordsPerThread + j;
      local[j] = sum;
      sum += w < hist_words ? byte_sum(s.hist[w]) : 0u;
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
#pragma unroll
    for (int j = 0; j < kWordsPerThread; ++j) {
      const int w = tid * kWordsPerThread + j;
      if (w < hist_words) s.word_prefix[w] = static_cast<uint16_t>(thread_base + local[j]);
    }
    // A byte counter that wrapped (more than 255 equal keys) loses 255 from the
    // total: hand the whole call to the digit-pass path.
    const bool wrapped = s.total != static_cast<uint32_t>(count);
    __syncthreads();
    if (wrapped) {
      if (tid == 0) hdr->use_standard = 1;
      continue;
    }

    // Cell tables of this bucket: every cell is 128 consecutive counters.
    {
      const int64_t first_cell = static_cast<int64_t>(b) << shift;
      const int cells_here = static_cast<int>(
          min(static_cast<long long>(1) << shift, static_cast<long long>(num_cells - first_cell)));
      for (int c = tid; c < cells_here; c += kFinishThreads) {
        const uint32_t lo = s.word_prefix[c * 32];
        const uint32_t hi = (c + 1) * 32 < hist_words ? s.word_prefix[(c + 1) * 32]
                                                       : static_cast<uint32_t>(count);
        cell_start[first_cell + c] = static_cast<int32_t>(begin + lo);
        cell_counts[first_cell + c] = static_cast<int32_t>(hi - lo);
      }
      if (b == buckets - 1 && tid == 0) cell_start[num_cells] = static_cast<int32_t>(n);
    }

    // Sorted slot of every record.
#pragma unroll
    for (int k = 0; k < kFinishItems; ++k) {
      const int r = tid + k * kFinishThreads;
      if (r < count) {
        const uint32_t low = packed[k] & 0xffffu, rank = packed[k] >> 16;
        const uint32_t word = s.hist[low >> 2];
        const uint32_t below = byte_sum(word & ((1u << (8 * (low & 3))) - 1u));
        const uint32_t slot = s.word_prefix[low >> 2] + below + rank;
        s.slot_of[slot] = static_cast<uint16_t>(r);
        s.low_key[slot] = static_cast<uint16_t>(low);
      }
    }
    __syncthreads();

    // Equal keys must appear in ascending original index: a slot inside a run
    // of equal keys moves to (run start + number of smaller indices in the run).
    for (int d = tid; d < count; d += kFinishThreads) {
      const uint16_t key = s.low_key[d];
      const uint16_t rec = s.slot_of[d];
      int dst = d;
      const bool tie = (d > 0 && s.low_key[d - 1] == key) || (d + 1 < count && s.low_key[d + 1] == key);
      if (tie) {
        const uint32_t mine = s.index[rec];
        int lo = d, smaller = 0;
        while (lo > 0 && s.low_key[lo - 1] == key) {
          --lo;
          smaller += s.index[s.slot_of[lo]] < mine;
        }
        for (int j = d + 1; j < count && s.low_key[j] == key; ++j)
          smaller += s.index[s.slot_of[j]] < mine;
        dst = lo + smaller;
      }
      final_slot[dst] = rec;
    }
    __syncthreads();

    // Coalesced output.
    const uint32_t key_high = static_cast<uint32_t>(b) << low_bits;
    for (int d = tid; d < count; d += kFinishThreads) {
      const int rec = final_slot[d];
      const size_t o = static_cast<size_t>(begin) + d;
      keys_out[o] = (low_bits < 32 ? key_high : 0u) | s.low_key[d];
      index_out[o] = static_cast<int32_t>(s.index[rec]);
      xs[o] = s.field[0][rec];
      ys[o] = s.field[1][rec];
      zs[o] = s.field[2][rec];
      if (vs) {
        vs[o] = s.field[3][rec];
        vs[padded_sorted + o] = s.field[4][rec];
        vs[2 * padded_sorted + o] = s.field[5][rec];
      }
    }
    __syncthreads();
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

struct BucketLayout {
  size_t count_off, start_off, cursor_off, records_off, total;
};

BucketLayout bucket_layout(int64_t n, int64_t buckets) {
  BucketLayout l;
  l.count_off = sizeof(Header);
  l.start_off = align_up(l.count_off + buckets * sizeof(uint32_t), 256);
  l.cursor_off = align_up(l.start_off + (buckets + 1) * sizeof(uint32_t), 256);
  l.records_off = align_up(l.cursor_off + buckets * sizeof(uint32_t), 256);
  l.total = align_up(l.records_off + static_cast<size_t>(n) * kRecordWords * sizeof(uint32_t), 256);
  return l;
}

}  // namespace

BucketPlan plan_buckets(int64_t n, int64_t num_cells) {
  // Largest bucket width 2^s (s <= 8 so the low key fits 15 bits) whose average
  // load stays at or below the target.
  BucketPlan p;
  p.shift = 0;
  const int64_t target = 4608;
  for (int s = 8; s >= 0; --s) {
    const int64_t buckets = (num_cells + (int64_t{1} << s) - 1) >> s;
    if (n <= target * buckets || s == 0) {
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
  Header* hdr = reinterpret_cast<Header*>(base);
  uint32_t* count = reinterpret_cast<uint32_t*>(base + l.count_off);
  uint32_t* start = reinterpret_cast<uint32_t*>(base + l.start_off);
  uint32_t* cursor = reinterpret_cast<uint32_t*>(base + l.cursor_off);
  uint32_t* records = reinterpret_cast<uint32_t*>(base + l.records_off);
  cudaError_t e = cudaMemsetAsync(base, 0, l.start_off, a.stream);
  if (e != cudaSuccess) return e;
  const int buckets = static_cast<int>(p.buckets);
  const uint32_t k0 = static_cast<uint32_t>(a.seed), k1 = static_cast<uint32_t>(a.seed >> 32);
  const bool vec = aligned16(a.x) && aligned16(a.y) && aligned16(a.z) &&
                   (!a.velocity || (aligned16(a.velocity) && a.padded % 4 == 0));

  stage_begin(kStageBucketCount, a.stream);
  {
    const int64_t groups = (a.n + 3) / 4;
    const size_t smem = static_cast<size_t>(buckets) * sizeof(uint32_t);
    const bool shared = smem <= 96 * 1024;
    const int per_sm = shared ? (smem <= 48 * 1024 ? 4 : 2) : 4;
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>((groups + kCountThreads - 1) / kCountThreads, kSmCount * per_sm)));
    if (shared) {
      auto kernel = vec ? bucket_count_kernel<true, true> : bucket_count_kernel<true, false>;
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
      if (e != cudaSuccess) return e;
      kernel<<<grid, kCountThreads, smem, a.stream>>>(a.x, a.y, a.z, a.n, a.grid, p.shift,
                                                       buckets, count);
    } else {
      auto kernel = vec ? bucket_count_kernel<false, true> : bucket_count_kernel<false, false>;
      kernel<<<grid, kCountThreads, 0, a.stream>>>(a.x, a.y, a.z, a.n, a.grid, p.shift, buckets,
                                                    count);
    }
  }
  stage_end(kStageBucketCount, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  stage_begin(kStageBucketScan, a.stream);
  bucket_scan_kernel<<<1, kScanThreads, 0, a.stream>>>(count, buckets, a.n, kFinishCapacity, start,
                                                       cursor, hdr);
  stage_end(kStageBucketScan, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  stage_begin(kStageBucketScatter, a.stream);
  {
    const int64_t groups = (a.n + 3) / 4;
    const int grid = static_cast<int>(std::max<int64_t>(
        1, std::min<int64_t>((groups + kScatterThreads - 1) / kScatterThreads, kSmCount * 2)));
    auto kernel = vec ? bucket_scatter_kernel<true> : bucket_scatter_kernel<false>;
    kernel<<<grid, kScatterThreads, 0, a.stream>>>(a.x, a.y, a.z, a.velocity, a.padded, a.n,
                                                    a.grid, k0, k1, p.shift, cursor, records, hdr);
  }
  stage_end(kStageBucketScatter, a.stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  stage_begin(kStageBucketFinish, a.stream);
  e = cudaFuncSetAttribute(bucket_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(sizeof(FinishSmem)));
  if (e != cudaSuccess) return e;
  bucket_finish_kernel<<<std::min(buckets, kSmCount), kFinishThreads, sizeof(FinishSmem),
                         a.stream>>>(records, start, buckets, p.shift, a.n, a.num_cells,
                                     a.keys_out, a.index_out, a.cell_counts, a.cell_start, a.xs,
                                     a.ys, a.zs, a.vs, a.padded_sorted, hdr);
  stage_end(kStageBucketFinish, a.stream);
  count_launches(4);
  return cudaGetLastError();
}

}  // namespace aether
