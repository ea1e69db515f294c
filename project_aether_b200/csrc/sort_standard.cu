// Digit-pass path of the particle sort:
//   keygen_upsweep_kernel  cell id + Philox shuffle bits -> keys, and the digit
//                          histograms of every pass from the same read
//                          (replaces _bin_keys_kernel, fused_radix_sort.py:63-113)
//   onesweep_pass_kernel   one stable 8-bit digit pass with a decoupled
//                          look-back chained scan over per-tile status words
//                          (replaces _onesweep_kernel, fused_radix_sort.py:116-203)
//   cell_bounds_kernel / cell_counts_kernel
//                          cell_start and cell_counts from the sorted keys
//                          (replaces the last-pass atomics and torch.cumsum,
//                          fused_radix_sort.py:201-203,277-279)
//   gather_kernel          sorted SoA payload (dsmc_gpu_pipeline.py:107-109)
#include <algorithm>

#include "common.cuh"

namespace aether {

namespace {

// ------------------------------------------------------------------------
// Key generation + upsweep.
// ------------------------------------------------------------------------
constexpr int kKeygenThreads = 256;
constexpr int kKeygenVec = 4;
constexpr int kKeygenChunk = kKeygenThreads * kKeygenVec;

template <int PASSES, bool VEC>
__global__ void __launch_bounds__(kKeygenThreads)
keygen_upsweep_kernel(const float* __restrict__ x, const float* __restrict__ y,
                      const float* __restrict__ z, const float4* __restrict__ records, int64_t n,
                      AetherGrid g, uint32_t k0, uint32_t k1, uint32_t* __restrict__ keys,
                      uint32_t* __restrict__ global_hist, const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  __shared__ uint32_t hist[PASSES][kRadix];
  for (int i = threadIdx.x; i < PASSES * kRadix; i += kKeygenThreads) (&hist[0][0])[i] = 0;
  __syncthreads();
  const int64_t chunks = (n + kKeygenChunk - 1) / kKeygenChunk;
  for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
    const int64_t i0 = c * kKeygenChunk + threadIdx.x * kKeygenVec;
    float px[kKeygenVec], py[kKeygenVec], pz[kKeygenVec];
    uint32_t key[kKeygenVec];
    if (records) {  // positions as the fused move stage left them in the payload records
#pragma unroll
      for (int k = 0; k < kKeygenVec; ++k) {
        const float4 r = i0 + k < n ? __ldg(records + 2 * (i0 + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
        px[k] = r.x; py[k] = r.y; pz[k] = r.z;
      }
    } else if (VEC && i0 + kKeygenVec <= n) {
      const float4 a = ldcs4(x + i0), b = ldcs4(y + i0), d = ldcs4(z + i0);
      px[0] = a.x; px[1] = a.y; px[2] = a.z; px[3] = a.w;
      py[0] = b.x; py[1] = b.y; py[2] = b.z; py[3] = b.w;
      pz[0] = d.x; pz[1] = d.y; pz[2] = d.z; pz[3] = d.w;
    } else {
#pragma unroll
      for (int k = 0; k < kKeygenVec; ++k) {
        const bool ok = i0 + k < n;
        px[k] = ok ? x[i0 + k] : 0.f;
        py[k] = ok ? y[i0 + k] : 0.f;
        pz[k] = ok ? z[i0 + k] : 0.f;
      }
    }
#pragma unroll
    for (int k = 0; k < kKeygenVec; ++k)
      key[k] = make_key(cell_of(px[k], py[k], pz[k], g), static_cast<uint32_t>(i0 + k), k0, k1);
    if (VEC && i0 + kKeygenVec <= n) {
      __stcs(reinterpret_cast<uint4*>(keys + i0), make_uint4(key[0], key[1], key[2], key[3]));
    } else {
#pragma unroll
      for (int k = 0; k < kKeygenVec; ++k)
        if (i0 + k < n) keys[i0 + k] = key[k];
    }
#pragma unroll
    for (int k = 0; k < kKeygenVec; ++k) {
      const bool ok = i0 + k < n;
#pragma unroll
      for (int p = 0; p < PASSES; ++p)
        bin_add(hist[p], (key[k] >> (kRadixBits * p)) & (kRadix - 1), ok);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < PASSES * kRadix; i += kKeygenThreads) {
    const uint32_t v = (&hist[0][0])[i];
    if (v) atomicAdd(&global_hist[i], v);
  }
}

template <bool VEC>
__global__ void __launch_bounds__(kKeygenThreads)
make_keys_kernel(const float* __restrict__ x, const float* __restrict__ y,
                 const float* __restrict__ z, int64_t n, AetherGrid g, uint32_t k0, uint32_t k1,
                 uint32_t* __restrict__ keys) {
  const int64_t chunks = (n + kKeygenChunk - 1) / kKeygenChunk;
  for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
    const int64_t i0 = c * kKeygenChunk + threadIdx.x * kKeygenVec;
#pragma unroll
    for (int k = 0; k < kKeygenVec; ++k)
      if (i0 + k < n)
        keys[i0 + k] = make_key(cell_of(x[i0 + k], y[i0 + k], z[i0 + k], g),
                                static_cast<uint32_t>(i0 + k), k0, k1);
  }
}

// ------------------------------------------------------------------------
// One Onesweep digit pass.
// ------------------------------------------------------------------------
constexpr int kPassThreads = 384;
constexpr int kPassItems = 16;
constexpr int kPassWarps = kPassThreads / 32;
constexpr int kPassTile = kPassThreads * kPassItems;  // 6144 keys
constexpr uint32_t kPollLimit = 1u << 22;             // look-back polls before giving up

struct PassSmem {
  uint32_t keys[kPassTile];
  uint32_t vals[kPassTile];
  uint32_t warp_count[kPassWarps][kRadix];
  uint32_t tile_offset[kRadix];   // exclusive scan of the tile's digit histogram
  int64_t global_base[kRadix];    // output index of staged slot 0 of each digit
  uint32_t scan_scratch[8];
  uint32_t tile_id;
  uint32_t abort;
};

// FIRST: the values are the particle indices themselves and are synthesised
// instead of read (the key kernel does not write an index array).
template <bool FIRST>
__global__ void __launch_bounds__(kPassThreads, 2)
onesweep_pass_kernel(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                     uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t n,
                     int shift, const uint32_t* __restrict__ digit_total,
                     uint32_t* __restrict__ status, uint32_t* __restrict__ tile_counter,
                     uint32_t tiles, int32_t* __restrict__ error, uint32_t poll_limit,
                     const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  PassSmem& s = *reinterpret_cast<PassSmem*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // A block works through tiles until none is left.  Tiles are handed out in
  // ticket order and a block holds one tile at a time, so every tile a block
  // waits on belongs to a block that is already running.
  if (tid == 0) s.abort = 0;
  for (;;) {
  if (tid == 0) s.tile_id = atomicAdd(tile_counter, 1u);
#pragma unroll
  for (int i = lane; i < kRadix; i += 32) s.warp_count[warp][i] = 0;
  __syncthreads();
  const uint32_t tile = s.tile_id;
  if (tile >= tiles) break;
  const int64_t tile_base = static_cast<int64_t>(tile) * kPassTile;
  const int valid = static_cast<int>(min(static_cast<long long>(kPassTile), static_cast<long long>(n - tile_base)));

  // Warp-striped load: item k of lane l is element warp*32*ITEMS + k*32 + l,
  // so (k, lane) order is index order.  Slots past the end get the largest key;
  // they rank after every real key of the last tile and are never written out.
  const int warp_first = warp * 32 * kPassItems + lane;
  uint32_t key[kPassItems], rank[kPassItems];
#pragma unroll
  for (int k = 0; k < kPassItems; ++k) {
    const int e = warp_first + k * 32;
    key[k] = e < valid ? __ldcs(keys_in + tile_base + e) : 0xffffffffu;
  }

  // Stable rank inside the warp's segment: lanes with equal digits find each
  // other with match.any; the lowest of them advances the warp's counter.
  uint32_t* wc = s.warp_count[warp];
#pragma unroll
  for (int k = 0; k < kPassItems; ++k) {
    const uint32_t d = (key[k] >> shift) & (kRadix - 1);
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    const int leader = __ffs(peers) - 1;
    uint32_t before = 0;
    if (lane == leader) {
      before = wc[d];
      wc[d] = before + __popc(peers);
    }
    __syncwarp();
    rank[k] = __shfl_sync(0xffffffffu, before, leader) + __popc(peers & lanemask_lt());
  }
  __syncthreads();

  // Per digit: turn the warps' counts into exclusive offsets, publish the tile
  // aggregate, scan the tile histogram, look back.
  uint32_t tile_count = 0;
  if (tid < kRadix) {
#pragma unroll
    for (int w = 0; w < kPassWarps; ++w) {
      const uint32_t c = s.warp_count[w][tid];
      s.warp_count[w][tid] = tile_count;
      tile_count += c;
    }
    st_relaxed(status + static_cast<size_t>(tile) * kRadix + tid,
               tile_count | (tile == 0 ? kFlagInclusive : kFlagAggregate));
  }
  // Exclusive scans over the 256 digits (threads 0..255 = warps 0..7): the
  // tile's own histogram and the pass's global histogram.
  uint32_t total = 0, tile_excl = 0, total_excl = 0;
  if (tid < kRadix) {
    total = digit_total[tid];
    uint32_t a = tile_count, b = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t ta = __shfl_up_sync(0xffffffffu, a, o), tb = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) { a += ta; b += tb; }
    }
    if (lane == 31) {
      s.scan_scratch[warp] = a;
      s.tile_offset[warp] = b;  // borrowed as scratch until the barrier below
    }
    tile_excl = a - tile_count;
    total_excl = b - total;
  }
  __syncthreads();
  uint32_t tile_carry = 0, total_carry = 0;
  if (tid < kRadix) {
    for (int w = 0; w < warp; ++w) {
      tile_carry += s.scan_scratch[w];
      total_carry += s.tile_offset[w];
    }
  }
  __syncthreads();
  if (tid < kRadix) {
    tile_excl += tile_carry;
    total_excl += total_carry;
    s.tile_offset[tid] = tile_excl;
    // Decoupled look-back over the predecessors' status words of this digit.
    uint32_t exclusive = 0;
    bool gave_up = false;
    for (int64_t pred = static_cast<int64_t>(tile) - 1; pred >= 0; --pred) {
      const uint32_t* word_ptr = status + static_cast<size_t>(pred) * kRadix + tid;
      uint32_t word = ld_relaxed(word_ptr);
      uint32_t polls = 0;
      while ((word & kFlagMask) == 0) {
        if (++polls > poll_limit) { gave_up = true; break; }
        __nanosleep(32);
        word = ld_relaxed(word_ptr);
      }
      if (gave_up) break;
      exclusive += word & kValueMask;
      if ((word & kFlagMask) == kFlagInclusive) break;
    }
    if (gave_up) {
      atomicCAS(error, 0, kErrLookbackTimeout);
      s.abort = 1;
    }
    if (tile != 0)
      st_relaxed(status + static_cast<size_t>(tile) * kRadix + tid,
                 ((exclusive + tile_count) & kValueMask) | kFlagInclusive);
    s.global_base[tid] = static_cast<int64_t>(total_excl) + exclusive - tile_excl;
  }
  __syncthreads();

  // Stage the tile in digit order in shared memory.
#pragma unroll
  for (int k = 0; k < kPassItems; ++k) {
    const uint32_t d = (key[k] >> shift) & (kRadix - 1);
    rank[k] += s.tile_offset[d] + s.warp_count[warp][d];
    s.keys[rank[k]] = key[k];
  }
#pragma unroll
  for (int k = 0; k < kPassItems; ++k) {
    const int e = warp_first + k * 32;
    uint32_t v;
    if (FIRST) v = static_cast<uint32_t>(tile_base + e);
    else v = e < valid ? __ldcs(vals_in + tile_base + e) : 0u;
    s.vals[rank[k]] = v;
  }
  __syncthreads();
  if (s.abort) return;

  // Coalesced scatter: consecutive staged slots of one digit go to consecutive
  // output slots.
#pragma unroll 4
  for (int j = tid; j < valid; j += kPassThreads) {
    const uint32_t kk = s.keys[j];
    const int64_t dst = s.global_base[(kk >> shift) & (kRadix - 1)] + j;
    keys_out[dst] = kk;
    vals_out[dst] = s.vals[j];
  }
  __syncthreads();  // the staged tile and the ticket slot are reused by the next tile
  }
}

// ------------------------------------------------------------------------
// cell_start / cell_counts from the sorted keys.
// ------------------------------------------------------------------------
constexpr int kBoundsThreads = 256;

// Position i in [0, n] is a boundary when its cell differs from the cell of
// position i-1 (cell -1 before the first key, cell C after the last).  The
// boundary thread writes `i` as the start of every cell in (previous, current];
// long runs of empty cells are filled by the whole warp.
__global__ void __launch_bounds__(kBoundsThreads)
cell_bounds_kernel(const uint32_t* __restrict__ keys, int64_t n, int64_t num_cells,
                   int32_t* __restrict__ cell_start, const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  const int lane = threadIdx.x & 31;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kBoundsThreads;
  const int64_t rounds = (n + 1 + stride - 1) / stride;
  for (int64_t r = 0; r < rounds; ++r) {
    const int64_t i = r * stride + static_cast<int64_t>(blockIdx.x) * kBoundsThreads + threadIdx.x;
    int64_t first = 0, last = -1;  // cells [first, last] start at i
    if (i <= n) {
      const int64_t cur = i < n ? static_cast<int64_t>(keys[i] >> kShuffleBits) : num_cells;
      const int64_t prev = i > 0 ? static_cast<int64_t>(keys[i - 1] >> kShuffleBits) : -1;
      first = prev + 1;
      last = cur;
    }
    const bool is_long = last - first >= 32;
    if (!is_long)
      for (int64_t c = first; c <= last; ++c) cell_start[c] = static_cast<int32_t>(i);
    uint32_t pending = __ballot_sync(0xffffffffu, is_long);
    while (pending) {
      const int src = __ffs(pending) - 1;
      pending &= pending - 1;
      const int64_t f = __shfl_sync(0xffffffffu, first, src);
      const int64_t l = __shfl_sync(0xffffffffu, last, src);
      const int32_t v = static_cast<int32_t>(__shfl_sync(0xffffffffu, i, src));
      for (int64_t c = f + lane; c <= l; c += 32) cell_start[c] = v;
    }
  }
}

__global__ void __launch_bounds__(kBoundsThreads)
cell_counts_kernel(const int32_t* __restrict__ cell_start, int64_t num_cells,
                   int32_t* __restrict__ cell_counts, const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kBoundsThreads;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * kBoundsThreads + threadIdx.x; c < num_cells;
       c += stride)
    cell_counts[c] = cell_start[c + 1] - cell_start[c];
}

// ------------------------------------------------------------------------
// Payload gather by the final permutation.
// ------------------------------------------------------------------------
constexpr int kGatherThreads = 256;

template <bool VEC>
__global__ void __launch_bounds__(kGatherThreads)
gather_kernel(const int32_t* __restrict__ index, int64_t n, const float* __restrict__ x,
              const float* __restrict__ y, const float* __restrict__ z,
              const float* __restrict__ v, int64_t padded, float* __restrict__ xs,
              float* __restrict__ ys, float* __restrict__ zs, float* __restrict__ vs,
              int64_t padded_sorted, const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kGatherThreads * 4;
  for (int64_t i0 = (static_cast<int64_t>(blockIdx.x) * kGatherThreads + threadIdx.x) * 4; i0 < n;
       i0 += stride) {
    if (VEC && i0 + 4 <= n) {
      const int4 p = __ldcs(reinterpret_cast<const int4*>(index + i0));
      const int q[4] = {p.x, p.y, p.z, p.w};
      float o[6][4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        o[0][k] = x[q[k]];
        o[1][k] = y[q[k]];
        o[2][k] = z[q[k]];
        if (v) {
          o[3][k] = v[q[k]];
          o[4][k] = v[padded + q[k]];
          o[5][k] = v[2 * padded + q[k]];
        }
      }
      __stcs(reinterpret_cast<float4*>(xs + i0), make_float4(o[0][0], o[0][1], o[0][2], o[0][3]));
      __stcs(reinterpret_cast<float4*>(ys + i0), make_float4(o[1][0], o[1][1], o[1][2], o[1][3]));
      __stcs(reinterpret_cast<float4*>(zs + i0), make_float4(o[2][0], o[2][1], o[2][2], o[2][3]));
      if (v) {
        __stcs(reinterpret_cast<float4*>(vs + i0),
               make_float4(o[3][0], o[3][1], o[3][2], o[3][3]));
        __stcs(reinterpret_cast<float4*>(vs + padded_sorted + i0),
               make_float4(o[4][0], o[4][1], o[4][2], o[4][3]));
        __stcs(reinterpret_cast<float4*>(vs + 2 * padded_sorted + i0),
               make_float4(o[5][0], o[5][1], o[5][2], o[5][3]));
      }
    } else {
      for (int k = 0; k < 4 && i0 + k < n; ++k) {
        const int q = index[i0 + k];
        xs[i0 + k] = x[q];
        ys[i0 + k] = y[q];
        zs[i0 + k] = z[q];
        if (v) {
          vs[i0 + k] = v[q];
          vs[padded_sorted + i0 + k] = v[padded + q];
          vs[2 * padded_sorted + i0 + k] = v[2 * padded + q];
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kBoundsThreads)
clear_words_kernel(uint32_t* __restrict__ words, size_t count, const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  const size_t stride = static_cast<size_t>(gridDim.x) * kBoundsThreads;
  for (size_t i = static_cast<size_t>(blockIdx.x) * kBoundsThreads + threadIdx.x; i < count;
       i += stride)
    words[i] = 0;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int grid_for(int64_t work_items, int per_block, int blocks_per_sm) {
  const int64_t blocks = (work_items + per_block - 1) / per_block;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks, sm_count() * blocks_per_sm)));
}

// ------------------------------------------------------------------------
// Payload gather through 32-byte records.  Gathering six arrays 4 bytes at a
// time costs six scattered 32-byte sector reads per particle; packing the
// payload into one 32-byte record per particle first (a streaming pass) makes
// it one.  Used when the workspace has room for the records.
// ------------------------------------------------------------------------
constexpr int kRecordThreads = 256;

__global__ void __launch_bounds__(kRecordThreads)
record_build_kernel(const float* __restrict__ x, const float* __restrict__ y,
                    const float* __restrict__ z, const float* __restrict__ v, int64_t padded,
                    PushSpec push, int64_t n, float4* __restrict__ records,
                    const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRecordThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kRecordThreads + threadIdx.x; i < n;
       i += stride) {
    float vx = v ? __ldcs(v + i) : 0.f, vy = v ? __ldcs(v + padded + i) : 0.f;
    float vz = v ? __ldcs(v + 2 * padded + i) : 0.f;
    float px = __ldcs(x + i), py = __ldcs(y + i), pz = __ldcs(z + i);
    if (push.enabled) {
      push_axis(px, vx, push.dt, push.lo[0], push.hi[0]);
      push_axis(py, vy, push.dt, push.lo[1], push.hi[1]);
      push_axis(pz, vz, push.dt, push.lo[2], push.hi[2]);
    }
    records[2 * i] = make_float4(px, py, pz, vx);
    records[2 * i + 1] = make_float4(vy, vz, 0.f, 0.f);
  }
}

__global__ void __launch_bounds__(kRecordThreads)
record_gather_kernel(const int32_t* __restrict__ index, int64_t n,
                     const float4* __restrict__ records, float* __restrict__ xs,
                     float* __restrict__ ys, float* __restrict__ zs, float* __restrict__ vs,
                     int64_t padded_sorted, const int32_t* __restrict__ run_if) {
  chain_begin();
  if (run_if && *run_if == 0) return;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRecordThreads;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * kRecordThreads + threadIdx.x; r < n;
       r += stride) {
    const int64_t i = __ldcs(index + r);
    const float4 a = __ldg(records + 2 * i), b = __ldg(records + 2 * i + 1);
    __stcs(xs + r, a.x);
    __stcs(ys + r, a.y);
    __stcs(zs + r, a.z);
    if (vs) {
      __stcs(vs + r, a.w);
      __stcs(vs + padded_sorted + r, b.x);
      __stcs(vs + 2 * padded_sorted + r, b.y);
    }
  }
}

struct StandardLayout {
  int passes;
  int64_t tiles;
  size_t status_off, keys_alt_off, index_alt_off, total;
};

StandardLayout standard_layout(int64_t n, int key_bits) {
  StandardLayout l;
  l.passes = std::max(1, (key_bits + kRadixBits - 1) / kRadixBits);
  l.tiles = std::max<int64_t>(1, (n + kPassTile - 1) / kPassTile);
  l.status_off = sizeof(Header);
  const size_t status_bytes = static_cast<size_t>(l.passes) * l.tiles * kRadix * sizeof(uint32_t);
  l.keys_alt_off = align_up(l.status_off + status_bytes, 256);
  l.index_alt_off = align_up(l.keys_alt_off + n * sizeof(uint32_t), 256);
  l.total = align_up(l.index_alt_off + n * sizeof(uint32_t), 256);
  return l;
}

}  // namespace

size_t standard_workspace_bytes(int64_t n, int64_t /*num_cells*/) {
  return standard_layout(n, 32).total;
}

// With room for one 32-byte payload record per particle behind the digit-pass arrays.
size_t standard_workspace_bytes_with_records(int64_t n, int64_t num_cells) {
  return standard_workspace_bytes(n, num_cells) + static_cast<size_t>(n) * 32;
}

cudaError_t launch_make_keys(const float* x, const float* y, const float* z, int64_t n,
                             const AetherGrid& g, uint64_t seed, uint32_t* keys,
                             cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  make_keys_kernel<false><<<grid_for(n, kKeygenChunk, 8), kKeygenThreads, 0, stream>>>(
      x, y, z, n, g, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), keys);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t launch_gather(const int32_t* index, int64_t n, const float* x, const float* y,
                          const float* z, const float* velocity, int64_t padded, float* xs,
                          float* ys, float* zs, float* vs, int64_t padded_sorted,
                          cudaStream_t stream, const int32_t* run_if) {
  if (n == 0) return cudaSuccess;
  bool vec = aligned16(index) && aligned16(xs) && aligned16(ys) && aligned16(zs);
  if (velocity) vec = vec && aligned16(vs) && padded_sorted % 4 == 0;
  const int grid = grid_for(n, kGatherThreads * 4, 8);
  const cudaError_t e = launch_chained(vec ? gather_kernel<true> : gather_kernel<false>, grid,
                                       kGatherThreads, 0, stream, index, n, x, y, z, velocity,
                                       padded, xs, ys, zs, vs, padded_sorted, run_if);
  count_launches(1);
  return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_cell_tables(const uint32_t* sorted_keys, int64_t n, int64_t num_cells,
                               int32_t* cell_counts, int32_t* cell_start, cudaStream_t stream,
                               const int32_t* run_if) {
  cudaError_t e = launch_chained(cell_bounds_kernel, grid_for(n + 1, kBoundsThreads, 8),
                                 kBoundsThreads, 0, stream, sorted_keys, n, num_cells, cell_start,
                                 run_if);
  if (e != cudaSuccess) return e;
  e = launch_chained(cell_counts_kernel, grid_for(num_cells, kBoundsThreads, 8), kBoundsThreads, 0,
                     stream, cell_start, num_cells, cell_counts, run_if);
  count_launches(2);
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <int PASSES>
static void launch_keygen(const SortArgs& a, bool vec, const float4* records, uint32_t* keys,
                          Header* hdr, const int32_t* run_if) {
  const int grid = grid_for(a.n, kKeygenChunk, 8);
  const uint32_t k0 = static_cast<uint32_t>(a.seed), k1 = static_cast<uint32_t>(a.seed >> 32);
  launch_chained(vec ? keygen_upsweep_kernel<PASSES, true> : keygen_upsweep_kernel<PASSES, false>,
                 grid, kKeygenThreads, 0, a.stream, a.x, a.y, a.z, records, a.n, a.grid, k0, k1, keys,
                 &hdr->digit_hist[0][0], run_if);
}

int64_t lookback_probe_particles() { return 3 * kPassTile; }

size_t lookback_probe_workspace_bytes() {
  const int64_t n = lookback_probe_particles();
  return standard_layout(n, 8).total + static_cast<size_t>(n) * sizeof(uint32_t);
}

cudaError_t lookback_give_up_probe(void* workspace, size_t workspace_bytes, uint32_t poll_limit,
                                   cudaStream_t stream) {
  const int64_t n = lookback_probe_particles();
  const StandardLayout l = standard_layout(n, 8);  // one pass
  if (workspace_bytes < lookback_probe_workspace_bytes()) return cudaErrorInvalidValue;
  auto* base = static_cast<unsigned char*>(workspace);
  Header* hdr = reinterpret_cast<Header*>(base);
  uint32_t* status = reinterpret_cast<uint32_t*>(base + l.status_off);
  uint32_t* keys_in = reinterpret_cast<uint32_t*>(base + l.keys_alt_off);  // all zero
  uint32_t* keys_out = reinterpret_cast<uint32_t*>(base + l.index_alt_off);
  uint32_t* values_out = reinterpret_cast<uint32_t*>(base + l.total);
  cudaError_t e = cudaMemsetAsync(base, 0, l.total, stream);
  if (e != cudaSuccess) return e;
  // Ticket dispenser at 1 (its low byte): tile 0 is never handed out and never publishes.
  e = cudaMemsetAsync(&hdr->tile_counter[0], 1, 1, stream);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(onesweep_pass_kernel<true>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(PassSmem));
  if (e != cudaSuccess) return e;
  // Two blocks take tiles 1 and 2.  Tile 1 waits for tile 0, runs out of polls, records the
  // error and still publishes its prefix, so that tile 2 does not wait in turn.
  onesweep_pass_kernel<true><<<2, kPassThreads, sizeof(PassSmem), stream>>>(
      keys_in, nullptr, keys_out, values_out, n, 0, hdr->digit_hist[0], status,
      &hdr->tile_counter[0], static_cast<uint32_t>(l.tiles), &hdr->error, poll_limit, nullptr);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t standard_sort(const SortArgs& a, const int32_t* run_if) {
  const StandardLayout l = standard_layout(a.n, a.key_bits);
  if (a.workspace_bytes < l.total) return cudaErrorInvalidValue;
  auto* base = static_cast<unsigned char*>(a.workspace);
  Header* hdr = reinterpret_cast<Header*>(base);
  uint32_t* status = reinterpret_cast<uint32_t*>(base + l.status_off);
  uint32_t* keys_alt = reinterpret_cast<uint32_t*>(base + l.keys_alt_off);
  uint32_t* index_alt = reinterpret_cast<uint32_t*>(base + l.index_alt_off);
  // Zero the header and the status words.  A predicated run keeps the error code and the
  // hand-over flag (the first 8 bytes) and clears with a kernel that, like the others,
  // returns at once when the flag is not set: the usual call then pays one empty launch
  // instead of a memset of tens of megabytes.
  cudaError_t e = cudaSuccess;
  if (run_if) {
    const size_t words = (l.keys_alt_off - 8) / sizeof(uint32_t);
    e = launch_chained(clear_words_kernel,
                       grid_for(static_cast<int64_t>(words), kBoundsThreads * 4, 8), kBoundsThreads,
                       0, a.stream, reinterpret_cast<uint32_t*>(base + 8), words, run_if);
    count_launches(1);
    if (e == cudaSuccess) e = cudaGetLastError();
  } else {
    e = cudaMemsetAsync(base, 0, l.keys_alt_off, a.stream);
  }
  if (e != cudaSuccess) return e;
  // Payload records (one 32-byte sector per particle) behind the digit-pass arrays, when
  // the workspace has room.  Key bits do not change where they start: a 32-bit layout's end.
  const size_t records_off = standard_workspace_bytes(a.n, a.num_cells);
  const bool have_records =
      a.xs && a.n > 0 && a.workspace_bytes >= records_off + static_cast<size_t>(a.n) * 32;
  float4* records = have_records ? reinterpret_cast<float4*>(base + records_off) : nullptr;
  // With the fused move stage the records are built first and the keys come from them.
  if (a.push.enabled && a.n > 0 && !have_records) return cudaErrorInvalidValue;
  const float4* moved = nullptr;
  if (a.push.enabled && a.n > 0) {
    stage_begin(kStagePush, a.stream);
    launch_chained(record_build_kernel, grid_for(a.n, kRecordThreads, 8), kRecordThreads, 0,
                   a.stream, a.x, a.y, a.z, a.velocity, a.padded, a.push, a.n, records, run_if);
    stage_end(kStagePush, a.stream);
    count_launches(1);
    moved = records;
  }

  if (a.n > 0) {
    e = cudaFuncSetAttribute(onesweep_pass_kernel<true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(PassSmem));
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(onesweep_pass_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, sizeof(PassSmem));
    if (e != cudaSuccess) return e;
    // Ping-pong so that the last pass lands in the caller's output arrays.
    uint32_t* out_k = a.keys_out;
    uint32_t* out_v = reinterpret_cast<uint32_t*>(a.index_out);
    uint32_t* cur_k = (l.passes % 2 == 0) ? out_k : keys_alt;
    uint32_t* cur_v = (l.passes % 2 == 0) ? out_v : index_alt;
    uint32_t* nxt_k = (l.passes % 2 == 0) ? keys_alt : out_k;
    uint32_t* nxt_v = (l.passes % 2 == 0) ? index_alt : out_v;
    const bool vec = aligned16(a.x) && aligned16(a.y) && aligned16(a.z) && aligned16(cur_k);
    stage_begin(kStageKeygen, a.stream);
    switch (l.passes) {
      case 1: launch_keygen<1>(a, vec, moved, cur_k, hdr, run_if); break;
      case 2: launch_keygen<2>(a, vec, moved, cur_k, hdr, run_if); break;
      case 3: launch_keygen<3>(a, vec, moved, cur_k, hdr, run_if); break;
      default: launch_keygen<4>(a, vec, moved, cur_k, hdr, run_if); break;
    }
    stage_end(kStageKeygen, a.stream);
    count_launches(1);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int pass_grid = static_cast<int>(std::min<int64_t>(l.tiles, sm_count() * 2));
    for (int p = 0; p < l.passes; ++p) {
      uint32_t* st = status + static_cast<size_t>(p) * l.tiles * kRadix;
      stage_begin(static_cast<Stage>(kStagePass0 + p), a.stream);
      if (p == 0)
        launch_chained(onesweep_pass_kernel<true>, pass_grid, kPassThreads, sizeof(PassSmem),
                       a.stream, cur_k, nullptr, nxt_k, nxt_v, a.n, 0, hdr->digit_hist[0], st,
                       &hdr->tile_counter[0], static_cast<uint32_t>(l.tiles), &hdr->error,
                       kPollLimit, run_if);
      else
        launch_chained(onesweep_pass_kernel<false>, pass_grid, kPassThreads, sizeof(PassSmem),
                       a.stream, cur_k, cur_v, nxt_k, nxt_v, a.n, kRadixBits * p,
                       hdr->digit_hist[p], st, &hdr->tile_counter[p],
                       static_cast<uint32_t>(l.tiles), &hdr->error, kPollLimit, run_if);
      stage_end(static_cast<Stage>(kStagePass0 + p), a.stream);
      count_launches(1);
      e = cudaGetLastError();
      if (e != cudaSuccess) return e;
      uint32_t* t = cur_k; cur_k = nxt_k; nxt_k = t;
      t = cur_v; cur_v = nxt_v; nxt_v = t;
    }
  }
  stage_begin(kStageCellTables, a.stream);
  e = launch_cell_tables(a.keys_out, a.n, a.num_cells, a.cell_counts, a.cell_start, a.stream,
                         run_if);
  stage_end(kStageCellTables, a.stream);
  if (e != cudaSuccess) return e;
  if (a.xs) {
    stage_begin(kStageGather, a.stream);
    if (have_records) {
      const int grid = grid_for(a.n, kRecordThreads, 8);
      if (!moved) {
        launch_chained(record_build_kernel, grid, kRecordThreads, 0, a.stream, a.x, a.y, a.z,
                       a.velocity, a.padded, a.push, a.n, records, run_if);
        count_launches(1);
      }
      launch_chained(record_gather_kernel, grid, kRecordThreads, 0, a.stream, a.index_out, a.n,
                     records, a.xs, a.ys, a.zs, a.vs, a.padded_sorted, run_if);
      count_launches(1);
      e = cudaGetLastError();
    } else {
      e = launch_gather(a.index_out, a.n, a.x, a.y, a.z, a.velocity, a.padded, a.xs, a.ys, a.zs,
                        a.vs, a.padded_sorted, a.stream, run_if);
    }
    stage_end(kStageGather, a.stream);
  }
  return e;
}

}  // namespace aether
