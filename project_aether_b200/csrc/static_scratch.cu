// AetherSortParticlesByCellStatic: the sort with its scratch memory in a fixed
// array that is part of the library image, for callers that are not allowed to
// allocate device memory.  Small calls (the bucketed layout of their records fits
// the array: up to a few hundred thousand particles) take the bucketed path, larger
// ones the digit passes; the results are the same.
#include "common.cuh"

namespace aether {
namespace {

// Largest particle count the fixed scratch serves (2^20).
constexpr int64_t kStaticMaxParticles = int64_t{1} << 20;
// Scratch of the digit-pass path for that many particles: header, per-tile
// status words of four passes, and one spare key and index array (about 8.7 MiB).
constexpr size_t kStaticScratchBytes = size_t{9} << 20;

// The scratch itself.  Every GPU that loads the library reserves it until the
// process exits.  In host code this name only stands for the symbol: the device
// address must be asked for with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_address[kMaxDevices];  // device address of the array, per device

// Device address of the array on the current device, looked up on first use.
cudaError_t scratch_address(void** address) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidValue;
  if (!g_scratch_address[device]) {
    void* looked_up = nullptr;
    e = cudaGetSymbolAddress(&looked_up, g_static_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_address[device] = looked_up;
  }
  *address = g_scratch_address[device];
  return cudaSuccess;
}

}  // namespace
}  // namespace aether

using namespace aether;

extern "C" int64_t AetherSortStaticMaxParticles(void) { return kStaticMaxParticles; }

extern "C" int AetherSortParticlesByCellStatic(const float* x, const float* y, const float* z,
                                               int64_t n, const AetherGrid* grid, uint64_t seed,
                                               uint32_t* keys_out, int32_t* index_out,
                                               int32_t* cell_counts, int32_t* cell_start,
                                               void* stream) {
  if (!grid || n < 0 || n > kStaticMaxParticles) return cudaErrorInvalidValue;
  const int64_t cells = static_cast<int64_t>(grid->nx_local) * grid->ny * grid->nz;
  if (cells <= 0) return cudaErrorInvalidValue;
  if (standard_workspace_bytes(n, cells) > kStaticScratchBytes) return cudaErrorInvalidValue;
  void* scratch = nullptr;  // the first call on a device looks the array's address up
  const cudaError_t e = scratch_address(&scratch);
  if (e != cudaSuccess) return e;
  return AetherSortParticlesByCell(x, y, z, n, grid, seed, keys_out, index_out, cell_counts,
                                   cell_start, scratch, kStaticScratchBytes, stream);
}

extern "C" int AetherSortStaticReadStatus(void* stream, int32_t* status) {
  void* scratch = nullptr;
  const cudaError_t e = scratch_address(&scratch);
  if (e != cudaSuccess) return e;
  return AetherSortReadStatus(scratch, stream, status);
}

extern "C" int AetherSortStaticReadUsedDigitPasses(void* stream, int32_t* used) {
  void* scratch = nullptr;
  const cudaError_t e = scratch_address(&scratch);
  if (e != cudaSuccess) return e;
  return AetherSortReadUsedDigitPasses(scratch, stream, used);
}
