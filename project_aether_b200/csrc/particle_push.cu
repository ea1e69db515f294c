// Move stage of the DSMC step: x += v*dt with specular reflection at the box
// walls, in place (replaces _push_kernel,
// project_aether/src/custom_kernels/triton/fused_particle_push.py:47-72; the
// arithmetic follows its unfused statement `reference_push`, :95-108: a rounded
// multiply, a rounded add, then `2*wall - c` in float32).
#include <algorithm>

#include "common.cuh"

namespace aether {
namespace {

constexpr int kPushThreads = 256;

template <bool VEC>
__global__ void __launch_bounds__(kPushThreads)
push_kernel(float* __restrict__ x, float* __restrict__ y, float* __restrict__ z,
            float* __restrict__ vx, float* __restrict__ vy, float* __restrict__ vz, int64_t n,
            float dt, float x_lo, float y_lo, float z_lo, float x_hi, float y_hi, float z_hi) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kPushThreads * 4;
  for (int64_t i0 = (static_cast<int64_t>(blockIdx.x) * kPushThreads + threadIdx.x) * 4; i0 < n;
       i0 += stride) {
    if (VEC && i0 + 4 <= n) {
      float4 c[3] = {*reinterpret_cast<float4*>(x + i0), *reinterpret_cast<float4*>(y + i0),
                     *reinterpret_cast<float4*>(z + i0)};
      float4 w[3] = {*reinterpret_cast<float4*>(vx + i0), *reinterpret_cast<float4*>(vy + i0),
                     *reinterpret_cast<float4*>(vz + i0)};
      const float lo[3] = {x_lo, y_lo, z_lo}, hi[3] = {x_hi, y_hi, z_hi};
#pragma unroll
      for (int a = 0; a < 3; ++a) {
        push_axis(c[a].x, w[a].x, dt, lo[a], hi[a]);
        push_axis(c[a].y, w[a].y, dt, lo[a], hi[a]);
        push_axis(c[a].z, w[a].z, dt, lo[a], hi[a]);
        push_axis(c[a].w, w[a].w, dt, lo[a], hi[a]);
      }
      *reinterpret_cast<float4*>(x + i0) = c[0];
      *reinterpret_cast<float4*>(y + i0) = c[1];
      *reinterpret_cast<float4*>(z + i0) = c[2];
      *reinterpret_cast<float4*>(vx + i0) = w[0];
      *reinterpret_cast<float4*>(vy + i0) = w[1];
      *reinterpret_cast<float4*>(vz + i0) = w[2];
    } else {
      for (int k = 0; k < 4 && i0 + k < n; ++k) {
        const int64_t i = i0 + k;
        float c = x[i], w = vx[i];
        push_axis(c, w, dt, x_lo, x_hi);
        x[i] = c; vx[i] = w;
        c = y[i]; w = vy[i];
        push_axis(c, w, dt, y_lo, y_hi);
        y[i] = c; vy[i] = w;
        c = z[i]; w = vz[i];
        push_axis(c, w, dt, z_lo, z_hi);
        z[i] = c; vz[i] = w;
      }
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

cudaError_t particle_push(float* x, float* y, float* z, float* vx, float* vy, float* vz, int64_t n,
                          float dt, const float* lo, const float* hi, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const bool vec = aligned16(x) && aligned16(y) && aligned16(z) && aligned16(vx) &&
                   aligned16(vy) && aligned16(vz);
  const int64_t blocks = (n + kPushThreads * 4 - 1) / (kPushThreads * 4);
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks, sm_count() * 16)));
  stage_begin(kStagePush, stream);
  if (vec)
    push_kernel<true><<<grid, kPushThreads, 0, stream>>>(x, y, z, vx, vy, vz, n, dt, lo[0], lo[1],
                                                         lo[2], hi[0], hi[1], hi[2]);
  else
    push_kernel<false><<<grid, kPushThreads, 0, stream>>>(x, y, z, vx, vy, vz, n, dt, lo[0], lo[1],
                                                          lo[2], hi[0], hi[1], hi[2]);
  stage_end(kStagePush, stream);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace aether
