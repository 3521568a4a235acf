// Geometry preprocessing in one pass each: metric depth -> colour-cube RGB, and uint8 normal
// maps -> unit vectors.  Both are pure elementwise maps over planar [B, C, T, H, W] tensors
// that the operator-by-operator formulation spreads over some twenty launches.
#include "agb.h"

#include <math.h>
#include <stdint.h>

namespace agb {
namespace {

constexpr int NT = 256;

__device__ __forceinline__ float ramp(float s, float offset) {
  return fminf(fmaxf(s - offset, 0.f), 1.f);
}

// depth [B, plane], scale [B or 1], out [B, 3, plane].
__global__ void __launch_bounds__(NT) colorize_depth_kernel(
    const float* __restrict__ depth, const float* __restrict__ scale, float* __restrict__ out,
    int64_t plane, int64_t total, int scale_count) {
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int64_t b = i / plane, p = i - b * plane;
    const float d = depth[i];
    const bool valid = isfinite(d) && d > 0.f;
    float r = 0.f, g = 0.f, bl = 0.f;
    if (valid) {
      const float base = 1.f + d * scale[scale_count == 1 ? 0 : b] / 10.f;
      const float t = fminf(fmaxf(1.f - 1.f / (base * base), 0.f), 1.f);
      const float s = t * 7.f;
      r = ramp(s, 0.f) - ramp(s, 2.f) + ramp(s, 5.f);
      g = ramp(s, 1.f) - ramp(s, 4.f) + ramp(s, 6.f);
      bl = ramp(s, 3.f);
    }
    float* o = out + b * 3 * plane + p;
    o[0] = r;
    o[plane] = g;
    o[2 * plane] = bl;
  }
}

// normal uint8 [B, 3, plane] -> float [B, 3, plane]: n = v / 127.5 - 1, normalised; 0 when degenerate.
__global__ void __launch_bounds__(NT) decode_normal_kernel(
    const uint8_t* __restrict__ normal, float* __restrict__ out, int64_t plane, int64_t total) {
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int64_t b = i / plane, p = i - b * plane;
    const uint8_t* src = normal + b * 3 * plane + p;
    const float x = float(src[0]) / 127.5f - 1.f;
    const float y = float(src[plane]) / 127.5f - 1.f;
    const float z = float(src[2 * plane]) / 127.5f - 1.f;
    const float length = sqrtf(x * x + y * y + z * z);
    const float eps = 1.1920929e-07f;
    const float inv = length > eps ? 1.f / length : 0.f;
    float* o = out + b * 3 * plane + p;
    o[0] = x * inv;
    o[plane] = y * inv;
    o[2 * plane] = z * inv;
  }
}

unsigned grid_for(int64_t total) {
  const int64_t blocks = (total + NT - 1) / NT;
  return unsigned(blocks < 148 * 32 ? blocks : 148 * 32);
}

}  // namespace

cudaError_t colorize_depth(const float* depth, const float* scale, float* out, int64_t batch,
                           int64_t plane, int scale_count, cudaStream_t stream) {
  const int64_t total = batch * plane;
  if (total == 0) return cudaSuccess;
  colorize_depth_kernel<<<grid_for(total), NT, 0, stream>>>(depth, scale, out, plane, total, scale_count);
  return cudaGetLastError();
}

cudaError_t decode_normal(const void* normal, float* out, int64_t batch, int64_t plane,
                          cudaStream_t stream) {
  const int64_t total = batch * plane;
  if (total == 0) return cudaSuccess;
  decode_normal_kernel<<<grid_for(total), NT, 0, stream>>>(static_cast<const uint8_t*>(normal), out,
                                                           plane, total);
  return cudaGetLastError();
}

}  // namespace agb
