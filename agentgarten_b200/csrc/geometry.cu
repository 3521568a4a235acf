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


// ------------------------------------------------------------------ pooling, blur, warp
// All three work on frame stacks [images, H, W] (fp32), one thread per output pixel.

// Mean over factor x factor windows (floor division of the extent, as avg_pool2d does), with
// non-finite inputs read as zero.
__global__ void __launch_bounds__(NT) pool_frames_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                         int64_t images, int h, int w, int factor) {
  const int oh = h / factor, ow = w / factor;
  const int64_t total = images * oh * ow;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int x = int(i % ow), y = int((i / ow) % oh);
    const int64_t image = i / (int64_t(ow) * oh);
    const float* base = src + (image * h + int64_t(y) * factor) * w + int64_t(x) * factor;
    float sum = 0.f;
    for (int dy = 0; dy < factor; ++dy) {
      for (int dx = 0; dx < factor; ++dx) {
        const float v = base[int64_t(dy) * w + dx];
        sum += isfinite(v) ? v : 0.f;
      }
    }
    dst[i] = sum / float(factor * factor);
  }
}

// One pass of a separable blur with replicated borders: along x (horizontal = 1) or along y.
__global__ void __launch_bounds__(NT) blur_pass_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                       const float* __restrict__ taps, int radius,
                                                       int64_t images, int h, int w, int horizontal) {
  const int64_t total = images * h * w;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int x = int(i % w), y = int((i / w) % h);
    const float* plane = src + (i / (int64_t(w) * h)) * int64_t(h) * w;
    float sum = 0.f;
    for (int k = -radius; k <= radius; ++k) {
      const int xx = horizontal ? min(max(x + k, 0), w - 1) : x;
      const int yy = horizontal ? y : min(max(y + k, 0), h - 1);
      sum += taps[k + radius] * plane[int64_t(yy) * w + xx];
    }
    dst[i] = sum;
  }
}

// Scale / shift / shear / perspective warp of frame t of sample b with bilinear sampling and
// border clamping (grid_sample, align_corners = false).  params[b * frames + t] holds
// (sx, sy, tx, ty, hx, hy, px, py); a frame whose `copy` flag is set is copied unchanged.
// Layout [B, C, T, H, W]; the sampling grid is never materialised.
__global__ void __launch_bounds__(NT) warp_frames_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                         const float* __restrict__ params,
                                                         const uint8_t* __restrict__ copy, int64_t batch,
                                                         int channels, int frames, int h, int w) {
  const int64_t total = batch * channels * frames * int64_t(h) * w;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int x = int(i % w), y = int((i / w) % h);
    const int64_t plane_index = i / (int64_t(w) * h);       // (b * C + c) * T + t
    const int t = int(plane_index % frames);
    const int64_t b = plane_index / (int64_t(frames) * channels);
    const float* plane = src + plane_index * int64_t(h) * w;
    if (copy[b * frames + t]) {
      dst[i] = plane[int64_t(y) * w + x];
      continue;
    }
    const float* q = params + (b * frames + t) * 8;
    const float gx = (x + 0.5f) * (2.0f / w) - 1.0f, gy = (y + 0.5f) * (2.0f / h) - 1.0f;
    const float denom = fmaxf(1.0f + q[6] * gx + q[7] * gy, 0.5f);
    const float u = (q[0] * gx + q[4] * gy + q[2]) / denom;
    const float v = (q[5] * gx + q[1] * gy + q[3]) / denom;
    // normalised -> pixel coordinates (align_corners = false), clamped to the border
    const float fx = fminf(fmaxf(((u + 1.0f) * w - 1.0f) * 0.5f, 0.f), float(w - 1));
    const float fy = fminf(fmaxf(((v + 1.0f) * h - 1.0f) * 0.5f, 0.f), float(h - 1));
    const int x0 = int(floorf(fx)), y0 = int(floorf(fy));
    const int x1 = min(x0 + 1, w - 1), y1 = min(y0 + 1, h - 1);
    const float ax = fx - x0, ay = fy - y0;
    const float top = plane[int64_t(y0) * w + x0] * (1.f - ax) + plane[int64_t(y0) * w + x1] * ax;
    const float bottom = plane[int64_t(y1) * w + x0] * (1.f - ax) + plane[int64_t(y1) * w + x1] * ax;
    dst[i] = top * (1.f - ay) + bottom * ay;
  }
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


static unsigned geometry_grid(int64_t total) {
  return unsigned(std::min<int64_t>((total + NT - 1) / NT, 148 * 32));
}

cudaError_t pool_frames(const float* src, float* dst, int64_t images, int h, int w, int factor,
                        cudaStream_t stream) {
  if (factor < 1 || h / factor < 1 || w / factor < 1) return cudaErrorInvalidValue;
  const int64_t total = images * (h / factor) * (w / factor);
  if (total == 0) return cudaSuccess;
  pool_frames_kernel<<<geometry_grid(total), NT, 0, stream>>>(src, dst, images, h, w, factor);
  return cudaGetLastError();
}

cudaError_t blur_frames(const float* src, float* scratch, float* dst, const float* taps, int radius,
                        int64_t images, int h, int w, cudaStream_t stream) {
  const int64_t total = images * int64_t(h) * w;
  if (total == 0) return cudaSuccess;
  if (radius < 0) return cudaErrorInvalidValue;
  blur_pass_kernel<<<geometry_grid(total), NT, 0, stream>>>(src, scratch, taps, radius, images, h, w, 1);
  blur_pass_kernel<<<geometry_grid(total), NT, 0, stream>>>(scratch, dst, taps, radius, images, h, w, 0);
  return cudaGetLastError();
}

cudaError_t warp_frames(const float* src, float* dst, const float* params, const uint8_t* copy, int64_t batch,
                        int channels, int frames, int h, int w, cudaStream_t stream) {
  const int64_t total = batch * channels * frames * int64_t(h) * w;
  if (total == 0) return cudaSuccess;
  warp_frames_kernel<<<geometry_grid(total), NT, 0, stream>>>(src, dst, params, copy, batch, channels, frames,
                                                             h, w);
  return cudaGetLastError();
}

}  // namespace agb
