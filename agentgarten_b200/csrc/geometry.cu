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


// ------------------------------------------------------------------ resampling
// Bilinear source position of output index `o` when `in` samples are resized to `out` with
// pixel centres aligned (the half-pixel rule of interpolate(..., align_corners=False)):
// the lower sample, whether an upper one exists, and the weight of the upper one.
struct Lerp {
  int lo, step;
  float w;
};
__device__ __forceinline__ Lerp lerp_of(int o, int in, int out) {
  const float scale = float(in) / float(out);
  float src = scale * (float(o) + 0.5f) - 0.5f;
  src = src < 0.f ? 0.f : src;
  Lerp r;
  r.lo = min(int(src), in - 1);
  r.step = r.lo < in - 1 ? 1 : 0;
  r.w = src - float(r.lo);
  return r;
}

// Mean over the source bin of each output pixel, bins as in adaptive average pooling:
// [floor(o * in / out), ceil((o + 1) * in / out)).
__global__ void __launch_bounds__(NT) area_frames_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                         int64_t images, int h, int w, int oh, int ow) {
  const int64_t total = images * oh * ow;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int x = int(i % ow), y = int((i / ow) % oh);
    const float* plane = src + (i / (int64_t(ow) * oh)) * int64_t(h) * w;
    const int y0 = int(int64_t(y) * h / oh), y1 = int((int64_t(y + 1) * h + oh - 1) / oh);
    const int x0 = int(int64_t(x) * w / ow), x1 = int((int64_t(x + 1) * w + ow - 1) / ow);
    float sum = 0.f;
    for (int yy = y0; yy < y1; ++yy)
      for (int xx = x0; xx < x1; ++xx) sum += plane[int64_t(yy) * w + xx];
    dst[i] = sum / float((y1 - y0) * (x1 - x0));
  }
}

__global__ void __launch_bounds__(NT) bilinear_frames_kernel(const float* __restrict__ src,
                                                             float* __restrict__ dst, int64_t images, int h,
                                                             int w, int oh, int ow) {
  const int64_t total = images * oh * ow;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int x = int(i % ow), y = int((i / ow) % oh);
    const float* plane = src + (i / (int64_t(ow) * oh)) * int64_t(h) * w;
    const Lerp ly = lerp_of(y, h, oh), lx = lerp_of(x, w, ow);
    const float* r0 = plane + int64_t(ly.lo) * w + lx.lo;
    const float* r1 = r0 + int64_t(ly.step) * w;
    const float top = (1.f - lx.w) * r0[0] + lx.w * r0[lx.step];
    const float bottom = (1.f - lx.w) * r1[0] + lx.w * r1[lx.step];
    dst[i] = (1.f - ly.w) * top + ly.w * bottom;
  }
}

// Quadrant stretch of [B, planes, H, W] to [B, planes, TH, TW]: the upper H/2 rows are resized
// bilinearly to H/2 + top[b] rows and the lower ones take the rest of TH; then the left W/2
// columns to W/2 + left[b] and the right ones the rest of TW.  Rows first, columns second, as
// two separate resizes would round.
__global__ void __launch_bounds__(NT) stretch_frames_kernel(const float* __restrict__ src,
                                                            float* __restrict__ dst,
                                                            const int* __restrict__ top,
                                                            const int* __restrict__ left, int64_t batch,
                                                            int64_t planes, int h, int w, int th, int tw) {
  const int64_t total = batch * planes * th * tw;
  const int up = h / 2, left_w = w / 2;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int x = int(i % tw), y = int((i / tw) % th);
    const int64_t plane_index = i / (int64_t(tw) * th);
    const int64_t sample = plane_index / planes;
    const float* plane = src + plane_index * int64_t(h) * w;
    const int rows_above = up + top[sample], cols_left = left_w + left[sample];
    Lerp ly, lx;
    int y_base = 0, x_base = 0;
    if (y < rows_above) {
      ly = lerp_of(y, up, rows_above);
    } else {
      ly = lerp_of(y - rows_above, h - up, th - rows_above);
      y_base = up;
    }
    if (x < cols_left) {
      lx = lerp_of(x, left_w, cols_left);
    } else {
      lx = lerp_of(x - cols_left, w - left_w, tw - cols_left);
      x_base = left_w;
    }
    const float* c0 = plane + int64_t(y_base + ly.lo) * w + x_base + lx.lo;
    const float* c1 = c0 + lx.step;
    const int64_t down = int64_t(ly.step) * w;
    const float near = (1.f - ly.w) * c0[0] + ly.w * c0[down];
    const float far = (1.f - ly.w) * c1[0] + ly.w * c1[down];
    dst[i] = (1.f - lx.w) * near + lx.w * far;
  }
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

cudaError_t resize_frames(const float* src, float* dst, int64_t images, int h, int w, int oh, int ow,
                          int area, cudaStream_t stream) {
  if (h < 1 || w < 1 || oh < 1 || ow < 1) return cudaErrorInvalidValue;
  const int64_t total = images * int64_t(oh) * ow;
  if (total == 0) return cudaSuccess;
  if (area)
    area_frames_kernel<<<geometry_grid(total), NT, 0, stream>>>(src, dst, images, h, w, oh, ow);
  else
    bilinear_frames_kernel<<<geometry_grid(total), NT, 0, stream>>>(src, dst, images, h, w, oh, ow);
  return cudaGetLastError();
}

cudaError_t stretch_frames(const float* src, float* dst, const int* top, const int* left, int64_t batch,
                           int64_t planes, int h, int w, int th, int tw, cudaStream_t stream) {
  if (h < 2 || w < 2 || th < h || tw < w) return cudaErrorInvalidValue;
  const int64_t total = batch * planes * int64_t(th) * tw;
  if (total == 0) return cudaSuccess;
  stretch_frames_kernel<<<geometry_grid(total), NT, 0, stream>>>(src, dst, top, left, batch, planes, h, w,
                                                                th, tw);
  return cudaGetLastError();
}

}  // namespace agb
