// Depthwise k x k convolution (stride 1, zero padding k / 2) of channels-last 16-bit frames:
//   out[n, h, w, c] = bias[c] + sum_{dh, dw} x[n, h + dh - k/2, w + dw - k/2, c] * weight[dh * k + dw, c]
// The 7x7 depthwise stage of the wide TAEHV decoder blocks is memory-bound; this kernel keeps
// each input value in registers for all the taps of a row that use it.  A thread owns 8
// channels (one 16-byte vector) of 4 consecutive pixels of a row, so neighbouring threads
// read neighbouring 16-byte vectors of the same pixels and the k + 3 vectors a thread loads
// per input row serve 4 * k products each.  Accumulation is fp32.
#include "agb.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace agb {
namespace {

constexpr int PIXELS = 4;  // consecutive output pixels per thread

template <bool HALF>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (HALF) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    } else {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
}

template <bool HALF>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (HALF) {
      const __half2 p = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&p);
    } else {
      const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

template <bool HALF, int K>
__global__ void __launch_bounds__(256)
depthwise_kernel(const uint4* __restrict__ x, const uint4* __restrict__ weight,
                 const uint4* __restrict__ bias, uint4* __restrict__ out, int frames, int height,
                 int width, int groups /* channels / 8 */, int64_t items) {
  const int64_t item = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= items) return;
  const int quads = (width + PIXELS - 1) / PIXELS;
  const int g = int(item % groups);
  int64_t rest = item / groups;
  const int w0 = int(rest % quads) * PIXELS;
  rest /= quads;
  const int h = int(rest % height);
  const int n = int(rest / height);

  float acc[PIXELS][8];
  {
    float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (bias) unpack8<HALF>(bias[g], b);
#pragma unroll
    for (int j = 0; j < PIXELS; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = b[i];
  }

  constexpr int R = K / 2;
  const uint4* frame = x + int64_t(n) * height * width * groups;
#pragma unroll 1
  for (int dh = 0; dh < K; ++dh) {
    const int hh = h + dh - R;
    if (hh < 0 || hh >= height) continue;
    const uint4* row = frame + int64_t(hh) * width * groups + g;
    uint4 in[PIXELS + K - 1];
#pragma unroll
    for (int j = 0; j < PIXELS + K - 1; ++j) {
      const int ww = w0 + j - R;
      in[j] = (ww >= 0 && ww < width) ? __ldg(row + int64_t(ww) * groups) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int dw = 0; dw < K; ++dw) {
      float wt[8];
      unpack8<HALF>(__ldg(weight + int64_t(dh * K + dw) * groups + g), wt);
#pragma unroll
      for (int j = 0; j < PIXELS; ++j) {
        float v[8];
        unpack8<HALF>(in[j + dw], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][i] = fmaf(v[i], wt[i], acc[j][i]);
      }
    }
  }

  uint4* dst = out + ((int64_t(n) * height + h) * width + w0) * groups + g;
#pragma unroll
  for (int j = 0; j < PIXELS; ++j)
    if (w0 + j < width) dst[int64_t(j) * groups] = pack8<HALF>(acc[j]);
}

template <bool HALF>
cudaError_t launch(const DepthwiseArgs& a, cudaStream_t stream) {
  const int groups = a.channels / 8;
  const int quads = (a.width + PIXELS - 1) / PIXELS;
  const int64_t items = int64_t(a.frames) * a.height * quads * groups;
  const int64_t blocks = (items + 255) / 256;
  if (blocks > 0x7FFFFFFF) {
    set_error_detail("depthwise: too many blocks for one launch");
    return cudaErrorInvalidValue;
  }
  const uint4* x = static_cast<const uint4*>(a.x);
  const uint4* w = static_cast<const uint4*>(a.weight);
  const uint4* b = static_cast<const uint4*>(a.bias);
  uint4* out = static_cast<uint4*>(a.out);
  (void)cudaGetLastError();
  switch (a.kernel) {
    case 3:
      depthwise_kernel<HALF, 3><<<int(blocks), 256, 0, stream>>>(x, w, b, out, a.frames, a.height,
                                                                 a.width, groups, items);
      break;
    case 5:
      depthwise_kernel<HALF, 5><<<int(blocks), 256, 0, stream>>>(x, w, b, out, a.frames, a.height,
                                                                 a.width, groups, items);
      break;
    case 7:
      depthwise_kernel<HALF, 7><<<int(blocks), 256, 0, stream>>>(x, w, b, out, a.frames, a.height,
                                                                 a.width, groups, items);
      break;
    default:
      set_error_detail("depthwise: kernel size must be 3, 5 or 7");
      return cudaErrorInvalidValue;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_error_detail("depthwise: kernel launch failed");
  return e;
}

}  // namespace

cudaError_t depthwise_conv(const DepthwiseArgs& a, cudaStream_t stream) {
  if (a.frames <= 0 || a.height <= 0 || a.width <= 0) return cudaSuccess;
  if ((a.channels % 8) || (reinterpret_cast<uintptr_t>(a.x) & 15) ||
      (reinterpret_cast<uintptr_t>(a.weight) & 15) || (reinterpret_cast<uintptr_t>(a.bias) & 15) ||
      (reinterpret_cast<uintptr_t>(a.out) & 15)) {
    set_error_detail("depthwise: channels must be a multiple of 8 and pointers 16-byte aligned");
    return cudaErrorInvalidValue;
  }
  return a.fp16 ? launch<true>(a, stream) : launch<false>(a, stream);
}

}  // namespace agb
