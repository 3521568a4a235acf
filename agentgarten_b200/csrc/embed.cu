// Small index kernels around the transformer: M-RoPE tables and the patch <-> latent layouts.
//
//   rope_tables   cos / sin [B, N, 128] from positions [B, N, 3] (time, row, column): slot j of the
//                 64 frequencies takes the position of axis[j] times inverse[j]; the angle is
//                 formed in FP32 (as the PyTorch definition does) and its cosine and sine are
//                 evaluated in double precision, so the FP32 value they are rounded from is
//                 exact whatever the fast-math setting of the build.
//   patchify      [B, C, T, H, W] -> [B, T, (H/p)(W/p), p*p*C] (patch pixels row-major, C fastest),
//                 with the cast to the output type in the same pass.
//   unpatchify    the inverse layout (also the gradient of patchify), with the cast.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "agb.h"

namespace agb {
namespace {

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T>
__global__ void __launch_bounds__(256) rope_tables_kernel(const float* __restrict__ positions,
                                                          const float* __restrict__ inverse,
                                                          const int* __restrict__ axis, T* __restrict__ cosine,
                                                          T* __restrict__ sine, int64_t tokens) {
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= tokens * 64) return;
  const int64_t token = i >> 6;
  const int slot = int(i & 63);
  const float angle = positions[token * 3 + axis[slot]] * inverse[slot];
  double s, c;
  sincos(double(angle), &s, &c);
  const T cv = from_float<T>(float(c)), sv = from_float<T>(float(s));
  cosine[token * 128 + slot] = cv;
  cosine[token * 128 + 64 + slot] = cv;
  sine[token * 128 + slot] = sv;
  sine[token * 128 + 64 + slot] = sv;
}

struct PatchShape {
  int64_t batch, channels, frames, height, width;  // of the latent
  int patch;
};

// One thread per element of the patch layout (coalesced on that side).
template <typename In, typename Out, bool TO_PATCHES>
__global__ void __launch_bounds__(256) patch_kernel(const In* __restrict__ src, Out* __restrict__ dst,
                                                    PatchShape s, int64_t total) {
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total) return;
  const int p = s.patch;
  const int64_t gw = s.width / p, gh = s.height / p;
  int64_t r = i;
  const int64_t c = r % s.channels; r /= s.channels;
  const int64_t q = r % p; r /= p;
  const int64_t pp = r % p; r /= p;
  const int64_t w = r % gw; r /= gw;
  const int64_t h = r % gh; r /= gh;
  const int64_t t = r % s.frames;
  const int64_t b = r / s.frames;
  const int64_t latent = (((b * s.channels + c) * s.frames + t) * s.height + h * p + pp) * s.width + w * p + q;
  if (TO_PATCHES) dst[i] = from_float<Out>(to_float<In>(src[latent]));
  else dst[latent] = from_float<Out>(to_float<In>(src[i]));
}

template <typename In, typename Out>
cudaError_t launch_patch(const void* src, void* dst, const PatchShape& s, bool to_patches, cudaStream_t stream) {
  const int64_t total = s.batch * s.channels * s.frames * s.height * s.width;
  if (total == 0) return cudaSuccess;
  const unsigned grid = unsigned((total + 255) / 256);
  if (to_patches) {
    patch_kernel<In, Out, true><<<grid, 256, 0, stream>>>(static_cast<const In*>(src), static_cast<Out*>(dst), s, total);
  } else {
    patch_kernel<In, Out, false><<<grid, 256, 0, stream>>>(static_cast<const In*>(src), static_cast<Out*>(dst), s, total);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t rope_tables(const float* positions, const float* inverse, const int* axis, void* cosine, void* sine,
                        int64_t tokens, bool bf16_out, cudaStream_t stream) {
  if (tokens == 0) return cudaSuccess;
  const unsigned grid = unsigned((tokens * 64 + 255) / 256);
  if (bf16_out) {
    rope_tables_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(positions, inverse, axis,
                                                                static_cast<__nv_bfloat16*>(cosine),
                                                                static_cast<__nv_bfloat16*>(sine), tokens);
  } else {
    rope_tables_kernel<float><<<grid, 256, 0, stream>>>(positions, inverse, axis, static_cast<float*>(cosine),
                                                        static_cast<float*>(sine), tokens);
  }
  return cudaGetLastError();
}

cudaError_t patch_layout(const void* src, void* dst, int64_t batch, int64_t channels, int64_t frames,
                         int64_t height, int64_t width, int patch, bool to_patches, bool src_bf16,
                         bool dst_bf16, cudaStream_t stream) {
  if (patch < 1 || height % patch || width % patch) return cudaErrorInvalidValue;
  const PatchShape s{batch, channels, frames, height, width, patch};
  if (src_bf16 && dst_bf16) return launch_patch<__nv_bfloat16, __nv_bfloat16>(src, dst, s, to_patches, stream);
  if (src_bf16) return launch_patch<__nv_bfloat16, float>(src, dst, s, to_patches, stream);
  if (dst_bf16) return launch_patch<float, __nv_bfloat16>(src, dst, s, to_patches, stream);
  return launch_patch<float, float>(src, dst, s, to_patches, stream);
}

}  // namespace agb
