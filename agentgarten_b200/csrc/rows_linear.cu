// y = x W^T + b for a handful of FP32 rows against a wide weight matrix (the timestep embedder:
// a few rows by 256 -> 4096 -> 4096), evaluated in FP32 with the weights read in their own type
// (bf16 or fp32) and never copied to FP32 first.  With at most 64 rows the products are bound by
// reading W once, which a tensor-core tile of 128 rows would not change.  Forward and the three
// gradients; every sum has a fixed order (no atomics).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "agb.h"

namespace agb {
namespace {

constexpr int RL_ROWS = 8;    // rows of x handled per pass over a weight row
constexpr int RL_SLICE = 64;  // output columns per block of the input-gradient kernel

template <typename T> __device__ __forceinline__ float rl_load(const T* p);
template <> __device__ __forceinline__ float rl_load<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float rl_load<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
// eight consecutive weights as floats (the row offset is a multiple of 8)
__device__ __forceinline__ void rl_load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void rl_load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// One warp per output column n: y[m, n] = b[n] + sum_k x[m, k] W[n, k]; a lane takes eight
// consecutive k per step (k is a multiple of 8).
template <typename T>
__global__ void __launch_bounds__(256) rows_linear_fwd_kernel(const float* __restrict__ x, const T* __restrict__ w,
                                                              const T* __restrict__ bias, float* __restrict__ y,
                                                              int m, int n, int k) {
  const int col = (blockIdx.x * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (col >= n) return;
  const T* row = w + int64_t(col) * k;
  for (int m0 = 0; m0 < m; m0 += RL_ROWS) {
    float acc[RL_ROWS];
#pragma unroll
    for (int r = 0; r < RL_ROWS; ++r) acc[r] = 0.f;
    for (int kk = lane * 8; kk < k; kk += 256) {
      float wv[8];
      rl_load8(row + kk, wv);
#pragma unroll
      for (int r = 0; r < RL_ROWS; ++r) {
        if (m0 + r < m) {
          float xv[8];
          rl_load8(x + int64_t(m0 + r) * k + kk, xv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[r] += wv[i] * xv[i];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RL_ROWS; ++r) {
      float v = acc[r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0 && m0 + r < m) y[int64_t(m0 + r) * n + col] = v + (bias ? rl_load<T>(bias + col) : 0.f);
    }
  }
}

// partial[slice, m, k] = sum over the RL_SLICE columns n of the slice of dy[m, n] W[n, k]:
// one thread per k (coalesced weight rows), dy of the slice in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) rows_linear_dx_kernel(const float* __restrict__ dy, const T* __restrict__ w,
                                                             float* __restrict__ partial, int m, int n, int k) {
  __shared__ float tile[RL_ROWS][RL_SLICE];
  const int kk = blockIdx.x * 256 + threadIdx.x;
  const int n0 = blockIdx.y * RL_SLICE;
  const int cols = min(RL_SLICE, n - n0);
  for (int m0 = 0; m0 < m; m0 += RL_ROWS) {
    __syncthreads();
    for (int i = threadIdx.x; i < RL_ROWS * RL_SLICE; i += 256) {
      const int r = i / RL_SLICE, c = i - r * RL_SLICE;
      tile[r][c] = (m0 + r < m && c < cols) ? dy[int64_t(m0 + r) * n + n0 + c] : 0.f;
    }
    __syncthreads();
    if (kk < k) {
      float acc[RL_ROWS];
#pragma unroll
      for (int r = 0; r < RL_ROWS; ++r) acc[r] = 0.f;
      for (int c = 0; c < cols; ++c) {
        const float wv = rl_load<T>(w + int64_t(n0 + c) * k + kk);
#pragma unroll
        for (int r = 0; r < RL_ROWS; ++r) acc[r] += wv * tile[r][c];
      }
#pragma unroll
      for (int r = 0; r < RL_ROWS; ++r) {
        if (m0 + r < m) partial[(int64_t(blockIdx.y) * m + m0 + r) * k + kk] = acc[r];
      }
    }
  }
}

// dx[i] = sum over the slices, in slice order.
__global__ void __launch_bounds__(256) rows_linear_dx_sum_kernel(const float* __restrict__ partial,
                                                                 float* __restrict__ dx, int64_t elements,
                                                                 int slices) {
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= elements) return;
  float acc = 0.f;
  for (int s = 0; s < slices; ++s) acc += partial[int64_t(s) * elements + i];
  dx[i] = acc;
}

// dW[n, k..k+3] = sum_m dy[m, n] x[m, k..k+3] (one thread per four elements, k a multiple of 4),
// db[n] = sum_m dy[m, n].
__global__ void __launch_bounds__(256) rows_linear_dw_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                             float* __restrict__ dw, float* __restrict__ db, int m,
                                                             int n, int k) {
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  const int quads = k / 4;
  if (i >= int64_t(n) * quads) return;
  const int col = int(i / quads), kk = int(i - int64_t(col) * quads) * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float accb = 0.f;
  for (int r = 0; r < m; ++r) {
    const float g = dy[int64_t(r) * n + col];
    const float4 xv = *reinterpret_cast<const float4*>(x + int64_t(r) * k + kk);
    acc.x += g * xv.x; acc.y += g * xv.y; acc.z += g * xv.z; acc.w += g * xv.w;
    accb += g;
  }
  *reinterpret_cast<float4*>(dw + int64_t(col) * k + kk) = acc;
  if (db && kk == 0) db[col] = accb;
}

}  // namespace

int rows_linear_slices(int n) { return (n + RL_SLICE - 1) / RL_SLICE; }

cudaError_t rows_linear_fwd(const float* x, const void* w, const void* bias, float* y, int m, int n, int k,
                            bool bf16_weights, cudaStream_t stream) {
  if (m == 0 || n == 0) return cudaSuccess;
  if (k % 8) return cudaErrorInvalidValue;
  const unsigned grid = unsigned((int64_t(n) * 32 + 255) / 256);
  if (bf16_weights) {
    rows_linear_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        x, static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(bias), y, m, n, k);
  } else {
    rows_linear_fwd_kernel<float><<<grid, 256, 0, stream>>>(x, static_cast<const float*>(w),
                                                           static_cast<const float*>(bias), y, m, n, k);
  }
  return cudaGetLastError();
}

cudaError_t rows_linear_bwd(const float* dy, const float* x, const void* w, float* dx, float* dx_partial,
                            float* dw, float* db, int m, int n, int k, bool bf16_weights, cudaStream_t stream) {
  if (m == 0 || n == 0 || k == 0) return cudaSuccess;
  if (k % 8) return cudaErrorInvalidValue;
  if (dx) {
    const int slices = rows_linear_slices(n);
    const dim3 grid(unsigned((k + 255) / 256), unsigned(slices));
    if (bf16_weights) {
      rows_linear_dx_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(dy, static_cast<const __nv_bfloat16*>(w),
                                                                     dx_partial, m, n, k);
    } else {
      rows_linear_dx_kernel<float><<<grid, 256, 0, stream>>>(dy, static_cast<const float*>(w), dx_partial, m, n, k);
    }
    const int64_t elements = int64_t(m) * k;
    rows_linear_dx_sum_kernel<<<unsigned((elements + 255) / 256), 256, 0, stream>>>(dx_partial, dx, elements, slices);
  }
  if (dw) {
    const unsigned grid = unsigned((int64_t(n) * (k / 4) + 255) / 256);
    rows_linear_dw_kernel<<<grid, 256, 0, stream>>>(dy, x, dw, db, m, n, k);
  }
  return cudaGetLastError();
}

}  // namespace agb
