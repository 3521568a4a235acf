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

constexpr int RL_ROWS = 8;  // rows of x handled per pass over a weight row

template <typename T> __device__ __forceinline__ float rl_load(const T* p);
template <> __device__ __forceinline__ float rl_load<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float rl_load<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

// One warp per output column n: y[m, n] = b[n] + sum_k x[m, k] W[n, k].
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
    for (int kk = lane; kk < k; kk += 32) {
      const float wv = rl_load<T>(row + kk);
#pragma unroll
      for (int r = 0; r < RL_ROWS; ++r) {
        if (m0 + r < m) acc[r] += wv * x[int64_t(m0 + r) * k + kk];
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

// dx[m, k] = sum_n dy[m, n] W[n, k]: one thread per k, RL_ROWS rows per block row.
template <typename T>
__global__ void __launch_bounds__(256) rows_linear_dx_kernel(const float* __restrict__ dy, const T* __restrict__ w,
                                                             float* __restrict__ dx, int m, int n, int k) {
  const int kk = blockIdx.x * 256 + threadIdx.x;
  const int m0 = blockIdx.y * RL_ROWS;
  if (kk >= k) return;
  float acc[RL_ROWS];
#pragma unroll
  for (int r = 0; r < RL_ROWS; ++r) acc[r] = 0.f;
  for (int col = 0; col < n; ++col) {
    const float wv = rl_load<T>(w + int64_t(col) * k + kk);
#pragma unroll
    for (int r = 0; r < RL_ROWS; ++r) {
      if (m0 + r < m) acc[r] += wv * dy[int64_t(m0 + r) * n + col];
    }
  }
#pragma unroll
  for (int r = 0; r < RL_ROWS; ++r) {
    if (m0 + r < m) dx[int64_t(m0 + r) * k + kk] = acc[r];
  }
}

// dW[n, k] = sum_m dy[m, n] x[m, k] (one thread per element), db[n] = sum_m dy[m, n].
__global__ void __launch_bounds__(256) rows_linear_dw_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                             float* __restrict__ dw, float* __restrict__ db, int m,
                                                             int n, int k) {
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= int64_t(n) * k) return;
  const int col = int(i / k), kk = int(i - int64_t(col) * k);
  float acc = 0.f, accb = 0.f;
  for (int r = 0; r < m; ++r) {
    const float g = dy[int64_t(r) * n + col];
    acc += g * x[int64_t(r) * k + kk];
    accb += g;
  }
  dw[i] = acc;
  if (db && kk == 0) db[col] = accb;
}

}  // namespace

cudaError_t rows_linear_fwd(const float* x, const void* w, const void* bias, float* y, int m, int n, int k,
                            bool bf16_weights, cudaStream_t stream) {
  if (m == 0 || n == 0) return cudaSuccess;
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

cudaError_t rows_linear_bwd(const float* dy, const float* x, const void* w, float* dx, float* dw, float* db, int m,
                            int n, int k, bool bf16_weights, cudaStream_t stream) {
  if (m == 0 || n == 0 || k == 0) return cudaSuccess;
  if (dx) {
    const dim3 grid(unsigned((k + 255) / 256), unsigned((m + RL_ROWS - 1) / RL_ROWS));
    if (bf16_weights) {
      rows_linear_dx_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(dy, static_cast<const __nv_bfloat16*>(w), dx,
                                                                     m, n, k);
    } else {
      rows_linear_dx_kernel<float><<<grid, 256, 0, stream>>>(dy, static_cast<const float*>(w), dx, m, n, k);
    }
  }
  if (dw) {
    const unsigned grid = unsigned((int64_t(n) * k + 255) / 256);
    rows_linear_dw_kernel<<<grid, 256, 0, stream>>>(dy, x, dw, db, m, n, k);
  }
  return cudaGetLastError();
}

}  // namespace agb
