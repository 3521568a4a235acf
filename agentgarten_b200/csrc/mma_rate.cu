// Diagnostic: cycles per tcgen05.mma (M = 128, K = 16, bf16) issued back to back by one warp.
//
// The attention kernels choose their tile shapes from this figure: on B200 an instruction of up
// to 128 columns takes about 90 cycles whatever its width (the tensor pipe would need 32 for
// N = 64 and 64 for N = 128), one of 256 columns takes 128, which is the pipe's full rate.  A
// kernel built from N <= 128 products is therefore bound by the number of instructions it
// issues, not by their arithmetic.
#include <cuda_runtime.h>

#include "agb.h"
#include "sm100.cuh"

namespace agb {
namespace {

constexpr int RATE_SMEM = 100 * 1024;

// The whole warp runs the loop (so that addresses stay warp-uniform) and one elected lane issues.
__device__ __forceinline__ void rate_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, 1;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void rate_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, 1;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc)
      : "memory");
}

// columns: 64, 128 or 256; a_from_tmem: A operand read from TMEM instead of shared memory.
// out[0] = cycles from the first issue to the completion of the last product.
__global__ void __launch_bounds__(128, 1)
mma_rate_kernel(int columns, int a_from_tmem, int iterations, long long* out, int* status) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&slot, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = slot;
  const WaitGuard guard{&abort_flag, status};
  if (warp == 1) {
    // A: 128 rows x 128 bytes per 64-element K block (16 KiB each); B: up to 256 rows (32 KiB each)
    const uint64_t a0 = make_smem_desc(smem_u32(smem), 16, 1024);
    const uint64_t b0 = make_smem_desc(smem_u32(smem + 32768), 16, 1024);
    const uint32_t idesc = make_idesc_bf16(128, columns, 0, 0);
    const long long t0 = clock64();
    for (int it = 0; it < iterations; ++it) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
        if (a_from_tmem) rate_mma_ts(tmem + 256, tmem + kk * 8, b0 + off, idesc);
        else rate_mma_ss(tmem + 256, a0 + off, b0 + off, idesc);
      }
    }
    if (lane == 0) {
      tc_commit(&bar);
      const bool ok = mbar_wait(&bar, 0, guard, kTimeoutMma);
      if (blockIdx.x == 0) out[0] = ok ? clock64() - t0 : -1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

cudaError_t mma_issue_rate(int columns, bool a_from_tmem, int iterations, int sm_count, long long* cycles,
                           int* status, cudaStream_t stream) {
  if ((columns != 64 && columns != 128 && columns != 256) || iterations < 1) return cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RATE_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  mma_rate_kernel<<<sm_count, 128, RATE_SMEM, stream>>>(columns, a_from_tmem ? 1 : 0, iterations, cycles, status);
  return cudaGetLastError();
}

}  // namespace agb
