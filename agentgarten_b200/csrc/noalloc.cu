// Allocation-free RMSNorm backward: see agb_noalloc.h for who needs this and why.
#include "agb_noalloc.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

#include "agb.h"

namespace {

// Partial weight-gradient sums, one row of `width` floats per block of 32 input rows.
// Device code names this array directly; host code must not pass its name to a kernel
// (on the host the name is only a stand-in), it asks the runtime for the device address.
static __device__ __align__(256) float g_scratch[AGB_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
// Written by whichever host thread calls first on a device (every writer stores the same
// address), read by all: atomic so that concurrent first calls are well defined.
std::atomic<float*> g_scratch_address[kMaxDevices] = {};
thread_local char g_error[256] = "";

int fail(int code, const char* format, long long a = 0, long long b = 0, long long c = 0) {
  snprintf(g_error, sizeof(g_error), format, a, b, c);
  return code;
}

// dw[c] = sum over partial rows, in row order (deterministic).
__global__ void __launch_bounds__(256) column_sum_kernel(float* __restrict__ dw, int parts,
                                                         int width) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  float total = 0.f;
  for (int p = 0; p < parts; ++p) total += g_scratch[int64_t(p) * width + c];
  dw[c] = total;
}

}  // namespace

extern "C" const char* agb_noalloc_last_error(void) { return g_error; }

extern "C" int agb_rms_norm_bwd_noalloc(const void* grad, const void* x, const void* w,
                                        const float* rstd, void* dx, float* dw, int64_t rows,
                                        int width, void* stream) {
  g_error[0] = 0;
  if (!grad || !x || !w || !rstd || !dx || !dw) return fail(-1, "null pointer argument");
  if (rows < 0) return fail(-2, "rows %lld must not be negative", (long long)rows);
  if (width <= 0 || (width % 8) || width > 8192)
    return fail(-2, "width %lld must be a positive multiple of 8 and at most 8192", width);
  const int parts = agb::rms_norm_bwd_partials(rows);
  if (int64_t(parts) * width > AGB_NOALLOC_SCRATCH_FLOATS)
    return fail(-3,
                "request needs %lld scratch floats (ceil(rows/32) * width) but the built-in "
                "scratch holds %lld; split the rows over several calls",
                (long long)parts * width, (long long)AGB_NOALLOC_SCRATCH_FLOATS);
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail(-4, "cudaGetDevice failed (%lld)", (long long)e);
  if (device < 0 || device >= kMaxDevices) return fail(-4, "device index %lld unsupported", device);
  float* address = g_scratch_address[device].load(std::memory_order_acquire);
  if (!address) {
    // Set-up, once per device, with that device current.
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_scratch);
    if (e != cudaSuccess || !address)
      return fail(-5, "cudaGetSymbolAddress failed (%lld)", (long long)e);
    g_scratch_address[device].store(address, std::memory_order_release);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    e = cudaMemsetAsync(dw, 0, sizeof(float) * width, s);
    return e == cudaSuccess ? 0 : fail(-6, "cudaMemsetAsync failed (%lld)", (long long)e);
  }
  e = agb::rms_norm_bwd(grad, x, w, rstd, dx, address, rows, width, s);
  if (e != cudaSuccess) return fail(-6, "rms_norm_bwd launch failed (%lld)", (long long)e);
  column_sum_kernel<<<(width + 255) / 256, 256, 0, s>>>(dw, parts, width);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : fail(-6, "column_sum launch failed (%lld)", (long long)e);
}
