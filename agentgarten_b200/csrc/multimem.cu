// Small collectives through the NVSwitch multicast mapping (NVLS): the maximum of a few 32-bit
// values over the GPUs of a node in one launch, no library call.
//
// Every GPU maps the same symmetric buffer twice: `local` (its own memory) and `mc`, a
// multicast address through which one instruction reaches the copy of every GPU.
//   1. each GPU stores its values into its own copy and announces that with one
//      multimem.red on the arrival counter (the switch increments the counter of every GPU);
//   2. once its own counter shows that all have arrived, GPU r reduces the elements
//      i = r, r + world, ... with multimem.ld_reduce.max (the switch combines the copies) and
//      writes each result to every copy with multimem.st;
//   3. a second arrival, then every GPU reads the results from its own copy.
// Each element is reduced exactly once, so all GPUs read identical bits.  The buffer has two
// halves used by alternating calls, and a call makes its first arrival only after finishing the
// reads of the previous one, so a half is never rewritten while a peer still reads it.  The
// call count lives in device memory: the kernel can be replayed from a CUDA graph.  Both waits
// are bounded (status word kTimeoutPeer).
#include <cuda_runtime.h>

#include "agb.h"
#include "sm100.cuh"

namespace agb {
namespace {

constexpr int MM_MAX = 32;  // values per call

__device__ __forceinline__ void mm_arrive(int* counter_mc) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], 1;" ::"l"(counter_mc) : "memory");
}
__device__ __forceinline__ int mm_load_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t mm_reduce_max(const uint32_t* mc) {
  uint32_t v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.max.u32 %0, [%1];" : "=r"(v) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_store(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// Waits until *counter has advanced to `target` (wrapped difference); false when the limit ran out.
__device__ __forceinline__ bool mm_wait(const int* counter, int target, int* status, uint64_t limit_ns) {
  const uint64_t start = global_timer_ns();
  uint32_t spins = 0;
  while (!counter_reached(mm_load_acquire(counter), target)) {
    if ((++spins & 63u) == 0 && global_timer_ns() - start > limit_ns) {
      if (status) atomicCAS(status, 0, kTimeoutPeer);
      return false;
    }
  }
  return true;
}

// buffer layout (uint32): [2 halves][MM_MAX values], then the arrival counter; `state` (local,
// not symmetric): [0] calls made.  One block of MM_MAX threads.
__global__ void __launch_bounds__(MM_MAX) multimem_max_kernel(uint32_t* local, uint32_t* mc, int* state,
                                                              const uint32_t* in, uint32_t* out, int n,
                                                              int world, int rank, int* status,
                                                              uint64_t limit_ns) {
  __shared__ int ok_shared;
  const int call = state[0];
  uint32_t* mine = local + (call & 1) * MM_MAX;
  uint32_t* all = mc + (call & 1) * MM_MAX;
  int* counter = reinterpret_cast<int*>(local + 2 * MM_MAX);
  int* counter_mc = reinterpret_cast<int*>(mc + 2 * MM_MAX);
  const int i = threadIdx.x;
  if (i < n) mine[i] = in[i];
  __threadfence_system();
  __syncthreads();
  if (i == 0) {
    mm_arrive(counter_mc);  // first arrival of this call: every copy holds its owner's values
    ok_shared = mm_wait(counter, counter_add(0, (2 * call + 1) * world), status, limit_ns) ? 1 : 0;
  }
  __syncthreads();
  bool ok = ok_shared != 0;
  if (ok && i < n && i % world == rank) mm_store(all + i, mm_reduce_max(all + i));
  __threadfence_system();
  __syncthreads();
  if (i == 0) {
    if (ok) mm_arrive(counter_mc);  // second arrival: every copy holds the results
    ok_shared = ok && mm_wait(counter, counter_add(0, (2 * call + 2) * world), status, limit_ns) ? 1 : 0;
    state[0] = call + 1;
  }
  __syncthreads();
  ok = ok_shared != 0;
  if (i < n) out[i] = ok ? *reinterpret_cast<volatile uint32_t*>(mine + i) : in[i];
}

// ------------------------------------------------------------------ shared payloads
// All-gather and broadcast through multicast stores.  The symmetric buffer holds an arrival
// counter (first SHARE_HEADER bytes) and two payload halves used by alternating calls.  Each GPU
// stores its part (possibly nothing) at its offset of the current half with multimem.st, so the
// bytes land in every GPU's copy; each CTA then announces its stores with one multimem.red and
// waits (bounded) until the CTAs of all GPUs have done so, and copies the whole payload from its
// own copy into `out`.  Every GPU launches the same grid (it depends on the total size only),
// at most one CTA per SM, so that all CTAs that wait on one another are resident.  A half is
// rewritten two calls later, after the call in between has seen every GPU arrive, i.e. after
// every GPU has finished copying out of it.  `state` (this GPU's memory): [0] calls made,
// [1] arrivals expected before this call; the second kernel advances both.
constexpr int SHARE_HEADER = 256;
constexpr int SHARE_THREADS = 256;

__device__ __forceinline__ void mm_store16(uint4* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

__global__ void __launch_bounds__(SHARE_THREADS) multimem_share_kernel(
    char* local, char* mc, int64_t half_vecs, const int* state, const uint4* __restrict__ src, int64_t vec_mine,
    int64_t vec_offset, uint4* __restrict__ out, int64_t vec_total, int world, int* status, uint64_t limit_ns) {
  __shared__ int ok_shared;
  const int call = state[0];
  const int target = counter_add(state[1], world * int(gridDim.x));
  const int64_t half = int64_t(call & 1) * half_vecs;
  uint4* everywhere = reinterpret_cast<uint4*>(mc + SHARE_HEADER) + half + vec_offset;
  const int64_t stride = int64_t(gridDim.x) * SHARE_THREADS;
  int64_t i = int64_t(blockIdx.x) * SHARE_THREADS + threadIdx.x;
  for (; i + 3 * stride < vec_mine; i += 4 * stride) {  // four loads in flight per thread
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < 4; ++u) mm_store16(everywhere + i + u * stride, v[u]);
  }
  for (; i < vec_mine; i += stride) mm_store16(everywhere + i, src[i]);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    mm_arrive(reinterpret_cast<int*>(mc));
    ok_shared = mm_wait(reinterpret_cast<const int*>(local), target, status, limit_ns) ? 1 : 0;
  }
  __syncthreads();
  if (!ok_shared) return;
  const uint4* mine = reinterpret_cast<const uint4*>(local + SHARE_HEADER) + half;
  i = int64_t(blockIdx.x) * SHARE_THREADS + threadIdx.x;
  for (; i + 3 * stride < vec_total; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcg(mine + i + u * stride);
#pragma unroll
    for (int u = 0; u < 4; ++u) out[i + u * stride] = v[u];
  }
  for (; i < vec_total; i += stride) out[i] = __ldcg(mine + i);
}

__global__ void multimem_share_done_kernel(int* state, int arrivals) {
  state[0] += 1;
  state[1] = counter_add(state[1], arrivals);
}

}  // namespace

cudaError_t multimem_max(void* local, void* multicast, int* state, const uint32_t* in, uint32_t* out, int n,
                         int world, int rank, int* status, uint64_t limit_ns, cudaStream_t stream) {
  if (n < 1 || n > MM_MAX || world < 1 || rank < 0 || rank >= world || !local || !multicast) {
    return cudaErrorInvalidValue;
  }
  multimem_max_kernel<<<1, MM_MAX, 0, stream>>>(static_cast<uint32_t*>(local), static_cast<uint32_t*>(multicast),
                                                state, in, out, n, world, rank, status, limit_ns);
  return cudaGetLastError();
}

int64_t multimem_share_capacity(int64_t buffer_bytes) {
  const int64_t half = (buffer_bytes - SHARE_HEADER) / 2;
  return half < 16 ? 0 : half / 16 * 16;
}

cudaError_t multimem_share(void* local, void* multicast, int64_t buffer_bytes, int* state, const void* src,
                           int64_t bytes_mine, int64_t offset, void* out, int64_t bytes_total, int world,
                           int sm_count, int* status, uint64_t limit_ns, cudaStream_t stream) {
  const int64_t capacity = multimem_share_capacity(buffer_bytes);
  if (!local || !multicast || world < 1 || bytes_total < 16 || bytes_total > capacity || bytes_mine < 0 ||
      offset < 0 || offset + bytes_mine > bytes_total || (bytes_mine | offset | bytes_total) % 16 != 0 ||
      (bytes_mine > 0 && (!src || reinterpret_cast<uintptr_t>(src) % 16 != 0)) ||
      reinterpret_cast<uintptr_t>(out) % 16 != 0 || sm_count < 1) {
    return cudaErrorInvalidValue;
  }
  const int64_t vec_total = bytes_total / 16;
  const int64_t wanted = (vec_total + SHARE_THREADS * 8 - 1) / (SHARE_THREADS * 8);
  const int grid = int(wanted < sm_count ? wanted : sm_count);
  multimem_share_kernel<<<grid, SHARE_THREADS, 0, stream>>>(
      static_cast<char*>(local), static_cast<char*>(multicast), capacity / 16, state,
      static_cast<const uint4*>(src), bytes_mine / 16, offset / 16, static_cast<uint4*>(out), vec_total, world,
      status, limit_ns);
  multimem_share_done_kernel<<<1, 1, 0, stream>>>(state, world * grid);
  return cudaGetLastError();
}

}  // namespace agb
