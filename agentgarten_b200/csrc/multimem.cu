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

}  // namespace agb
