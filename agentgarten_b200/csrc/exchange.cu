// All-to-all between the GPUs of one node over peer memory (the Ulysses exchange of context
// parallelism): rank r sends block d of its buffer to rank d and receives block s from rank s.
//
// Two launches per exchange on every rank, in stream order:
//   push:  copy block d of `send` into slot `rank` of rank d's receive buffer with plain
//          16-byte stores through the peer mapping (block `rank` goes to the local buffer),
//          then the last CTA to finish adds 1 (release, system scope) to every rank's
//          arrival counter;
//   pull:  wait (bounded) until the local arrival counter shows the blocks of all ranks for
//          this exchange, copy the receive buffer into the result tensor, and let the last
//          CTA advance the exchange count.
// The receive buffer has two halves used alternately (parity of the exchange count, which
// lives in device memory, so a captured sequence of exchanges replays): a rank can be at
// most one exchange ahead of a peer, because finishing exchange k + 1 needs that peer's
// blocks of k + 1, which it sends only after its own pull of exchange k.
// Counters are monotonic.  A wait that runs out records kTimeoutPeer in the status word; the
// copy is skipped and the kernels return.
#include "agb.h"
#include "sm100.cuh"

namespace agb {
namespace {

constexpr int NT = 256;

__device__ __forceinline__ void copy16(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                       int64_t vectors) {
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < vectors; i += int64_t(gridDim.x) * NT)
    dst[i] = src[i];
}

__global__ void __launch_bounds__(NT) exchange_push_kernel(const ExchangeArgs a) {
  const int parity = *reinterpret_cast<volatile int*>(a.count) & 1;
  const int64_t vectors = a.bytes_per_rank / 16;
  for (int d = 0; d < a.world; ++d) {
    const int peer = (a.rank + d) % a.world;  // start with the local block, spread the links
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.recv[peer]) + parity * a.half_bytes +
                                          int64_t(a.rank) * a.bytes_per_rank);
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.send) +
                                                      int64_t(peer) * a.bytes_per_rank);
    copy16(dst, src, vectors);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(a.ticket, 1) == int(gridDim.x) - 1) {
      *a.ticket = 0;
      __threadfence();
      for (int d = 0; d < a.world; ++d)
        asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(a.arrive[d]) : "memory");
    }
  }
}

__global__ void __launch_bounds__(NT) exchange_pull_kernel(const ExchangeArgs a) {
  __shared__ int proceed;
  const int count = *reinterpret_cast<volatile int*>(a.count);
  if (threadIdx.x == 0) {
    const int target = static_cast<int>((static_cast<unsigned>(count) + 1u) * static_cast<unsigned>(a.world));
    const int* counter = a.arrive[a.rank];
    int go = 1;
    const uint64_t start = global_timer_ns();
    for (;;) {
      int seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
      if (counter_reached(seen, target)) break;
      if (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) {
        go = 0;  // an earlier wait on this device already ran out: do not spend the limit again
        break;
      }
      if (global_timer_ns() - start > AGB_PEER_WAIT_LIMIT_NS) {
        if (a.status) atomicCAS(a.status, 0, kTimeoutPeer);
        go = 0;
        break;
      }
      __nanosleep(64);
    }
    proceed = go;
  }
  __syncthreads();
  if (proceed) {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.recv[a.rank]) +
                                                      (count & 1) * a.half_bytes);
    copy16(static_cast<uint4*>(a.out), src, a.bytes_per_rank / 16 * a.world);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.ticket, 1) == int(gridDim.x) - 1) {
      *a.ticket = 0;
      // The exchange is counted even when it failed, so that the ranks stay in step.
      *reinterpret_cast<volatile int*>(a.count) = counter_add(count, 1);
      __threadfence();
    }
  }
}

}  // namespace

cudaError_t exchange_all_to_all(const ExchangeArgs& a, int sm_count, cudaStream_t stream) {
  if (a.world < 1 || a.world > 8 || a.rank < 0 || a.rank >= a.world || (a.bytes_per_rank % 16) ||
      a.bytes_per_rank * a.world > a.half_bytes || (a.half_bytes % 16) ||
      (reinterpret_cast<uintptr_t>(a.send) & 15) || (reinterpret_cast<uintptr_t>(a.out) & 15)) {
    set_error_detail("exchange: 1..8 ranks, 16-byte aligned blocks that fit half the receive buffer");
    return cudaErrorInvalidValue;
  }
  if (a.bytes_per_rank == 0) return cudaSuccess;
  const int64_t vectors = a.bytes_per_rank / 16;
  int64_t blocks = (vectors + NT - 1) / NT;
  const int64_t cap = int64_t(sm_count) * 4;
  if (blocks > cap) blocks = cap;
  (void)cudaGetLastError();
  exchange_push_kernel<<<unsigned(blocks), NT, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error_detail("exchange: push launch failed");
    return e;
  }
  exchange_pull_kernel<<<unsigned(blocks), NT, 0, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) set_error_detail("exchange: pull launch failed");
  return e;
}

}  // namespace agb
