// Owner side of the tensor-parallel residual stream (serving).
//
// A row-parallel GEMM on every rank pushes its partial output tiles into the slot of the
// rank that owns the rows (see TpLink in agb.h).  This kernel is the other half of that
// reduce-scatter and the first half of the following all-gather, in one pass over the row:
// wait for the partial sums, add them to the residual, apply RMSNorm, and store the
// normalised row straight into every rank's input buffer of the next GEMM, whose TMA
// producer waits for the rows tile by tile.  All cross-GPU traffic is plain peer stores and
// system-scope counters.
#include "agb.h"
#include "sm100.cuh"

namespace agb {
namespace {

constexpr int NT = 256;
// Rows per CTA.  Four rows (two warps each) share one wait, one fence and one signal: best when
// a rank owns many rows.  With few rows (many ranks) one row per CTA, walked by all eight
// warps, has the shorter critical path.
constexpr int MANY_ROWS = 4;
constexpr int MAX_WIDTH = 8192;

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = bf16_lo(w[i]);
    f[2 * i + 1] = bf16_hi(w[i]);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                    pack_bf16(f[6], f[7]));
}

// ROWS rows per CTA, NT / ROWS threads per row, CHUNKS 16-byte vectors per thread and row.
template <int ROWS, int CHUNKS>
__global__ void __launch_bounds__(NT) tp_reduce_norm_kernel(const TpReduceArgs a) {
  constexpr int ROW_THREADS = NT / ROWS;
  constexpr int ROW_WARPS = ROW_THREADS / 32;
  __shared__ float scratch[NT / 32];
  __shared__ int proceed;
  // ROWS consecutive rows of one owned tile (128 is a multiple of ROWS).
  const int sub = threadIdx.x / ROW_THREADS;      // row of this thread inside the CTA's group
  const int lane = threadIdx.x % ROW_THREADS;
  const int first_local = blockIdx.x * ROWS;      // row inside this rank's owned tiles
  const int local_tile = first_local / 128;
  const int tile = local_tile * a.world + a.rank;  // global row tile
  const int64_t first_row = int64_t(tile) * 128 + first_local % 128;
  const int live_rows = int(min(int64_t(ROWS), max(int64_t(0), a.m - first_row)));
  const int local_row = first_local + sub;
  const int64_t row = first_row + sub;
  const bool live = sub < live_rows;

  if (threadIdx.x == 0) {
    int go = 1;
    if (live_rows > 0) {
      // Partial sums of this tile for the current use; or, when seeding a new step, the end
      // of every rank's previous step.
      const int* counter = a.seed ? a.done : a.arrive + local_tile;
      const int target = a.seed
          ? static_cast<int>(static_cast<unsigned>(a.world) *
                             static_cast<unsigned>(*reinterpret_cast<volatile int*>(a.done_uses)))
          : counter_add(reinterpret_cast<volatile int*>(a.arrive_seen)[local_tile],
                        a.world * a.arrivals_per_source);
      const uint64_t start = global_timer_ns();
      for (;;) {
        int seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
        if (counter_reached(seen, target)) break;
        // A wait that already ran out on this device (this launch or an earlier one) means the
        // step is lost: give up at once instead of spending the limit again in every CTA.
        if (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) {
          go = 0;
          break;
        }
        if (global_timer_ns() - start > AGB_PEER_WAIT_LIMIT_NS) {
          if (a.status) atomicCAS(a.status, 0, kTimeoutPeer);
          go = 0;
          break;
        }
        __nanosleep(64);
      }
    }
    proceed = go;
  }
  __syncthreads();

  if (live_rows > 0 && proceed) {  // uniform across the CTA
    const __nv_bfloat16* slot = static_cast<const __nv_bfloat16*>(a.slot);
    __nv_bfloat16* hidden = static_cast<__nv_bfloat16*>(a.hidden_own) + int64_t(local_row) * a.width;
    const __nv_bfloat16* residual =
        a.seed ? static_cast<const __nv_bfloat16*>(a.seed) + row * a.width : hidden;
    const int64_t slot_stride = int64_t(a.tiles_owned) * 128 * a.width;  // between source ranks
    uint4 kept[CHUNKS];
    float sumsq = 0.f;
    if (live) {
#pragma unroll
      for (int k = 0; k < CHUNKS; ++k) {
        const int c = (k * ROW_THREADS + lane) * 8;
        if (c < a.width) {
          float v[8];
          unpack8(*reinterpret_cast<const uint4*>(residual + c), v);
          if (!a.seed) {
            float total[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int src = 0; src < a.world; ++src) {  // fixed order: reproducible sums
              float part[8];
              unpack8(*reinterpret_cast<const uint4*>(slot + src * slot_stride +
                                                      int64_t(local_row) * a.width + c), part);
#pragma unroll
              for (int i = 0; i < 8; ++i) total[i] += part[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = round_bf16(v[i] + total[i]);
          }
          kept[k] = pack8(v);
          *reinterpret_cast<uint4*>(hidden + c) = kept[k];
#pragma unroll
          for (int i = 0; i < 8; ++i) sumsq += v[i] * v[i];
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = sumsq;
    __syncthreads();
    float total = 0.f;  // over the warps of this row
#pragma unroll
    for (int w = 0; w < ROW_WARPS; ++w) total += scratch[ROW_WARPS * sub + w];
    if (live) {
      const float rstd = rsqrtf(total / float(a.width) + a.eps);
      const __nv_bfloat16* weight = static_cast<const __nv_bfloat16*>(a.weight);
#pragma unroll
      for (int k = 0; k < CHUNKS; ++k) {
        const int c = (k * ROW_THREADS + lane) * 8;
        if (c < a.width) {
          float v[8], g[8];
          unpack8(kept[k], v);
          unpack8(*reinterpret_cast<const uint4*>(weight + c), g);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = g[i] * round_bf16(v[i] * rstd);
          const uint4 packed = pack8(v);
          for (int peer = 0; peer < a.world; ++peer)
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.xbuf[peer]) + row * a.width + c) = packed;
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < a.world) {
      // the consumer counts rows: one addition of this CTA's rows per peer
      int* counter = a.ready[threadIdx.x] + tile;
      asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(counter), "r"(live_rows) : "memory");
    }
  }

  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.ticket, 1) == int(gridDim.x) - 1) {
      *a.ticket = 0;
      if (a.seed) {
        volatile int* steps = reinterpret_cast<volatile int*>(a.done_uses);
        *steps = counter_add(*steps, 1);
      } else {
        volatile int* seen = reinterpret_cast<volatile int*>(a.arrive_seen);
        for (int t = 0; t < a.tiles_owned; ++t)
          if ((int64_t(t) * a.world + a.rank) * 128 < a.m)
            seen[t] = counter_add(seen[t], a.world * a.arrivals_per_source);
      }
      __threadfence();
    }
  }
}

struct DonePeers {
  int* counter[8];
};
__global__ void tp_signal_done_kernel(const DonePeers peers, int world) {
  if (int(threadIdx.x) < world) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(peers.counter[threadIdx.x]) : "memory");
  }
}

}  // namespace

cudaError_t tp_reduce_norm(const TpReduceArgs& a, cudaStream_t stream) {
  if (a.world < 1 || a.world > 8 || a.width % 8 || a.width > MAX_WIDTH || a.m <= 0 ||
      (a.rows_per_cta != 0 && a.rows_per_cta != 1 && a.rows_per_cta != MANY_ROWS)) {
    set_error_detail("tp_reduce_norm: world 1..8, width a multiple of 8 up to 8192, rows per CTA 0 (auto), 1 or 4");
    return cudaErrorInvalidValue;
  }
  const int rows = a.tiles_owned * 128;
  if (rows == 0) return cudaSuccess;
  (void)cudaGetLastError();
  // auto: four rows per CTA once that still gives every SM two CTAs
  const int per_cta = a.rows_per_cta ? a.rows_per_cta : (rows / MANY_ROWS >= 2 * 148 ? MANY_ROWS : 1);
  const bool narrow = a.width <= MAX_WIDTH / 2;
  if (per_cta == MANY_ROWS) {
    if (narrow)
      tp_reduce_norm_kernel<MANY_ROWS, 8><<<rows / MANY_ROWS, NT, 0, stream>>>(a);
    else
      tp_reduce_norm_kernel<MANY_ROWS, 16><<<rows / MANY_ROWS, NT, 0, stream>>>(a);
  } else {
    if (narrow)
      tp_reduce_norm_kernel<1, 2><<<rows, NT, 0, stream>>>(a);
    else
      tp_reduce_norm_kernel<1, 4><<<rows, NT, 0, stream>>>(a);
  }
  return cudaGetLastError();
}

cudaError_t tp_signal_done(int* const done[8], int world, cudaStream_t stream) {
  if (world < 1 || world > 8) return cudaErrorInvalidValue;
  DonePeers peers{};
  for (int i = 0; i < world; ++i) peers.counter[i] = done[i];
  (void)cudaGetLastError();
  tp_signal_done_kernel<<<1, 32, 0, stream>>>(peers, world);
  return cudaGetLastError();
}

}  // namespace agb
