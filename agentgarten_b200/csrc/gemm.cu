// bf16 GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
// Persistent kernel, one CTA per SM, 128x256 output tiles, K blocks of 64:
//   warp 4 (one lane)  TMA producer: operand tiles -> 4-stage shared-memory ring
//   warp 5 (one lane)  MMA issuer:   tcgen05.mma from shared memory into TMEM
//   warps 0-3          epilogue:     TMEM -> registers -> bias/residual/accumulate -> global
// Two 256-column TMEM accumulators let the epilogue of tile i overlap the main loop of
// tile i+1.  Operands may be K-major or MN-major in memory (chosen per call), so forward,
// input-gradient and weight-gradient products run without any transposed copy.
//
// The value of an output row depends only on that row of A (fixed tile shape, fixed K
// order, no split-K), so results are invariant to how many rows are multiplied together.
#include <cstdlib>

#include "agb.h"
#include "sm100.cuh"
#include "tensormap.h"

namespace agb {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ATOM_BYTES = 64 * BK * 2;  // one 64-wide MN-major atom column: BK rows x 128 B
constexpr int GROUP_M = 16;              // tile rasterisation: 16 M-tiles per N sweep
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
// A pushing (tensor-parallel) launch adds 4 KiB per epilogue warp: 32 rows x 64 columns of bf16
// are transposed there so that rows leave for the peer as whole 128-byte lines.
constexpr int PUSH_STAGE_BYTES = 32 * 128;
constexpr int SMEM_BYTES_PUSH = SMEM_BYTES + 4 * PUSH_STAGE_BYTES;

struct Params {
  __nv_bfloat16* out_bf16;
  float* out_f32;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int64_t ldo, ldr;
  int m, n, k;
  int tiles_m, tiles_n;
  int accumulate;
  int* status;
  TpLink tp;   // tp.world == 0: not coupled
};

// Bounded wait until a monotonic counter written by peers reaches `target`.
__device__ __forceinline__ bool wait_counter(const int* counter, int target, const WaitGuard& g) {
  const uint64_t start = global_timer_ns();
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (counter_reached(seen, target)) return true;
    if (*g.abort_flag) return false;
    // A wait that already ran out on this device (this launch or an earlier one) means the step
    // is lost: give up at once instead of spending the limit again in every CTA and launch.
    if (g.status && *reinterpret_cast<volatile int*>(g.status) != 0) {
      *g.abort_flag = 1;
      return false;
    }
    if (global_timer_ns() - start > AGB_PEER_WAIT_LIMIT_NS) {
      *g.abort_flag = 1;
      if (g.status) atomicCAS(g.status, 0, kTimeoutPeer);
      return false;
    }
    __nanosleep(64);
  }
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int local = tile - group * per_group;
  tm = first_m + local % rows;
  tn = local / rows;
}

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                     // [STAGES] producer -> MMA
  uint64_t* empty = bars + STAGES;           // [STAGES] MMA -> producer
  uint64_t* acc_full = bars + 2 * STAGES;    // [2] MMA -> epilogue
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.k + BK - 1) / BK;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0;  // bit s: stage s was armed at least once
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        if (p.tp.wait_a) {
          // Rows of this A tile are pushed into local memory by their owner; the counter
          // counts rows.  The copy below reads them through the async proxy.
          const int target =
              counter_add(reinterpret_cast<volatile int*>(p.tp.a_seen)[tm], min(BM, p.m - m0));
          if (!wait_counter(p.tp.a_ready + tm, target, guard)) {
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, guard, kTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          armed |= 1u << stage;
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d(sa, &tm_a, &full[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * ATOM_BYTES, &tm_a, &full[stage], m0 + 64 * j, k0);
          }
          if (B_MN == 0) {
            tma_load_2d(sb, &tm_b, &full[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * ATOM_BYTES, &tm_b, &full[stage], n0 + 64 * j, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok || *abort_flag) {
        // Abort path: let this thread's copies land before the CTA's shared memory dies.
        // The parity of the last armed phase of stage s is `phase` for s < stage, else phase^1.
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          const uint32_t last = (s < stage) ? phase : (phase ^ 1);
          const uint64_t start = global_timer_ns();
          while (!mbar_try_wait(&full[s], last)) {
            if (global_timer_ns() - start > 50000000ull) break;  // 50 ms
          }
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------------- MMA issuer
    {  // the whole warp runs the loop (addresses stay warp-uniform); one elected lane issues
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait_w(&acc_empty[acc], acc_phase ^ 1, guard, kTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_w(&full[stage], phase, guard, kTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc(sa + kk * 2048, ATOM_BYTES, 1024)
                                     : make_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + kk * 2048, ATOM_BYTES, 1024)
                                     : make_smem_desc(sb + kk * 32, 16, 1024);
            tc_mma_ss_w(d_tmem, da, db, idesc, (kb | kk) != 0);
          }
          tc_commit_w(&empty[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit_w(&acc_full[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------------- epilogue
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, guard, kTimeoutEpilogue)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = tm * BM + warp * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t t_row = tmem_base + (uint32_t(warp * 32) << 16) + acc * BN;
      // Where this thread's output row lives: the local output, or (tensor parallel, push)
      // the partial-sum slot of the tile's owner, reached through the peer mapping.
      __nv_bfloat16* out_row = p.out_bf16 ? p.out_bf16 + int64_t(row) * p.ldo : nullptr;
      const int owner = p.tp.push ? tm % p.tp.world : 0;
      if (p.tp.push) {
        const int64_t slot_row =
            (int64_t(p.tp.rank) * p.tp.tiles_owned + tm / p.tp.world) * BM + warp * 32 + lane;
        out_row = static_cast<__nv_bfloat16*>(p.tp.slot[owner]) + slot_row * p.ldo;
      }
      if (p.tp.push) {
        // Tensor-parallel push: rows go to the owner's slot through NVLink.  A lane holds one
        // row in TMEM order; 64 columns at a time are exchanged through shared memory (16-byte
        // chunks, XOR-swizzled by row so neither side has bank conflicts) and leave as 128
        // contiguous bytes per row, 4 rows per store instruction.
        uint8_t* stage = smem + STAGES * STAGE_BYTES + 256 + warp * PUSH_STAGE_BYTES;
        __nv_bfloat16* tile_base = static_cast<__nv_bfloat16*>(p.tp.slot[owner]) +
            ((int64_t(p.tp.rank) * p.tp.tiles_owned + tm / p.tp.world) * BM + warp * 32) * p.ldo;
        const int rows_left = p.m - (tm * BM + warp * 32);  // valid rows of this warp's 32
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = tn * BN + c * 32;
          if (col0 >= p.n) break;  // uniform across the CTA
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = (c & 1) * 4 + g;
            *reinterpret_cast<uint4*>(stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = make_uint4(
                pack_bf16(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1])),
                pack_bf16(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3])),
                pack_bf16(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5])),
                pack_bf16(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7])));
          }
          const bool last = (c & 1) || (col0 + 32 >= p.n);
          if (last) {
            __syncwarp();
            const int first_col = tn * BN + (c & ~1) * 32;  // of the 64-column group
            const int chunk = lane & 7;
            const int col = first_col + chunk * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = 4 * i + (lane >> 3);
              const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((chunk ^ (rr & 7)) << 4));
              const bool filled = (c & 1) || chunk < 4;  // an odd group of 32 columns fills half
              if (rr < rows_left && col < p.n && filled)
                *reinterpret_cast<uint4*>(tile_base + int64_t(rr) * p.ldo + col) = v;
            }
            __syncwarp();
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.n) break;  // uniform across the CTA
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {  // groups of 8 columns (16 bytes of bf16)
            const int col = col0 + g * 8;
            if (col >= p.n) break;  // N is a multiple of 8
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
            if (p.bias) {
              const uint4 b = *reinterpret_cast<const uint4*>(p.bias + col);
              const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                v[2 * i] += bf16_lo(bw[i]);
                v[2 * i + 1] += bf16_hi(bw[i]);
              }
            }
            if (p.residual) {
              const uint4 b =
                  *reinterpret_cast<const uint4*>(p.residual + int64_t(row) * p.ldr + col);
              const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                v[2 * i] += bf16_lo(bw[i]);
                v[2 * i + 1] += bf16_hi(bw[i]);
              }
            }
            if (p.out_f32) {
              float4* dst = reinterpret_cast<float4*>(p.out_f32 + int64_t(row) * p.ldo + col);
              if (p.accumulate) {
                const float4 o0 = dst[0], o1 = dst[1];
                v[0] += o0.x; v[1] += o0.y; v[2] += o0.z; v[3] += o0.w;
                v[4] += o1.x; v[5] += o1.y; v[6] += o1.z; v[7] += o1.w;
              }
              dst[0] = make_float4(v[0], v[1], v[2], v[3]);
              dst[1] = make_float4(v[4], v[5], v[6], v[7]);
            } else {
              uint4* dst = reinterpret_cast<uint4*>(out_row + col);
              if (p.accumulate) {
                const uint4 o = *dst;
                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  v[2 * i] += bf16_lo(ow[i]);
                  v[2 * i + 1] += bf16_hi(ow[i]);
                }
              }
              *dst = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]),
                                pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            }
          }
        }
      }
      }
      tc_fence_before_sync();
      if (p.tp.push) __threadfence_system();  // this lane's stores before the warp's arrival
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty[acc]);
        if (p.tp.push) {
          int* counter = p.tp.arrive[owner] + tm / p.tp.world;
          asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(counter) : "memory");
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (p.tp.wait_a && p.tp.ticket && threadIdx.x == 0) {
    // The last CTA to finish closes this use of the A buffer (not when more GEMMs of the
    // same use follow: those pass no ticket).
    __threadfence();
    if (atomicAdd(p.tp.ticket, 1) == int(gridDim.x) - 1) {
      *p.tp.ticket = 0;
      volatile int* seen = reinterpret_cast<volatile int*>(p.tp.a_seen);
      for (int t = 0; t < p.tiles_m; ++t) seen[t] = counter_add(seen[t], min(BM, p.m - t * BM));
      __threadfence();
    }
  }
}

}  // namespace

// ------------------------------------------------------------------------------- host
namespace {

template <int A_MN, int B_MN>
cudaError_t launch(const GemmArgs& g, const CUtensorMap& ta, const CUtensorMap& tb,
                   const Params& p, int grid, cudaStream_t stream) {
  auto kernel = gemm_kernel<A_MN, B_MN>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_PUSH);
    if (e != cudaSuccess) {
      set_error_detail("gemm: cudaFuncSetAttribute(max dynamic shared memory) failed");
      return e;
    }
    configured = true;
  }
  (void)cudaGetLastError();  // do not report an error left behind by an earlier call
  kernel<<<grid, NUM_THREADS, p.tp.push ? SMEM_BYTES_PUSH : SMEM_BYTES, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_error_detail("gemm: kernel launch failed");
  return e;
}

}  // namespace

// Products with enough 256 x 256 tiles run on CTA pairs (csrc/gemm2.cu); both kernels add the
// K slices in the same order, so a result does not depend on which of the two a call got
// (tests/test_gpu_kernels.py compares them bit for bit).  AGB200_GEMM_PAIRS=0 keeps every
// product on single-CTA tiles; the variable is read at each call so that a test can switch it.
static bool use_cta_pairs() {
  const char* choice = getenv("AGB200_GEMM_PAIRS");
  return choice == nullptr || choice[0] != '0';
}

cudaError_t gemm_bf16(const GemmArgs& g, int sm_count, cudaStream_t stream) {
  if (g.m <= 0 || g.n <= 0 || g.k <= 0) return cudaSuccess;
  if ((g.n % 8) || (g.lda % 8) || (g.ldb % 8) || (g.ldo % 4) ||
      (reinterpret_cast<uintptr_t>(g.a) & 15) || (reinterpret_cast<uintptr_t>(g.b) & 15) ||
      (reinterpret_cast<uintptr_t>(g.out) & 15)) {
    set_error_detail("gemm: sizes/strides must be multiples of 8 elements and pointers 16-byte aligned");
    return cudaErrorInvalidValue;
  }

  // Two SMs per 256 x 256 tile once there are enough tiles to give every pair of SMs one;
  // smaller products keep 128-row tiles, which spread over more SMs.
  if (!g.tp && use_cta_pairs() &&
      ((g.m + 255) / 256) * ((g.n + 255) / 256) >= int64_t(sm_count) / 2) {
    return gemm_bf16_pairs(g, sm_count, stream);
  }

  CUtensorMap ta, tb;
  {
    // K-major: dims (K, M), box (64, 128).  MN-major: dims (M, K), box (64, 64).
    const uint64_t dims[2] = {uint64_t(g.a_mn_major ? g.m : g.k),
                              uint64_t(g.a_mn_major ? g.k : g.m)};
    const uint64_t strides[1] = {uint64_t(g.lda) * 2};
    const uint32_t box[2] = {64, uint32_t(g.a_mn_major ? BK : BM)};
    if (!make_tensor_map_bf16(&ta, g.a, 2, dims, strides, box)) {
      return cudaErrorInvalidValue;
    }
  }
  {
    const uint64_t dims[2] = {uint64_t(g.b_mn_major ? g.n : g.k),
                              uint64_t(g.b_mn_major ? g.k : g.n)};
    const uint64_t strides[1] = {uint64_t(g.ldb) * 2};
    const uint32_t box[2] = {64, uint32_t(g.b_mn_major ? BK : BN)};
    if (!make_tensor_map_bf16(&tb, g.b, 2, dims, strides, box)) {
      return cudaErrorInvalidValue;
    }
  }
  Params p;
  p.out_bf16 = g.out_fp32 ? nullptr : static_cast<__nv_bfloat16*>(g.out);
  p.out_f32 = g.out_fp32 ? static_cast<float*>(g.out) : nullptr;
  p.bias = static_cast<const __nv_bfloat16*>(g.bias);
  p.residual = static_cast<const __nv_bfloat16*>(g.residual);
  p.ldo = g.ldo;
  p.ldr = g.ldr;
  p.m = g.m;
  p.n = g.n;
  p.k = g.k;
  p.tiles_m = (g.m + BM - 1) / BM;
  p.tiles_n = (g.n + BN - 1) / BN;
  p.accumulate = g.accumulate;
  p.status = g.status;
  p.tp = TpLink{};
  if (g.tp) {
    if (g.a_mn_major || g.b_mn_major || g.out_fp32 || g.accumulate || g.tp->world < 1 ||
        g.tp->world > 8 || (g.tp->push && (g.residual || g.bias))) {
      set_error_detail("gemm: a tensor-parallel GEMM is K-major, bf16, without accumulate; a pushing one has no bias/residual");
      return cudaErrorInvalidValue;
    }
    p.tp = *g.tp;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  if (g.a_mn_major == 0 && g.b_mn_major == 0) return launch<0, 0>(g, ta, tb, p, grid, stream);
  if (g.a_mn_major == 0 && g.b_mn_major == 1) return launch<0, 1>(g, ta, tb, p, grid, stream);
  if (g.a_mn_major == 1 && g.b_mn_major == 0) return launch<1, 0>(g, ta, tb, p, grid, stream);
  return launch<1, 1>(g, ta, tb, p, grid, stream);
}

}  // namespace agb
