// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 with 256x256 output tiles.
//
// Two CTAs of a cluster (two neighbouring SMs) work on one 256x256 tile.  CTA r of the pair
// loads rows [128 r, 128 r + 128) of the A tile and rows [128 r, 128 r + 128) of the B tile
// into its own shared memory (plain TMA tile loads, no multicast) and owns rows
// [128 r, 128 r + 128) of the accumulator in its own TMEM.  One thread of the leader CTA
// (rank 0) issues the MMAs for both: the tensor cores of the two SMs read A from their own
// CTA and B from both, so every byte of B is fetched from shared memory once per 256 output
// rows instead of once per 128, which lifts the shared-memory bound of the single-CTA form.
//
// Synchronisation (all waits bounded, as everywhere in this library):
//   full[s]   in the leader only: one arrival (the leader's expect_tx for the 64 KiB of both
//             CTAs) plus the transaction bytes of both CTAs' TMA loads (the follower's loads
//             name the leader's barrier through its cluster address);
//   empty[s]  in both CTAs: tcgen05.commit with cluster multicast from the leader frees the
//             stage for both producers;
//   acc_full  in both CTAs (multicast commit), acc_empty in the leader (eight arrivals: four
//             epilogue warps of each CTA, the follower's through the cluster address).
// The pair enters a cluster barrier after initialising its barriers and before releasing
// TMEM, so neither CTA touches the other's shared memory or barriers outside that window.
#include "agb.h"
#include "sm100.cuh"
#include "tensormap.h"

namespace agb {
namespace {

constexpr int BM = 128;          // rows of A per CTA (256 per pair)
constexpr int BN_HALF = 128;     // rows of B per CTA (256 per pair)
constexpr int BN = 256;          // accumulator columns
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = BN_HALF * BK * 2;   // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ATOM_BYTES = 64 * BK * 2;
constexpr int GROUP_M = 8;       // 256-row tiles per N sweep
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

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
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Cluster address of `local_smem_addr` in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// TMA tile load whose completion is counted on a barrier that may live in the pair's other CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr),
        "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* result_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(result_in_smem)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the pair.  Called by every lane of one warp of the
// leader CTA; one elected lane issues (a single lane inside a divergent branch pays for moving
// each operand into uniform registers: 166 instead of 128 cycles per 256-column product).
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs once every MMA issued so far
// has completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint16_t both = 0x3;
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}"
      ::"r"(smem_u32(bar)), "h"(both)
      : "memory");
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
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
             const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                        // [STAGES] (used in the leader)
  uint64_t* empty = bars + STAGES;              // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;       // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] (used in the leader)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_rank();   // 0 = leader
  const bool leader = cta == 0;
  const WaitGuard guard{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);  // four epilogue warps in each CTA of the pair
    }
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before either signals the other
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.k + BK - 1) / BK;
  const int pair = int(blockIdx.x >> 1);
  const int pairs = int(gridDim.x >> 1);

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * 2 * BM + int(cta) * BM;
        const int n0 = tn * BN + int(cta) * BN_HALF;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, guard, kTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d_pair(sa, &tm_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d_pair(sa + j * ATOM_BYTES, &tm_a, bar, m0 + 64 * j, k0);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(sb, &tm_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN_HALF / 64; ++j)
              tma_load_2d_pair(sb + j * ATOM_BYTES, &tm_b, bar, n0 + 64 * j, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok || *abort_flag) {
        // give copies in flight time to land before shared memory is released
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) {}
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------------- MMA issuer
    if (leader) {  // the whole warp runs the loop; one elected lane issues
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++local) {
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
            tc_mma_pair(d_tmem, da, db, idesc, (kb | kk) != 0);
          }
          tc_commit_pair(&empty[stage]);  // frees the stage in both CTAs
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit_pair(&acc_full[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------------- epilogue
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++local) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, guard, kTimeoutEpilogue)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = tm * 2 * BM + int(cta) * BM + warp * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t t_row = tmem_base + (uint32_t(warp * 32) << 16) + acc * BN;
      __nv_bfloat16* out_row = p.out_bf16 ? p.out_bf16 + int64_t(row) * p.ldo : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.n) break;  // uniform across the pair
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
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();  // the peer has stopped reading this CTA's shared memory and barriers
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int A_MN, int B_MN>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int pairs,
                   cudaStream_t stream) {
  auto kernel = gemm2_kernel<A_MN, B_MN>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) {
      set_error_detail("gemm (CTA pairs): cudaFuncSetAttribute(max dynamic shared memory) failed");
      return e;
    }
    configured = true;
  }
  (void)cudaGetLastError();
  kernel<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_error_detail("gemm (CTA pairs): kernel launch failed");
  return e;
}

}  // namespace

// Same contract as gemm_bf16 without the tensor-parallel coupling; g.tp must be null.
cudaError_t gemm_bf16_pairs(const GemmArgs& g, int sm_count, cudaStream_t stream) {
  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {uint64_t(g.a_mn_major ? g.m : g.k), uint64_t(g.a_mn_major ? g.k : g.m)};
    const uint64_t strides[1] = {uint64_t(g.lda) * 2};
    const uint32_t box[2] = {64, uint32_t(g.a_mn_major ? BK : BM)};
    if (!make_tensor_map_bf16(&ta, g.a, 2, dims, strides, box)) return cudaErrorInvalidValue;
  }
  {
    const uint64_t dims[2] = {uint64_t(g.b_mn_major ? g.n : g.k), uint64_t(g.b_mn_major ? g.k : g.n)};
    const uint64_t strides[1] = {uint64_t(g.ldb) * 2};
    const uint32_t box[2] = {64, uint32_t(g.b_mn_major ? BK : BN_HALF)};
    if (!make_tensor_map_bf16(&tb, g.b, 2, dims, strides, box)) return cudaErrorInvalidValue;
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
  p.tiles_m = (g.m + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (g.n + BN - 1) / BN;
  p.accumulate = g.accumulate;
  p.status = g.status;
  const int tiles = p.tiles_m * p.tiles_n;
  const int most = sm_count / 2;
  const int pairs = tiles < most ? tiles : most;
  if (g.a_mn_major == 0 && g.b_mn_major == 0) return launch<0, 0>(ta, tb, p, pairs, stream);
  if (g.a_mn_major == 0 && g.b_mn_major == 1) return launch<0, 1>(ta, tb, p, pairs, stream);
  if (g.a_mn_major == 1 && g.b_mn_major == 0) return launch<1, 0>(ta, tb, p, pairs, stream);
  return launch<1, 1>(ta, tb, p, pairs, stream);
}

}  // namespace agb
