// Flash-attention backward in one pass over the scores (head_dim 128, bf16, grouped KV heads,
// segment lists): five products and one set of exponentials per 128 x 128 block of scores,
// where the two-kernel form in attention_bwd.cu needs seven and two.
//
// One CTA per (key tile of 128 rows, KV head, sample), handed out by an atomic ticket in
// key-tile order.  For every (query head of the group, block of 128 query rows) that can see
// the tile:
//   S^T  = K Q^T, dP^T = V dO^T                       (operands in shared memory)
//   P^T  = exp2(S^T scale - lse), dS^T = P^T (dP^T - delta) scale     (elementwise warps)
//   dV  += P^T dO,  dK += dS^T Q                      (P^T / dS^T read from TMEM)
//   dQ   = dS K                                       (dS^T read from shared memory, MN-major)
// dQ of a block is a partial sum over this CTA's keys.  Four drain warps add it to an FP32
// accumulator in global memory with red.global.add.v4.f32.  To keep the sum bit-reproducible the
// CTAs add in a fixed order: the schedule gives every (key tile, query block) its turn among
// the key tiles that see the block, a counter per (sample, query head, query block) holds the
// number of turns taken, and a CTA adds only when the counter equals its turn.  Tickets are
// taken at CTA start in key-tile order, so a CTA only ever waits for CTAs that started before
// it: no launch order is assumed.  Every wait is bounded.
//
// Issue order (a tcgen05.mma of up to 128 columns costs about 90 cycles to issue whatever its
// width, so the blocks are as wide as TMEM allows and the overlap comes from the order):
//   dV(i) | S^T(i+1) | dK(i) | dQ^T(i) | dP^T(i+1)
// TMEM: S^T [0,128) | dP^T, then dS^T packed, then dQ^T [128,256) | dV [256,384) | dK [384,512).
// dS^T goes to shared memory into the dO stage of its block, which is dead once dP^T and dV of
// the block have run.
#include <cuda_bf16.h>

#include "agb.h"
#include "attention_common.cuh"
#include "tensormap.h"

namespace agb {

bool make_rows_map_bwd(CUtensorMap* map, const void* base, int heads, int64_t rows, int64_t batch,
                       int64_t row_stride, int64_t batch_stride, int box_rows);

namespace {

constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int FUSED_THREADS = 448;  // 8 elementwise warps, TMA, MMA, 4 drain warps
constexpr int FUSED_BQ = 128;
constexpr int FUSED_MAX_BLOCKS = 1024;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int FUSED_SMEM = 6 * TILE_BYTES + FUSED_MAX_BLOCKS * 16 + 2 * 2 * FUSED_BQ * 4 + 1024 + 512;

struct FusedParams {
  const int* k_tiles;  // [tiles, 5]: k_row, rows, first_block, blocks, source (0 text, 1 visual)
  const int* text_valid;  // [B] valid text keys per sample (prefix), or null
  const int4* blocks;  // (q_block_row, lo, hi, turn): query rows [q_block_row + lo, q_block_row + hi)
  const float* lse;
  const float* delta;
  __nv_bfloat16* dk;   // [B, NK, Hkv, 128]
  __nv_bfloat16* dv;   // rows at dv_row_stride
  float* dq_acc;       // [B, nq_pad, Hq, 128], zeroed by the caller
  int* turns;          // [B, Hq, nq_pad / 128] counters, zeroed by the caller; turns[-1] is the ticket
  int* ticket;
  int64_t dv_row_stride, dv_batch_stride;
  int nq, nq_pad, nk, text_len, hq, hkv, group, batch_count;
  float scale, scale_log2;
  int* status;
};

__device__ __forceinline__ int load_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void add_release(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// p[0..3] += v (16-byte aligned): one L2 operation for four elements
__device__ __forceinline__ void red_add4(float* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(a)),
               "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}

__global__ void __launch_bounds__(FUSED_THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_vt,
                      const FusedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;        // [2]
  uint8_t* sdO = sQ + 2 * TILE_BYTES;         // [2]; receives dS^T of its block
  int4* blocks = reinterpret_cast<int4*>(sdO + 2 * TILE_BYTES);
  float* stats = reinterpret_cast<float*>(blocks + FUSED_MAX_BLOCKS);  // [2][nl[128], nd[128]]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stats + 2 * 2 * FUSED_BQ);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = bars + 1;      // [2]
  uint64_t* qd_empty = bars + 3;     // [2]
  uint64_t* st_full = bars + 5;      // S^T of an item complete
  uint64_t* dp_full = bars + 6;      // dP^T of an item complete
  uint64_t* pt_ready = bars + 7;     // [2] P^T of query chunk c of both halves written (count 8)
  uint64_t* dv_done = bars + 9;      // dV of an item finished: its dO stage may take dS^T
  uint64_t* ds_ready = bars + 10;    // dS^T in TMEM and in shared memory (count 8)
  uint64_t* dq_full = bars + 11;     // dQ^T of an item complete
  uint64_t* dq_drained = bars + 12;  // dQ^T read out of TMEM (count 4)
  uint64_t* grad_done = bars + 13;   // all products finished
  uint64_t* stats_bar = bars + 14;   // lse/delta of an item staged (count 256)
  uint64_t* turn_bar = bars + 15;    // this CTA's turn for the block has come (count 1)
  uint64_t* added_bar = bars + 16;   // every drain thread has issued and fenced its adds (count 128)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* n_blocks_smem = abort_flag + 1;
  volatile int* work_smem = abort_flag + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *work_smem = atomicAdd(p.ticket, 1);
    mbar_init(kv_full, 1);
    mbar_init(grad_done, 1);
    mbar_init(stats_bar, 256);
    mbar_init(st_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(&pt_ready[0], 8);
    mbar_init(&pt_ready[1], 8);
    mbar_init(dv_done, 1);
    mbar_init(ds_ready, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 4);
    mbar_init(turn_bar, 1);
    mbar_init(added_bar, 128);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qd_full[i], 1);
      mbar_init(&qd_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // Work in ticket order: KV head fastest, then sample, then key tile, so that a later ticket
  // never has an earlier key tile of the same (sample, head).
  const int work = *work_smem;
  const int kv_head = work % p.hkv;
  const int batch = (work / p.hkv) % p.batch_count;
  const int tile = work / (p.hkv * p.batch_count);
  const int* kt = p.k_tiles + 5 * tile;
  const int k_row = kt[0], k_rows = kt[1];
  // Text keys shape dQ like any other key but receive no gradient themselves; only the first
  // text_valid[b] of them exist for sample b.
  const bool text = kt[4] == 0;
  int k_valid = k_rows;
  if (text && p.text_valid) k_valid = max(0, min(k_rows, p.text_valid[batch] - k_row));
  for (int i = threadIdx.x; i < min(max(kt[3], 0), FUSED_MAX_BLOCKS); i += FUSED_THREADS) {
    blocks[i] = p.blocks[max(kt[2], 0) + i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = kt[3];
    // the entries this CTA is about to follow, against the extents of its tensors
    bool inside = rows_inside(k_row, k_rows, text ? p.text_len : p.nk, 128) && kt[2] >= 0 && n >= 0;
    for (int i = 0; i < min(n, FUSED_MAX_BLOCKS) && inside; ++i) {
      const int4 blk = blocks[i];
      inside = blk.x >= 0 && blk.x % FUSED_BQ == 0 && blk.x < p.nq_pad && blk.y >= 0 && blk.y < blk.z &&
               blk.z <= FUSED_BQ && blk.w >= 0;
    }
    if (n > FUSED_MAX_BLOCKS || !inside) {
      if (p.status) atomicCAS(p.status, 0, inside ? kBadArgument : kBadIndex);
      n = 0;
    }
    *n_blocks_smem = n;
  }
  __syncthreads();
  const uint32_t tmem_base = *tmem_slot;
  const int n_blocks = *n_blocks_smem;
  // item i: head kv_head * group + i / n_blocks, block i % n_blocks.  A tile without a valid key
  // (text beyond a sample's length) computes nothing but still takes its turns, below.
  const int n_turns = n_blocks * p.group;
  const int n_items = k_valid > 0 ? n_turns : 0;
  constexpr uint32_t C_ST = 0, C_DPT = 128, C_DV = 256, C_DK = 384;

  if (warp == 8) {
    if (lane == 0 && n_items > 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      const CUtensorMap* mk = text ? &tm_kt : &tm_k;
      const CUtensorMap* mv = text ? &tm_vt : &tm_v;
      tma_load_3d(sK, mk, kv_full, kv_head * ATT_D, k_row, batch);
      tma_load_3d(sK + HALF_BYTES, mk, kv_full, kv_head * ATT_D + 64, k_row, batch);
      tma_load_3d(sV, mv, kv_full, kv_head * ATT_D, k_row, batch);
      tma_load_3d(sV + HALF_BYTES, mv, kv_full, kv_head * ATT_D + 64, k_row, batch);
      bool ok = true;
      for (int i = 0; i < n_items && ok; ++i) {
        const int st = i & 1;
        const int head = kv_head * p.group + i / n_blocks;
        const int q0 = blocks[i % n_blocks].x;
        if (!mbar_wait(&qd_empty[st], ((i >> 1) & 1) ^ 1, guard, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&qd_full[st], 2 * TILE_BYTES);
        tma_load_3d(sQ + st * TILE_BYTES, &tm_q, &qd_full[st], head * ATT_D, q0, batch);
        tma_load_3d(sQ + st * TILE_BYTES + HALF_BYTES, &tm_q, &qd_full[st], head * ATT_D + 64, q0, batch);
        tma_load_3d(sdO + st * TILE_BYTES, &tm_do, &qd_full[st], head * ATT_D, q0, batch);
        tma_load_3d(sdO + st * TILE_BYTES + HALF_BYTES, &tm_do, &qd_full[st], head * ATT_D + 64, q0, batch);
      }
      if (!ok || *abort_flag) {
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 100000ull) {}
      }
    }
  } else if (warp == 9) {
    if (n_items > 0) {  // the whole warp runs the loop; one elected lane issues
      constexpr uint32_t idesc_s = make_idesc_bf16(128, FUSED_BQ, 0, 0);  // 128 keys x 128 queries
      constexpr uint32_t idesc_g = make_idesc_bf16(128, 128, 0, 1);       // 128 keys x 128 d, B MN-major
      constexpr uint32_t idesc_q = make_idesc_bf16(128, 128, 1, 1);       // 128 d x 128 queries, both MN-major
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      auto score_s = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait_w(&qd_full[st], (i >> 1) & 1, guard, kTimeoutMma)) return false;
        tc_fence_after_sync();
        const uint32_t q_addr = smem_u32(sQ + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
          tc_mma_ss_w(tmem_base + C_ST, make_smem_desc(k_addr + off, 16, 1024),
                      make_smem_desc(q_addr + off, 16, 1024), idesc_s, kk != 0);
        }
        tc_commit_w(st_full);
        return true;
      };
      auto score_p = [&](int i) {
        const int st = i & 1;
        const uint32_t do_addr = smem_u32(sdO + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
          tc_mma_ss_w(tmem_base + C_DPT, make_smem_desc(v_addr + off, 16, 1024),
                      make_smem_desc(do_addr + off, 16, 1024), idesc_s, kk != 0);
        }
        tc_commit_w(dp_full);
      };
      bool ok = mbar_wait_w(kv_full, 0, guard, kTimeoutMma);
      if (ok) ok = score_s(0);
      if (ok) score_p(0);
      for (int i = 0; i < n_items && ok; ++i) {
        const int st = i & 1;
        const uint32_t q_addr = smem_u32(sQ + st * TILE_BYTES);
        const uint32_t do_addr = smem_u32(sdO + st * TILE_BYTES);
        // dV: 16 queries per step; the packed columns of the 32 queries [32 g, 32 g + 32) start at
        // column 32 g.  P^T comes in two parts (g = c and g = 2 + c).
#pragma unroll
        for (int c = 0; c < 2 && ok; ++c) {
          if (!mbar_wait_w(&pt_ready[c], i & 1, guard, kTimeoutMma)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const int kk = (s4 >> 1) * 4 + c * 2 + (s4 & 1);
            tc_mma_ts_w(tmem_base + C_DV, tmem_base + C_ST + (kk >> 1) * 32 + (kk & 1) * 8,
                        make_smem_desc(do_addr + kk * 2048, HALF_BYTES, 1024), idesc_g, (i | c | s4) != 0);
          }
        }
        if (!ok) break;
        tc_commit_w(dv_done);
        if (i + 1 < n_items && !score_s(i + 1)) { ok = false; break; }
        if (!mbar_wait_w(ds_ready, i & 1, guard, kTimeoutMma)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          tc_mma_ts_w(tmem_base + C_DK, tmem_base + C_DPT + (kk >> 1) * 32 + (kk & 1) * 8,
                      make_smem_desc(q_addr + kk * 2048, HALF_BYTES, 1024), idesc_g, (i | kk) != 0);
        }
        // dQ = dS K (queries on the lanes) over the columns that held dS^T (behind dK, which read
        // them); dS^T comes from the dO stage of this item, read as an MN-major A operand.
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          tc_mma_ss_w(tmem_base + C_DPT, make_smem_desc(do_addr + kk * 2048, HALF_BYTES, 1024),
                      make_smem_desc(k_addr + kk * 2048, HALF_BYTES, 1024), idesc_q, kk != 0);
        }
        tc_commit_w(dq_full);
        tc_commit_w(&qd_empty[st]);
        if (!mbar_wait_w(dq_drained, i & 1, guard, kTimeoutMma)) { ok = false; break; }
        tc_fence_after_sync();
        if (i + 1 < n_items) score_p(i + 1);
      }
      if (ok) tc_commit_w(grad_done);
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------------ drain warps: dQ^T
    const int quarter = warp & 3;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const int row = quarter * 32 + lane;  // query row of this thread within the block
    const bool leader = warp == 10 && lane == 0;
    bool ok = n_items > 0;
    if (leader && n_items == 0) {
      // nothing to add: pass every turn on in order, so that later key tiles are not kept waiting
      for (int i = 0; i < n_turns; ++i) {
        const int4 blk = blocks[i % n_blocks];
        const int head = kv_head * p.group + i / n_blocks;
        int* turn = p.turns + (int64_t(batch) * p.hq + head) * (p.nq_pad / FUSED_BQ) + blk.x / FUSED_BQ;
        const uint64_t start = global_timer_ns();
        bool mine = load_acquire(turn) == blk.w;
        uint32_t spins = 0;
        while (!mine) {
          mine = load_acquire(turn) == blk.w;
          if ((++spins & 63u) == 0 && global_timer_ns() - start > AGB_WAIT_LIMIT_NS) break;
        }
        if (!mine) {
          if (p.status) atomicCAS(p.status, 0, kTimeoutPeer);
          break;
        }
        add_release(turn, 1);
      }
    }
    for (int i = 0; i < n_items && ok; ++i) {
      const int4 blk = blocks[i % n_blocks];
      const int head = kv_head * p.group + i / n_blocks;
      float* dst = p.dq_acc + ((int64_t(batch) * p.nq_pad + blk.x + row) * p.hq + head) * ATT_D;
      const bool row_ok = row >= blk.y && row < blk.z;
      int* turn = p.turns + (int64_t(batch) * p.hq + head) * (p.nq_pad / FUSED_BQ) + blk.x / FUSED_BQ;
      if (!mbar_wait(dq_full, i & 1, guard, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t a[32], b[32];
      tmem_ld_32x32(tmem_base + lane_base + C_DPT, a);
      tmem_ld_32x32(tmem_base + lane_base + C_DPT + 32, b);
      tmem_ld_wait();
      if (leader) {
        // wait for this CTA's turn on the block (CTAs of earlier key tiles add first)
        const uint64_t start = global_timer_ns();
        bool mine = load_acquire(turn) == blk.w;
        uint32_t spins = 0;
        while (!mine) {
          mine = load_acquire(turn) == blk.w;
          if ((++spins & 63u) == 0 && (*abort_flag || global_timer_ns() - start > AGB_WAIT_LIMIT_NS)) break;
        }
        if (!mine) {
          *abort_flag = 1;
          if (p.status) atomicCAS(p.status, 0, kTimeoutPeer);
        }
        mbar_arrive(turn_bar);
      }
      if (!mbar_wait(turn_bar, i & 1, guard, kTimeoutEpilogue) || *abort_flag) { ok = false; break; }
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          red_add4(dst + 4 * c, a[4 * c], a[4 * c + 1], a[4 * c + 2], a[4 * c + 3]);
          red_add4(dst + 32 + 4 * c, b[4 * c], b[4 * c + 1], b[4 * c + 2], b[4 * c + 3]);
        }
      }
      tmem_ld_32x32(tmem_base + lane_base + C_DPT + 64, a);
      tmem_ld_32x32(tmem_base + lane_base + C_DPT + 96, b);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_drained);  // the MMA warp may overwrite the columns
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          red_add4(dst + 64 + 4 * c, a[4 * c], a[4 * c + 1], a[4 * c + 2], a[4 * c + 3]);
          red_add4(dst + 96 + 4 * c, b[4 * c], b[4 * c + 1], b[4 * c + 2], b[4 * c + 3]);
        }
      }
      __threadfence();
      mbar_arrive(added_bar);
      if (leader) {
        if (mbar_wait(added_bar, i & 1, guard, kTimeoutEpilogue)) add_release(turn, 1);
        else ok = false;
      }
    }
  } else {
    // ------------------------------------------------------------------ elementwise warps
    const int quarter = warp & 3, half = warp >> 2;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const int tid = (warp << 5) + lane;      // 0..255
    const int key = quarter * 32 + lane;     // key row of this thread
    // rows past the tile's keys (a partial last tile, text beyond its valid length) hold other
    // data: their probabilities are zero so that they add nothing to dQ
    const bool key_ok = key < k_valid;
    bool ok = n_items > 0;
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    const float2 ps2 = make_float2(p.scale, p.scale);
    auto fetch_stat = [&](int i) -> float {
      // threads 0..127: -lse*log2(e) (or -inf: probability 0), threads 128..255: -delta*scale
      const int4 blk = blocks[i % n_blocks];
      const int head = kv_head * p.group + i / n_blocks;
      const int col = tid & (FUSED_BQ - 1);
      const int q = blk.x + col;
      const bool valid = col >= blk.y && col < blk.z && q < p.nq;
      const int64_t idx = (int64_t(batch) * p.hq + head) * p.nq + q;
      if (tid < FUSED_BQ) return valid ? -p.lse[idx] * LOG2E : -INFINITY;
      return valid ? -p.delta[idx] * p.scale : 0.f;
    };
    if (ok) {
      stats[tid] = fetch_stat(0);
      mbar_arrive(stats_bar);
    }
    for (int i = 0; i < n_items && ok; ++i) {
      const bool more = i + 1 < n_items;
      float next_stat = 0.f;
      if (more) next_stat = fetch_stat(i + 1);
      const float* my_stats = stats + (i & 1) * 2 * FUSED_BQ + half * 64;
      if (!mbar_wait(stats_bar, i & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      if (!mbar_wait(st_full, i & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t prob[32];  // P^T of this thread's 64 query columns as packed bf16, kept for dS^T
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], pp[16];
        tmem_ld_32x32(tmem_base + lane_base + C_ST + half * 64 + c * 32, sv);
        tmem_ld_wait();
        const float4* nl4 = reinterpret_cast<const float4*>(my_stats + c * 32);
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {  // four query columns per step
          const float4 nl = nl4[k4];
          const float2 x0 = ffma2(make_float2(__uint_as_float(sv[4 * k4]), __uint_as_float(sv[4 * k4 + 1])),
                                  sc2, make_float2(nl.x, nl.y));
          const float2 x1 = ffma2(make_float2(__uint_as_float(sv[4 * k4 + 2]), __uint_as_float(sv[4 * k4 + 3])),
                                  sc2, make_float2(nl.z, nl.w));
          pp[2 * k4] = key_ok ? pack_bf16(exp2f(x0.x), exp2f(x0.y)) : 0u;
          pp[2 * k4 + 1] = key_ok ? pack_bf16(exp2f(x1.x), exp2f(x1.y)) : 0u;
          prob[c * 16 + 2 * k4] = pp[2 * k4];
          prob[c * 16 + 2 * k4 + 1] = pp[2 * k4 + 1];
        }
        // the packed results land in columns this thread has already read
        tmem_st_32x16(tmem_base + lane_base + C_ST + half * 64 + c * 32, pp);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pt_ready[c]);
      }
      if (!mbar_wait(dp_full, i & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t ds[32];  // dS^T of the 64 columns, packed: to TMEM in place and to shared memory
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dv[32];
        tmem_ld_32x32(tmem_base + lane_base + C_DPT + half * 64 + c * 32, dv);
        tmem_ld_wait();
        const float4* nd4 = reinterpret_cast<const float4*>(my_stats + FUSED_BQ + c * 32);
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
          const float4 nd = nd4[k4];
          const float2 g0 = ffma2(make_float2(__uint_as_float(dv[4 * k4]), __uint_as_float(dv[4 * k4 + 1])),
                                  ps2, make_float2(nd.x, nd.y));
          const float2 g1 = ffma2(make_float2(__uint_as_float(dv[4 * k4 + 2]), __uint_as_float(dv[4 * k4 + 3])),
                                  ps2, make_float2(nd.z, nd.w));
          const uint32_t p0 = prob[c * 16 + 2 * k4], p1 = prob[c * 16 + 2 * k4 + 1];
          const float2 d0 = fmul2(make_float2(bf16_lo(p0), bf16_hi(p0)), g0);
          const float2 d1 = fmul2(make_float2(bf16_lo(p1), bf16_hi(p1)), g1);
          ds[c * 16 + 2 * k4] = pack_bf16(d0.x, d0.y);
          ds[c * 16 + 2 * k4 + 1] = pack_bf16(d1.x, d1.y);
        }
        uint32_t part[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) part[k] = ds[c * 16 + k];
        tmem_st_32x16(tmem_base + lane_base + C_DPT + half * 64 + c * 32, part);
      }
      // dS^T also goes to shared memory for the dQ^T product: row = key, this half's 64 query
      // columns are one 128-byte row of atom column `half`, 16-byte chunks swizzled by the row.
      if (!mbar_wait(dv_done, i & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      {
        uint8_t* row = sdO + (i & 1) * TILE_BYTES + half * HALF_BYTES + key * 128;
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          *reinterpret_cast<uint4*>(row + ((cc ^ (key & 7)) << 4)) =
              make_uint4(ds[4 * cc], ds[4 * cc + 1], ds[4 * cc + 2], ds[4 * cc + 3]);
        }
      }
      fence_proxy_async_smem();
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
      // The other stats buffer was last read for item i - 1; every thread has passed the wait
      // of phase i above, which all threads entered only after finishing item i - 1.
      if (more) {
        stats[((i + 1) & 1) * 2 * FUSED_BQ + tid] = next_stat;
        mbar_arrive(stats_bar);
      }
    }
    if (ok) ok = mbar_wait(grad_done, 0, guard, kTimeoutEpilogue);
    if (ok && !text) {
      tc_fence_after_sync();
      const bool row_ok = key < k_rows;
      const int64_t base = ((int64_t(batch) * p.nk + k_row + key) * p.hkv + kv_head) * ATT_D;
      const int64_t base_v = int64_t(batch) * p.dv_batch_stride + int64_t(k_row + key) * p.dv_row_stride +
                             int64_t(kv_head) * ATT_D;
      __nv_bfloat16* dst = half == 0 ? p.dv + base_v : p.dk + base;
      const uint32_t col0 = half == 0 ? C_DV : C_DK;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_base + col0 + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[g * 8 + 0]), __uint_as_float(o[g * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(o[g * 8 + 2]), __uint_as_float(o[g * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(o[g * 8 + 4]), __uint_as_float(o[g * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(o[g * 8 + 6]), __uint_as_float(o[g * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = v;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// dq[b, q, h, :] = bf16(acc[b, q, h, :]) for q < nq (acc has nq_pad rows per sample).
__global__ void __launch_bounds__(256) attn_dq_cast_kernel(const float* __restrict__ acc,
                                                           __nv_bfloat16* __restrict__ dq, int64_t nq,
                                                           int64_t nq_pad, int64_t row_floats, int64_t vecs) {
  const int64_t per_row = row_floats / 8;
  for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < vecs; i += int64_t(gridDim.x) * 256) {
    const int64_t row = i / per_row, col = (i - row * per_row) * 8;
    const int64_t b = row / nq, q = row - b * nq;
    const float4* src = reinterpret_cast<const float4*>(acc + (b * nq_pad + q) * row_floats + col);
    const float4 lo = src[0], hi = src[1];
    uint4 v;
    v.x = pack_bf16(lo.x, lo.y);
    v.y = pack_bf16(lo.z, lo.w);
    v.z = pack_bf16(hi.x, hi.y);
    v.w = pack_bf16(hi.z, hi.w);
    *reinterpret_cast<uint4*>(dq + row * row_floats + col) = v;
  }
}

__global__ void __launch_bounds__(256) attn_delta_fused_kernel(const __nv_bfloat16* __restrict__ out,
                                                               const __nv_bfloat16* __restrict__ grad,
                                                               float* __restrict__ delta, int64_t nq,
                                                               int hq, int64_t units) {
  // one warp per (sample, query, head): delta = sum_d dO * O
  const int64_t unit = (int64_t(blockIdx.x) * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (unit >= units) return;
  const uint2 o = *reinterpret_cast<const uint2*>(out + unit * ATT_D + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(grad + unit * ATT_D + lane * 4);
  float s = bf16_lo(o.x) * bf16_lo(g.x) + bf16_hi(o.x) * bf16_hi(g.x) + bf16_lo(o.y) * bf16_lo(g.y) +
            bf16_hi(o.y) * bf16_hi(g.y);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    const int64_t h = unit % hq, rest = unit / hq;
    const int64_t q = rest % nq, b = rest / nq;
    delta[(b * hq + h) * nq + q] = s;
  }
}

}  // namespace

cudaError_t attention_bwd_fused(const AttnBwdArgs& b, const int* k_tiles, const int* blocks, float* dq_acc,
                                int* turns, int64_t nq_pad, cudaStream_t stream) {
  // b.k_tiles / b.q_lists are not used: k_tiles / blocks describe the work (text tiles included).
  const AttnArgs& a = b.fwd;
  if (a.batch == 0 || a.nq == 0) return cudaSuccess;
  CUtensorMap tq, tdo, tk, tv, tkt, tvt;
  const int64_t dense_row = int64_t(a.hq) * ATT_D;
  if (!make_rows_map_bwd(&tq, a.q, a.hq, a.nq, a.batch, a.q_row_stride, a.q_batch_stride, 128) ||
      !make_rows_map_bwd(&tdo, b.grad_out, a.hq, a.nq, a.batch, dense_row, dense_row * a.nq, 128) ||
      !make_rows_map_bwd(&tk, a.k, a.hkv, a.nk, a.batch, a.kv_row_stride, a.kv_batch_stride, 128) ||
      !make_rows_map_bwd(&tv, a.v, a.hkv, a.nk, a.batch, a.v_row_stride ? a.v_row_stride : a.kv_row_stride,
                         a.v_row_stride ? a.v_batch_stride : a.kv_batch_stride, 128)) {
    set_error_detail("attention_bwd_fused: tensor map refused by the driver");
    return cudaErrorInvalidValue;
  }
  if (a.text_k) {
    if (!make_rows_map_bwd(&tkt, a.text_k, a.hkv, a.text_len, a.batch, a.text_row_stride, a.text_batch_stride, 128) ||
        !make_rows_map_bwd(&tvt, a.text_v, a.hkv, a.text_len, a.batch, a.text_row_stride, a.text_batch_stride, 128)) {
      set_error_detail("attention_bwd_fused: text tensor map refused by the driver");
      return cudaErrorInvalidValue;
    }
  } else {
    tkt = tk;
    tvt = tv;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FUSED_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int64_t units = a.batch * a.nq * a.hq;
  attn_delta_fused_kernel<<<unsigned((units + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a.out), static_cast<const __nv_bfloat16*>(b.grad_out), b.delta, a.nq,
      a.hq, units);
  if (b.num_k_tiles > 0) {
    FusedParams p;
    p.k_tiles = k_tiles;
    p.text_valid = a.text_valid;
    p.blocks = reinterpret_cast<const int4*>(blocks);
    p.lse = a.lse;
    p.delta = b.delta;
    p.dk = static_cast<__nv_bfloat16*>(b.dk);
    p.dv = static_cast<__nv_bfloat16*>(b.dv);
    p.dq_acc = dq_acc;
    p.turns = turns + 1;
    p.ticket = turns;
    p.dv_row_stride = b.dv_row_stride ? b.dv_row_stride : int64_t(a.hkv) * ATT_D;
    p.dv_batch_stride = b.dv_row_stride ? b.dv_batch_stride : int64_t(a.nk) * a.hkv * ATT_D;
    p.nq = int(a.nq);
    p.nq_pad = int(nq_pad);
    p.nk = int(a.nk);
    p.text_len = int(a.text_len);
    p.hq = a.hq;
    p.hkv = a.hkv;
    p.group = a.hq / a.hkv;
    p.batch_count = int(a.batch);
    p.scale = a.scale;
    p.scale_log2 = a.scale * LOG2E;
    p.status = a.status;
    const unsigned ctas = unsigned(b.num_k_tiles) * unsigned(a.hkv) * unsigned(a.batch);
    attn_bwd_fused_kernel<<<ctas, FUSED_THREADS, FUSED_SMEM, stream>>>(tq, tdo, tk, tv, tkt, tvt, p);
  }
  const int64_t vecs = a.batch * a.nq * dense_row / 8;
  const unsigned grid = unsigned(std::min<int64_t>((vecs + 255) / 256, 148 * 16));
  attn_dq_cast_kernel<<<grid, 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(b.dq), a.nq, nq_pad,
                                                dense_row, vecs);
  return cudaGetLastError();
}

}  // namespace agb
