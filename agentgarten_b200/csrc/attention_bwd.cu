// Flash-attention backward on tcgen05 (head_dim 128, bf16, grouped KV heads, segment lists).
//
// Three kernels, all deterministic (no atomics):
//   attn_delta   delta[b, h, q] = sum_d dO * O                      (row-wise, HBM-bound)
//   attn_dq      one CTA per (query tile, query head, sample) walks the key tiles of the
//                tile's segments:  S = Q K^T, dP = dO V^T, dS = P o (dP - delta) * scale,
//                dQ += dS K.  Text keys take part (they shape P) but get no gradient.
//   attn_dkdv    one CTA per (visual key tile, KV head, sample) walks every query tile that
//                sees it, for the query heads of its group, in a fixed order:
//                S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q.
// Probabilities are recomputed from the saved log-sum-exp.  P / dS are handed to the tensor
// core as packed bf16 in TMEM (A operand), K/V/Q/dO tiles are read from shared memory both
// K-major (for the score products) and MN-major (for the gradient products) without any
// transposed copy: the same swizzled tile serves both descriptors.
#include "agb.h"
#include "attention_common.cuh"
#include "tensormap.h"

namespace agb {
namespace {

constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int BWD_THREADS = 192;
constexpr int DQ_THREADS = 320;  // 8 elementwise warps + TMA + MMA
constexpr float LOG2E = 1.4426950408889634f;

// ---------------------------------------------------------------------------- delta
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ out,
                                                         const __nv_bfloat16* __restrict__ grad,
                                                         float* __restrict__ delta, int64_t nq,
                                                         int hq, int64_t units) {
  // one warp per (b, q, h); delta laid out [B, Hq, NQ]
  const int64_t unit = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const uint2 a = *reinterpret_cast<const uint2*>(out + unit * 128 + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(grad + unit * 128 + lane * 4);
  float s = bf16_lo(a.x) * bf16_lo(g.x) + bf16_hi(a.x) * bf16_hi(g.x) +
            bf16_lo(a.y) * bf16_lo(g.y) + bf16_hi(a.y) * bf16_hi(g.y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const int h = int(unit % hq);
    const int64_t bq = unit / hq;
    const int64_t b = bq / nq, q = bq % nq;
    delta[(b * hq + h) * nq + q] = s;
  }
}

// ------------------------------------------------------------------------------- dQ
// One CTA per (query tile of 128 rows, query head, sample) walks the key tiles of the tile's
// segments.  Three products per key tile, issued one tile staggered so that the tensor pipe
// never waits for the elementwise warps (a tcgen05.mma of 128 rows costs about 90 cycles to
// issue whatever its width up to 128 columns, so the products are as wide as they can be):
//   S(j+1) = Q K^T | dQ += dS(j) K | dP(j+1) = dO V^T
// The exponentials of tile j+1 run under dQ(j) and dP(j+1), its dS under S(j+2).  The
// probabilities stay in registers; dS is packed over the first half of the dP columns it came
// from and read from there by the dQ product.
// smem: Q, dO (resident) + K, V rings (2 stages each, released separately: V after dP, K
// after dQ).  TMEM: S[2] [0,256) dP [256,384) dQ [384,512).
constexpr int DQ_SMEM = 6 * TILE_BYTES + ATT_MAX_TILES * int(sizeof(KeyTile)) + 1024 + 512;

struct DqParams {
  const int* q_tiles;
  const int* entries;
  const int* text_valid;
  const float* lse;    // [B, Hq, NQ]
  const float* delta;  // [B, Hq, NQ]
  __nv_bfloat16* dq;   // [B, NQ, Hq, 128]
  int nq, hq, group;
  int nk, text_len;    // extents the work lists are checked against
  float scale, scale_log2;
  int* status;
};

__global__ void __launch_bounds__(DQ_THREADS, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_vt,
               const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
               const DqParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;
  uint8_t* sV = smem + 4 * TILE_BYTES;
  KeyTile* tiles = reinterpret_cast<KeyTile*>(smem + 6 * TILE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + ATT_MAX_TILES);
  uint64_t* q_full = bars;        // Q and dO
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* k_empty = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] S of a tile is in TMEM
  uint64_t* dp_full = bars + 11;  // dP of a tile is in TMEM
  uint64_t* ds_ready = bars + 12; // [2] dS of key chunk c of both halves written over dP (count 8)
  uint64_t* dq_done = bars + 14;  // every dQ product finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* n_tiles_smem = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / p.group;
  const int* qt = p.q_tiles + 5 * blockIdx.x;
  const int q_row = qt[0], q_rows = qt[1], q_local = qt[4];
  const WaitGuard guard{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(&ds_ready[0], 8);
    mbar_init(&ds_ready[1], 8);
    mbar_init(dq_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_fence_init();
    int n = rows_inside(q_row, q_rows, p.nq, ATT_BM) && qt[2] >= 0 && qt[3] >= 0
                ? build_key_tiles(p.entries, qt[2], qt[3], p.text_valid, batch, q_local, q_rows, tiles, p.nk,
                                  p.text_len)
                : -2;
    if (n < 0) {
      if (p.status) atomicCAS(p.status, 0, n == -2 ? kBadIndex : kBadArgument);
      n = 0;
    }
    *n_tiles_smem = n;
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int n_tiles = *n_tiles_smem;
  constexpr uint32_t C_S = 0, C_DP = 256, C_DQ = 384;

  if (warp == 8) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      tma_load_3d(sQ, &tm_q, q_full, head * ATT_D, q_row, batch);
      tma_load_3d(sQ + HALF_BYTES, &tm_q, q_full, head * ATT_D + 64, q_row, batch);
      tma_load_3d(sdO, &tm_do, q_full, head * ATT_D, q_row, batch);
      tma_load_3d(sdO + HALF_BYTES, &tm_do, q_full, head * ATT_D + 64, q_row, batch);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t parity = ((j >> 1) & 1) ^ 1;
        const KeyTile t = tiles[j];
        const CUtensorMap* mk = t.source == 0 ? &tm_kt : &tm_k;
        const CUtensorMap* mv = t.source == 0 ? &tm_vt : &tm_v;
        // the V stage comes free one product earlier than the K stage
        if (!mbar_wait(&v_empty[st], parity, guard, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], TILE_BYTES);
        tma_load_3d(sV + st * TILE_BYTES, mv, &v_full[st], kv_head * ATT_D, t.row, batch);
        tma_load_3d(sV + st * TILE_BYTES + HALF_BYTES, mv, &v_full[st], kv_head * ATT_D + 64, t.row, batch);
        if (!mbar_wait(&k_empty[st], parity, guard, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], TILE_BYTES);
        tma_load_3d(sK + st * TILE_BYTES, mk, &k_full[st], kv_head * ATT_D, t.row, batch);
        tma_load_3d(sK + st * TILE_BYTES + HALF_BYTES, mk, &k_full[st], kv_head * ATT_D + 64, t.row, batch);
      }
      if (!ok || *abort_flag) {
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 100000ull) {}
      }
    }
  } else if (warp == 9) {
    if (n_tiles > 0) {  // the whole warp runs the loop; one elected lane issues
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);  // both K-major
      constexpr uint32_t idesc_mn = make_idesc_bf16(128, 128, 0, 1);  // B MN-major
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      bool ok = mbar_wait_w(q_full, 0, guard, kTimeoutMma);
      // S of tile j into buffer j & 1 (its last reader, the exponentials of tile j - 2, finished
      // before dS(j-2) was announced, which the dQ product of that tile waited for).
      auto score_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait_w(&k_full[st], (j >> 1) & 1, guard, kTimeoutMma)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
          tc_mma_ss_w(tmem_base + C_S + st * 128, make_smem_desc(q_addr + off, 16, 1024),
                    make_smem_desc(k_addr + off, 16, 1024), idesc_kk, kk != 0);
        }
        tc_commit_w(&s_full[st]);
        return true;
      };
      // dP of tile j over dS(j-1), behind the dQ product that read it.
      auto score_p = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait_w(&v_full[st], (j >> 1) & 1, guard, kTimeoutMma)) return false;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
          tc_mma_ss_w(tmem_base + C_DP, make_smem_desc(do_addr + off, 16, 1024),
                    make_smem_desc(v_addr + off, 16, 1024), idesc_kk, kk != 0);
        }
        tc_commit_w(dp_full);
        tc_commit_w(&v_empty[st]);
        return true;
      };
      if (ok) ok = score_s(0);
      if (ok) ok = score_p(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_tiles && !score_s(j + 1)) { ok = false; break; }
        const uint32_t k_addr = smem_u32(sK + st * TILE_BYTES);
        // 16 keys per step; the packed columns of the 32 keys [32 g, 32 g + 32) start at column
        // 32 g.  The warps announce dS in two parts (their first and their second 32 columns:
        // g = c and g = 2 + c), so half of the product is issued while they finish the rest.
#pragma unroll
        for (int c = 0; c < 2 && ok; ++c) {
          if (!mbar_wait_w(&ds_ready[c], j & 1, guard, kTimeoutMma)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const int kk = (s4 >> 1) * 4 + c * 2 + (s4 & 1);
            tc_mma_ts_w(tmem_base + C_DQ, tmem_base + C_DP + (kk >> 1) * 32 + (kk & 1) * 8,
                      make_smem_desc(k_addr + kk * 2048, HALF_BYTES, 1024), idesc_mn,
                      (j | c | s4) != 0);
          }
        }
        if (!ok) break;
        tc_commit_w(&k_empty[st]);
        if (j + 1 < n_tiles && !score_p(j + 1)) { ok = false; break; }
      }
      if (ok) tc_commit_w(dq_done);
    }
  } else {
    // Eight warps: warps q and q + 4 share the 32 rows of TMEM lane quarter q and take one
    // half of the 128 key columns each, so every scheduler has two of them to interleave.
    const int quarter = warp & 3, half = warp >> 2;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const int my_row = quarter * 32 + lane;
    const bool row_ok = my_row < q_rows;
    const int64_t stat_index = (int64_t(batch) * p.hq + head) * p.nq + q_row + my_row;
    const bool in_range = q_row + my_row < p.nq;
    const float lse2 = in_range ? p.lse[stat_index] * LOG2E : 0.f;
    const float delta = in_range ? p.delta[stat_index] : 0.f;
    // dS = exp2(S scale_log2 - lse2) * (dP scale - delta scale): two-lane arithmetic, 32 key
    // columns at a time.
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    const float2 nl2 = make_float2(-lse2, -lse2);
    const float2 ps2 = make_float2(p.scale, p.scale);
    const float2 nd2 = make_float2(-delta * p.scale, -delta * p.scale);
    bool ok = n_tiles > 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int buf = j & 1;
      const KeyTile t = tiles[j];
      if (!mbar_wait(&s_full[buf], (j >> 1) & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      tc_fence_after_sync();
      // Only tiles with masked keys or rows (a partial last tile, the causal diagonal, the
      // ragged last query tile) pay for the masking; the test is uniform over the CTA.
      const bool plain = t.valid == ATT_BN && t.causal0 < 0 && q_rows == ATT_BM;
      int valid = t.valid;
      if (t.causal0 >= 0) valid = min(valid, q_local + my_row + 1 - t.causal0);
      if (!row_ok) valid = 0;
      float2 prob[32];  // probabilities of this thread's 64 key columns, kept for dS
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(tmem_base + lane_base + C_S + buf * 128 + half * 64 + c * 32, sv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = ffma2(make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])),
                                 sc2, nl2);
          float2 e = make_float2(exp2f(x.x), exp2f(x.y));
          if (!plain) {
            const int col = half * 64 + c * 32 + 2 * i;
            if (col >= valid) e.x = 0.f;
            if (col + 1 >= valid) e.y = 0.f;
          }
          prob[c * 16 + i] = e;
        }
      }
      if (!mbar_wait(dp_full, j & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dv[32], packed[16];
        tmem_ld_32x32(tmem_base + lane_base + C_DP + half * 64 + c * 32, dv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 g = ffma2(make_float2(__uint_as_float(dv[2 * i]), __uint_as_float(dv[2 * i + 1])),
                                 ps2, nd2);
          const float2 ds = fmul2(prob[c * 16 + i], g);
          packed[i] = pack_bf16(ds.x, ds.y);
        }
        // the packed results land in columns this thread has already read
        tmem_st_32x16(tmem_base + lane_base + C_DP + half * 64 + c * 32, packed);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_ready[c]);
      }
    }
    if (ok) ok = mbar_wait(dq_done, 0, guard, kTimeoutEpilogue);
    if (n_tiles == 0 || ok) {
      tc_fence_after_sync();
      __nv_bfloat16* dst = p.dq + ((int64_t(batch) * p.nq + q_row + my_row) * p.hq + head) * ATT_D;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem_base + lane_base + C_DQ + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
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

// ---------------------------------------------------------------------------- dK / dV
// One CTA per (key tile of 128 rows, KV head, sample).  It walks every (query head of the
// group, block of 128 query rows) that can see the tile:
//   S^T  = K Q^T, dP^T = V dO^T                 (128 keys x 128 queries each, operands in smem)
//   P^T  = exp2(S^T scale - lse), dS^T = P^T (dP^T - delta) scale   (softmax warps)
//   dV  += P^T dO,  dK += dS^T Q                (P^T / dS^T read from TMEM)
// A tcgen05.mma of 128 rows costs about 90 cycles to issue whatever its width up to 128
// columns (measured: 92 cycles for N = 64 and N = 128 alike, 128 for N = 256), so the kernel
// issues as few and as wide products as TMEM allows: blocks of 128 queries, which fill TMEM
// with one S^T, one dP^T and the two accumulators.  With single score buffers the overlap
// comes from the order of issue, one block staggered against the next:
//   dV(i) | S^T(i+1) | dK(i) | dP^T(i+1)
// The exponentials of block i+1 run under dK(i) and dP^T(i+1), its dS^T under dV(i+1) and
// S^T(i+2); tcgen05.mma operations of one thread execute in issue order, which makes
// refilling a buffer behind the product that reads its P^T / dS^T safe without a barrier.
// smem: K, V (resident) + Q, dO rings (2 stages of 128 rows) + item list + lse/delta vectors.
// TMEM: S^T [0,128) dP^T [128,256) dV [256,384) dK [384,512).  Eight warps: warps k and k + 4
// share the 32 key rows of lane quarter k and take 64 of the 128 query columns each, 32 at a
// time; the packed bf16 results overwrite the first 16 columns of the 32 they came from.
constexpr int DKV_BQ = 128;                     // query rows per item
constexpr int DKV_STAGES = 2;
constexpr int DKV_MAX_ITEMS = 2048;
constexpr int DKV_SMEM = 2 * TILE_BYTES + 2 * DKV_STAGES * TILE_BYTES + DKV_MAX_ITEMS * 8 +
                         2 * 2 * DKV_BQ * 4 + 1024 + 512;

struct DkvParams {
  const int* k_tiles;  // [tiles, 5]: k_row, rows, first_reader, readers, causal (unused)
  const int* q_lists;  // [*, 2]: q_row, q_len
  const float* lse;
  const float* delta;
  __nv_bfloat16* dk;  // [B, NK, Hkv, 128]
  __nv_bfloat16* dv;  // rows at dv_row_stride (dense by default)
  int64_t dv_row_stride, dv_batch_stride;
  int nq, nk, hq, hkv, group;
  float scale, scale_log2;
  int* status;
};

__global__ void __launch_bounds__(DQ_THREADS, 1)
attn_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const DkvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;                 // [DKV_STAGES]
  uint8_t* sdO = sQ + DKV_STAGES * TILE_BYTES;         // [DKV_STAGES]
  int2* items = reinterpret_cast<int2*>(sdO + DKV_STAGES * TILE_BYTES);  // (q_row, rows | head << 8)
  float* stats = reinterpret_cast<float*>(items + DKV_MAX_ITEMS);        // [2][nl[128], nd[128]]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stats + 2 * 2 * DKV_BQ);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = bars + 1;     // [2]
  uint64_t* qd_empty = bars + 3;    // [2]
  uint64_t* st_full = bars + 5;     // S^T of an item complete
  uint64_t* dp_full = bars + 6;     // dP^T of an item complete
  uint64_t* pt_ready = bars + 7;    // [2] P^T of query chunk c of both halves written (count 8)
  uint64_t* ds_ready = bars + 9;    // dS^T written (count 8)
  uint64_t* grad_done = bars + 10;  // all gradient products finished
  uint64_t* stats_bar = bars + 11;  // lse/delta of an item staged (count 256)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* n_items_smem = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_head = blockIdx.y, batch = blockIdx.z;
  const int* kt = p.k_tiles + 5 * blockIdx.x;
  const int k_row = kt[0], k_rows = kt[1];
  const WaitGuard guard{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    mbar_init(grad_done, 1);
    mbar_init(stats_bar, 256);
    mbar_init(st_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(&pt_ready[0], 8);
    mbar_init(&pt_ready[1], 8);
    mbar_init(ds_ready, 8);
    for (int i = 0; i < DKV_STAGES; ++i) {
      mbar_init(&qd_full[i], 1);
      mbar_init(&qd_empty[i], 1);
    }
    mbar_fence_init();
    int n = 0;
    bool overflow = false;
    bool inside = rows_inside(k_row, k_rows, p.nk, 128) && kt[2] >= 0 && kt[3] >= 0;
    for (int g = 0; g < p.group && !overflow && inside; ++g) {
      const int head = kv_head * p.group + g;
      for (int r = kt[2]; r < kt[2] + kt[3] && !overflow; ++r) {
        const int q0 = p.q_lists[2 * r], len = p.q_lists[2 * r + 1];
        if (q0 < 0 || len < 0 || int64_t(q0) + len > p.nq) {
          inside = false;
          break;
        }
        for (int off = 0; off < len; off += DKV_BQ) {
          if (n >= DKV_MAX_ITEMS) { overflow = true; break; }
          items[n++] = make_int2(q0 + off, min(DKV_BQ, len - off) | (head << 8));
        }
      }
    }
    if (overflow || !inside) {
      if (p.status) atomicCAS(p.status, 0, inside ? kBadArgument : kBadIndex);
      n = 0;
    }
    *n_items_smem = n;
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int n_items = *n_items_smem;
  constexpr uint32_t C_ST = 0, C_DPT = 128, C_DV = 256, C_DK = 384;

  if (warp == 8) {
    if (lane == 0 && n_items > 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_3d(sK, &tm_k, kv_full, kv_head * ATT_D, k_row, batch);
      tma_load_3d(sK + HALF_BYTES, &tm_k, kv_full, kv_head * ATT_D + 64, k_row, batch);
      tma_load_3d(sV, &tm_v, kv_full, kv_head * ATT_D, k_row, batch);
      tma_load_3d(sV + HALF_BYTES, &tm_v, kv_full, kv_head * ATT_D + 64, k_row, batch);
      bool ok = true;
      for (int i = 0; i < n_items && ok; ++i) {
        const int st = i % DKV_STAGES;
        const int2 it = items[i];
        const int head = it.y >> 8;
        if (!mbar_wait(&qd_empty[st], ((i / DKV_STAGES) & 1) ^ 1, guard, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&qd_full[st], 2 * TILE_BYTES);
        tma_load_3d(sQ + st * TILE_BYTES, &tm_q, &qd_full[st], head * ATT_D, it.x, batch);
        tma_load_3d(sQ + st * TILE_BYTES + HALF_BYTES, &tm_q, &qd_full[st], head * ATT_D + 64, it.x, batch);
        tma_load_3d(sdO + st * TILE_BYTES, &tm_do, &qd_full[st], head * ATT_D, it.x, batch);
        tma_load_3d(sdO + st * TILE_BYTES + HALF_BYTES, &tm_do, &qd_full[st], head * ATT_D + 64, it.x, batch);
      }
      if (!ok || *abort_flag) {
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 100000ull) {}
      }
    }
  } else if (warp == 9) {
    if (n_items > 0) {  // the whole warp runs the loop; one elected lane issues
      constexpr uint32_t idesc_s = make_idesc_bf16(128, DKV_BQ, 0, 0);   // 128 keys x 128 queries
      constexpr uint32_t idesc_g = make_idesc_bf16(128, 128, 0, 1);      // 128 keys x 128 d
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      // S^T of item i (needs its Q in shared memory; the buffer's last reader, dV(i-1), was
      // issued before).
      auto score_s = [&](int i) -> bool {
        const int st = i % DKV_STAGES;
        if (!mbar_wait_w(&qd_full[st], (i / DKV_STAGES) & 1, guard, kTimeoutMma)) return false;
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
      // dP^T of item i (its dO arrived with Q; the buffer's last reader, dK(i-1), was issued before).
      auto score_p = [&](int i) {
        const int st = i % DKV_STAGES;
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
        const int st = i % DKV_STAGES;
        const uint32_t q_addr = smem_u32(sQ + st * TILE_BYTES);
        const uint32_t do_addr = smem_u32(sdO + st * TILE_BYTES);
        // 16 queries per step; the packed columns of the 32 queries [32 g, 32 g + 32) start at
        // column 32 g.  The warps announce P^T in two parts (their first and their second 32
        // columns: g = c and g = 2 + c), so the first half of dV is issued while the second half
        // of the exponentials is still being computed.
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
        if (i + 1 < n_items && !score_s(i + 1)) { ok = false; break; }
        if (!mbar_wait_w(ds_ready, i & 1, guard, kTimeoutMma)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < DKV_BQ / 16; ++kk) {
          tc_mma_ts_w(tmem_base + C_DK, tmem_base + C_DPT + (kk >> 1) * 32 + (kk & 1) * 8,
                    make_smem_desc(q_addr + kk * 2048, HALF_BYTES, 1024), idesc_g, (i | kk) != 0);
        }
        tc_commit_w(&qd_empty[st]);
        if (i + 1 < n_items) score_p(i + 1);
      }
      if (ok) tc_commit_w(grad_done);
    }
  } else {
    const int quarter = warp & 3, half = warp >> 2;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const int tid = (warp << 5) + lane;      // 0..255
    const int key = quarter * 32 + lane;     // key row of this thread
    bool ok = n_items > 0;
    // Per query column the warps need -lse*log2(e) and -delta*scale.  They are staged in shared
    // memory one item ahead: the global loads of item i + 1 are issued before the work on item
    // i and stored behind it, so their latency never sits between two items.
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    const float2 ps2 = make_float2(p.scale, p.scale);
    auto fetch_stat = [&](int i) -> float {
      // threads 0..127: -lse*log2(e) (or -inf: probability 0), threads 128..255: -delta*scale
      const int2 it = items[i];
      const int head = it.y >> 8, rows = it.y & 0xff;
      const int col = tid & (DKV_BQ - 1);
      const int q = it.x + col;
      const bool valid = col < rows && q < p.nq;
      const int64_t idx = (int64_t(batch) * p.hq + head) * p.nq + q;
      if (tid < DKV_BQ) return valid ? -p.lse[idx] * LOG2E : -INFINITY;
      return valid ? -p.delta[idx] * p.scale : 0.f;
    };
    if (ok) {
      stats[tid] = fetch_stat(0);  // buffer 0: [nl[128], nd[128]]
      mbar_arrive(stats_bar);
    }
    for (int i = 0; i < n_items && ok; ++i) {
      const bool more = i + 1 < n_items;
      float next_stat = 0.f;
      if (more) next_stat = fetch_stat(i + 1);
      const float* my_stats = stats + (i & 1) * 2 * DKV_BQ + half * 64;
      if (!mbar_wait(stats_bar, i & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      if (!mbar_wait(st_full, i & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      tc_fence_after_sync();
      float2 prob[32];  // the probabilities of this thread's 64 query columns, kept for dS^T
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
          const float2 e0 = make_float2(exp2f(x0.x), exp2f(x0.y));
          const float2 e1 = make_float2(exp2f(x1.x), exp2f(x1.y));
          prob[c * 16 + 2 * k4] = e0;
          prob[c * 16 + 2 * k4 + 1] = e1;
          pp[2 * k4] = pack_bf16(e0.x, e0.y);
          pp[2 * k4 + 1] = pack_bf16(e1.x, e1.y);
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
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dv[32], dd[16];
        tmem_ld_32x32(tmem_base + lane_base + C_DPT + half * 64 + c * 32, dv);
        tmem_ld_wait();
        const float4* nd4 = reinterpret_cast<const float4*>(my_stats + DKV_BQ + c * 32);
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
          const float4 nd = nd4[k4];
          const float2 g0 = ffma2(make_float2(__uint_as_float(dv[4 * k4]), __uint_as_float(dv[4 * k4 + 1])),
                                  ps2, make_float2(nd.x, nd.y));
          const float2 g1 = ffma2(make_float2(__uint_as_float(dv[4 * k4 + 2]), __uint_as_float(dv[4 * k4 + 3])),
                                  ps2, make_float2(nd.z, nd.w));
          const float2 d0 = fmul2(prob[c * 16 + 2 * k4], g0), d1 = fmul2(prob[c * 16 + 2 * k4 + 1], g1);
          dd[2 * k4] = pack_bf16(d0.x, d0.y);
          dd[2 * k4 + 1] = pack_bf16(d1.x, d1.y);
        }
        tmem_st_32x16(tmem_base + lane_base + C_DPT + half * 64 + c * 32, dd);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
      // The other stats buffer was last read for item i - 1; every thread has passed the wait
      // of phase i above, which all threads entered only after finishing item i - 1.
      if (more) {
        stats[((i + 1) & 1) * 2 * DKV_BQ + tid] = next_stat;
        mbar_arrive(stats_bar);
      }
    }
    if (ok) ok = mbar_wait(grad_done, 0, guard, kTimeoutEpilogue);
    if (ok) {
      tc_fence_after_sync();
      const bool row_ok = key < k_rows;
      const int64_t base = ((int64_t(batch) * p.nk + k_row + key) * p.hkv + kv_head) * ATT_D;
      const int64_t base_v = int64_t(batch) * p.dv_batch_stride + int64_t(k_row + key) * p.dv_row_stride +
                             int64_t(kv_head) * ATT_D;
      {  // the two halves write one gradient each
        const int which = half;
        __nv_bfloat16* dst = which == 0 ? p.dv + base_v : p.dk + base;
        const uint32_t col0 = which == 0 ? C_DV : C_DK;
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
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

bool make_rows_map_bwd(CUtensorMap* map, const void* base, int heads, int64_t rows, int64_t batch,
                       int64_t row_stride, int64_t batch_stride, int box_rows = 128) {
  const uint64_t dims[3] = {uint64_t(heads) * ATT_D, uint64_t(rows), uint64_t(batch)};
  const uint64_t strides[2] = {uint64_t(row_stride) * 2, uint64_t(batch_stride) * 2};
  const uint32_t box[3] = {64, uint32_t(box_rows), 1};
  return make_tensor_map_bf16(map, base, 3, dims, strides, box);
}

cudaError_t attention_bwd(const AttnBwdArgs& b, cudaStream_t stream) {
  const AttnArgs& a = b.fwd;
  if (a.num_q_tiles == 0 || a.batch == 0) return cudaSuccess;
  CUtensorMap tq, tdo, tkt, tvt, tk, tv;
  const int64_t dense_row = int64_t(a.hq) * ATT_D;
  if (!make_rows_map_bwd(&tq, a.q, a.hq, a.nq, a.batch, a.q_row_stride, a.q_batch_stride) ||
      !make_rows_map_bwd(&tdo, b.grad_out, a.hq, a.nq, a.batch, dense_row, dense_row * a.nq) ||
      !make_rows_map_bwd(&tk, a.k, a.hkv, a.nk, a.batch, a.kv_row_stride, a.kv_batch_stride) ||
      !make_rows_map_bwd(&tv, a.v, a.hkv, a.nk, a.batch, a.v_row_stride ? a.v_row_stride : a.kv_row_stride,
                     a.v_row_stride ? a.v_batch_stride : a.kv_batch_stride)) {
    set_error_detail("attention_bwd: tensor map refused by the driver");
    return cudaErrorInvalidValue;
  }
  if (a.text_k) {
    if (!make_rows_map_bwd(&tkt, a.text_k, a.hkv, a.text_len, a.batch, a.text_row_stride,
                           a.text_batch_stride) ||
        !make_rows_map_bwd(&tvt, a.text_v, a.hkv, a.text_len, a.batch, a.text_row_stride,
                           a.text_batch_stride)) {
      set_error_detail("attention_bwd: text tensor map refused by the driver");
      return cudaErrorInvalidValue;
    }
  } else {
    tkt = tk;
    tvt = tv;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_dq_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               DKV_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int64_t units = a.batch * a.nq * a.hq;
  attn_delta_kernel<<<unsigned((units + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a.out), static_cast<const __nv_bfloat16*>(b.grad_out),
      b.delta, a.nq, a.hq, units);
  const float scale_log2 = a.scale * LOG2E;
  {
    DqParams p;
    p.q_tiles = a.q_tiles; p.entries = a.entries; p.text_valid = a.text_valid;
    p.lse = a.lse; p.delta = b.delta; p.dq = static_cast<__nv_bfloat16*>(b.dq);
    p.nq = int(a.nq); p.hq = a.hq; p.group = a.hq / a.hkv;
    p.nk = int(a.nk); p.text_len = int(a.text_len);
    p.scale = a.scale; p.scale_log2 = scale_log2; p.status = a.status;
    dim3 grid(a.num_q_tiles, a.hq, unsigned(a.batch));
    attn_dq_kernel<<<grid, DQ_THREADS, DQ_SMEM, stream>>>(tq, tdo, tkt, tvt, tk, tv, p);
  }
  if (b.num_k_tiles > 0) {
    DkvParams p;
    p.k_tiles = b.k_tiles; p.q_lists = b.q_lists; p.lse = a.lse; p.delta = b.delta;
    p.dk = static_cast<__nv_bfloat16*>(b.dk); p.dv = static_cast<__nv_bfloat16*>(b.dv);
    p.dv_row_stride = b.dv_row_stride ? b.dv_row_stride : int64_t(a.hkv) * ATT_D;
    p.dv_batch_stride = b.dv_row_stride ? b.dv_batch_stride : int64_t(a.nk) * a.hkv * ATT_D;
    p.nq = int(a.nq); p.nk = int(a.nk); p.hq = a.hq; p.hkv = a.hkv; p.group = a.hq / a.hkv;
    p.scale = a.scale; p.scale_log2 = scale_log2; p.status = a.status;
    dim3 grid(b.num_k_tiles, a.hkv, unsigned(a.batch));
    attn_dkv_kernel<<<grid, DQ_THREADS, DKV_SMEM, stream>>>(tq, tdo, tk, tv, p);
  }
  return cudaGetLastError();
}

}  // namespace agb
