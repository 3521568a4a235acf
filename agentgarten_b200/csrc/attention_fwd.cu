// Flash-attention forward on tcgen05 for head_dim 128 with grouped KV heads and
// segment-list keys (text prefix with per-sample valid length + visual segments).
//
// One CTA per (query tile of 128 rows, PAIR of query heads that share a KV head, sample):
//   warps 0-3  softmax of head A: one query row per thread
//   warps 4-7  softmax of head B
//   warp 8     TMA producer: both Q tiles once, then K and V tiles through 2-stage rings
//   warp 9     MMA issuer:   S_h = Q_h K^T (operands in shared memory) and O_h += P_h V with
//              P_h read from TMEM, for h = A, B, all accumulating in TMEM
// Every K and V tile that reaches shared memory is used by two heads, which halves the
// traffic from L2 per FLOP (the single-head kernel ran at the L2 bandwidth limit), and while
// one head is in its softmax (exponentials on the special-function unit, conversion,
// packing) the tensor core serves the other.  The probabilities overwrite the first half of
// the head's score buffer; tcgen05.mma operations of one thread execute in issue order, so
// the next scores of a head are issued right behind the product that reads its
// probabilities, without a round trip through a barrier.  The running output stays in TMEM
// and is rescaled lazily: only when a row maximum grows by more than 2^8 does a warp
// rescale its 32 rows.  With an odd number of query heads per KV head the CTA serves one
// head and the second group idles.
//
// TMEM columns: S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512); P_h = S_h[0,64).
#include "agb.h"
#include "attention_common.cuh"
#include "tensormap.h"

namespace agb {
namespace {

constexpr int KV_STAGES = 2;
constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KiB: a 128x128 bf16 tile (2 atoms of 16 KiB)
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int FWD_THREADS = 320;
constexpr int SMEM_TILES = 2 + 2 * KV_STAGES;  // Q_A, Q_B + K ring + V ring
constexpr int FWD_SMEM = SMEM_TILES * TILE_BYTES + ATT_MAX_TILES * int(sizeof(KeyTile)) + 1024 + 512;

constexpr uint32_t COL_S = 0, COL_O = 256;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

struct FwdParams {
  const int* q_tiles;     // [tiles, 5]: q_row, rows, first_entry, entries, q_local
  const int* entries;     // [*, 3]
  const int* text_valid;  // [B] or null
  __nv_bfloat16* out;     // [B, NQ, Hq, 128]
  float* lse;             // [B, Hq, NQ] natural-log LSE
  int nq, hq, group;      // group = Hq / Hkv
  int nk, text_len;       // extents the work lists are checked against
  int heads_per_cta;      // 2 when group is even, else 1
  int base_tiles;         // query tiles of one key split: tile t belongs to split t / base_tiles
  int out_rows;           // rows of out / lse per sample (= splits * nq); split s writes rows s*nq + q
  float scale_log2;       // softmax scale * log2(e)
  int* status;
};

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kt,
                const __grid_constant__ CUtensorMap tm_vt, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;                          // [2] tiles
  uint8_t* sK = smem + 2 * TILE_BYTES;
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
  KeyTile* tiles = reinterpret_cast<KeyTile*>(sV + KV_STAGES * TILE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + ATT_MAX_TILES);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2 heads] MMA -> softmax: scores of the next tile complete
  uint64_t* p_ready = bars + 11;      // [2 heads] softmax -> MMA: probabilities in TMEM
  uint64_t* o_done = bars + 13;       // [2 heads] MMA -> softmax: last product complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* n_tiles_smem = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.heads_per_cta;
  const int head0 = blockIdx.y * heads;
  const int batch = blockIdx.z;
  const int kv_head = head0 / p.group;
  const int* qt = p.q_tiles + 5 * blockIdx.x;
  const int q_row = qt[0], q_rows = qt[1], q_local = qt[4];
  const int out_row = q_row + (int(blockIdx.x) / p.base_tiles) * p.nq;
  const WaitGuard guard{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_done[i], 1);
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
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int n_tiles = *n_tiles_smem;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(q_full, heads * TILE_BYTES);
      for (int h = 0; h < heads; ++h) {
        tma_load_3d(sQ + h * TILE_BYTES, &tm_q, q_full, (head0 + h) * ATT_D, q_row, batch);
        tma_load_3d(sQ + h * TILE_BYTES + HALF_BYTES, &tm_q, q_full, (head0 + h) * ATT_D + 64, q_row, batch);
      }
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const KeyTile t = tiles[j];
        const CUtensorMap* mk = t.source == 0 ? &tm_kt : &tm_k;
        const CUtensorMap* mv = t.source == 0 ? &tm_vt : &tm_v;
        if (!mbar_wait(&k_empty[st], ph ^ 1, guard, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], TILE_BYTES);
        tma_load_3d(sK + st * TILE_BYTES, mk, &k_full[st], kv_head * ATT_D, t.row, batch);
        tma_load_3d(sK + st * TILE_BYTES + HALF_BYTES, mk, &k_full[st], kv_head * ATT_D + 64, t.row, batch);
        if (!mbar_wait(&v_empty[st], ph ^ 1, guard, kTimeoutProducer)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], TILE_BYTES);
        tma_load_3d(sV + st * TILE_BYTES, mv, &v_full[st], kv_head * ATT_D, t.row, batch);
        tma_load_3d(sV + st * TILE_BYTES + HALF_BYTES, mv, &v_full[st], kv_head * ATT_D + 64, t.row, batch);
      }
      if (!ok || *abort_flag) {
        // give in-flight copies time to land before shared memory is released
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 100000ull) {}
      }
    }
  } else if (warp == 9) {
    // -------------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_tiles > 0) {
      // S = Q K^T: both K-major, 8 k-steps of 16 over d = 128 (two 64-wide atoms).
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      // O += P V: A = P from TMEM (K-major), B = V MN-major (d contiguous), 8 k-steps over keys.
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, 0, 1);
      auto scores = [&](int h, int j) {
        const uint32_t q_addr = smem_u32(sQ + h * TILE_BYTES);
        const uint32_t k_addr = smem_u32(sK + (j % KV_STAGES) * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
          tc_mma_ss(tmem_base + COL_S + h * 128, make_smem_desc(q_addr + off, 16, 1024),
                    make_smem_desc(k_addr + off, 16, 1024), idesc_s, kk != 0);
        }
        tc_commit(&s_full[h]);
      };
      bool ok = mbar_wait(q_full, 0, guard, kTimeoutMma) &&
                mbar_wait(&k_full[0], 0, guard, kTimeoutMma);
      if (ok) {
        tc_fence_after_sync();
        for (int h = 0; h < heads; ++h) scores(h, 0);
        tc_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % KV_STAGES;
        const bool more = j + 1 < n_tiles;
        if (!mbar_wait(&v_full[st], (j / KV_STAGES) & 1, guard, kTimeoutMma)) { ok = false; break; }
        if (more && !mbar_wait(&k_full[(j + 1) % KV_STAGES], ((j + 1) / KV_STAGES) & 1, guard,
                               kTimeoutMma)) { ok = false; break; }
        const uint32_t v_addr = smem_u32(sV + st * TILE_BYTES);
        for (int h = 0; h < heads && ok; ++h) {
          if (!mbar_wait(&p_ready[h], j & 1, guard, kTimeoutMma)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            // 16 keys per step: P advances 8 packed columns, V advances 16 rows (2048 B).
            tc_mma_ts(tmem_base + COL_O + h * 128, tmem_base + COL_S + h * 128 + kk * 8,
                      make_smem_desc(v_addr + kk * 2048, HALF_BYTES, 1024), idesc_o, (j | kk) != 0);
          }
          // Issued behind the product above, which reads P from the buffer these scores refill:
          // the tensor core executes one thread's operations in issue order.
          if (more) scores(h, j + 1);
          else tc_commit(&o_done[h]);
        }
        if (!ok) break;
        tc_commit(&v_empty[st]);
        if (more) tc_commit(&k_empty[(j + 1) % KV_STAGES]);
      }
    }
  } else if ((warp >> 2) < heads) {
    // ----------------------------------------------------------------------- softmax
    const int h = warp >> 2;                     // which head of the pair
    const int head = head0 + h;
    const int quarter = warp & 3;                // TMEM lanes 32*quarter .. +31
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const int my_row = quarter * 32 + lane;      // row within the query tile
    const uint32_t col_s = tmem_base + lane_base + COL_S + h * 128;
    const uint32_t col_o = tmem_base + lane_base + COL_O + h * 128;
    float m_ref = -INFINITY;                     // reference maximum (log2 domain)
    float l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const KeyTile t = tiles[j];
      if (!mbar_wait(&s_full[h], j & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(col_s + c * 32, s[c]);
      tmem_ld_wait();

      // Row maximum of the raw scores (the scale is positive).  Only tiles with masked keys
      // (a partial last tile, the causal diagonal) pay for the masking.
      float m_raw = -INFINITY;
      if (t.valid == ATT_BN && t.causal0 < 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            m_raw = fmax3(m_raw, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
      } else {
        int valid = t.valid;
        if (t.causal0 >= 0) valid = min(valid, q_local + my_row + 1 - t.causal0);
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = (c * 32 + i < valid) ? __uint_as_float(s[c][i]) : -INFINITY;
            s[c][i] = __float_as_uint(v);
            m_raw = fmaxf(m_raw, v);
          }
      }
      const float m_tile = m_raw * p.scale_log2;
      // Lazy rescale, decided per warp so that the TMEM accesses stay warp-uniform.  The
      // previous product of this head is complete: these scores were executed after it.
      const bool grow = m_tile > m_ref + RESCALE_THRESHOLD;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(col_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(col_o + c * 32, o);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_ref = m_new;
      }
      // exp2(s * scale - m): one two-lane FMA per pair of keys, then the exponentials.  A
      // fully masked row keeps m_ref = -inf: its scores are -inf and the shift is 0.
      const float shift = (m_ref == -INFINITY) ? 0.f : m_ref;
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 shift2 = make_float2(-shift, -shift);
      float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          // columns (2i, 2i+1) of the 64-key half c
          const uint32_t* src = &s[2 * c + (i >> 4)][(2 * i) & 31];
          const float2 x = ffma2(make_float2(__uint_as_float(src[0]), __uint_as_float(src[1])),
                                 scale2, shift2);
          const float2 e = make_float2(exp2f(x.x), exp2f(x.y));
          sum2 = fadd2(sum2, e);
          packed[i] = pack_bf16(e.x, e.y);
        }
        tmem_st_32x32(col_s + c * 32, packed);  // over the scores, which are in registers
      }
      l_sum += sum2.x + sum2.y;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[h]);
    }
    // ---------------------------------------------------------------------- epilogue
    if (ok && n_tiles > 0) ok = mbar_wait(&o_done[h], 0, guard, kTimeoutEpilogue);
    if (ok) {
      tc_fence_after_sync();
      const float inv = (l_sum > 0.f) ? 1.f / l_sum : 0.f;
      const bool row_ok = my_row < q_rows;
      __nv_bfloat16* dst =
          p.out + ((int64_t(batch) * p.out_rows + out_row + my_row) * p.hq + head) * ATT_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(col_o + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[g * 8 + 0]) * inv, __uint_as_float(o[g * 8 + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = v;
          }
        }
      }
      if (row_ok && p.lse) {
        const float lse = (l_sum > 0.f) ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
        p.lse[(int64_t(batch) * p.hq + head) * p.out_rows + out_row + my_row] = lse;
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

bool make_rows_map(CUtensorMap* map, const void* base, int heads, int64_t rows, int64_t batch,
                   int64_t row_stride, int64_t batch_stride) {
  // dims (head*128 contiguous, rows, batch); box = 64 columns x 128 rows.
  const uint64_t dims[3] = {uint64_t(heads) * ATT_D, uint64_t(rows), uint64_t(batch)};
  const uint64_t strides[2] = {uint64_t(row_stride) * 2, uint64_t(batch_stride) * 2};
  const uint32_t box[3] = {64, 128, 1};
  return make_tensor_map_bf16(map, base, 3, dims, strides, box);
}

cudaError_t attention_fwd(const AttnArgs& a, cudaStream_t stream) {
  if (a.num_q_tiles == 0 || a.batch == 0) return cudaSuccess;
  CUtensorMap tq, tkt, tvt, tk, tv;
  if (!make_rows_map(&tq, a.q, a.hq, a.nq, a.batch, a.q_row_stride, a.q_batch_stride) ||
      !make_rows_map(&tk, a.k, a.hkv, a.nk, a.batch, a.kv_row_stride, a.kv_batch_stride) ||
      !make_rows_map(&tv, a.v, a.hkv, a.nk, a.batch, a.v_row_stride ? a.v_row_stride : a.kv_row_stride,
                     a.v_row_stride ? a.v_batch_stride : a.kv_batch_stride))
    return cudaErrorInvalidValue;
  if (a.text_k) {
    if (!make_rows_map(&tkt, a.text_k, a.hkv, a.text_len, a.batch, a.text_row_stride,
                       a.text_batch_stride) ||
        !make_rows_map(&tvt, a.text_v, a.hkv, a.text_len, a.batch, a.text_row_stride,
                       a.text_batch_stride))
      return cudaErrorInvalidValue;
  } else {
    tkt = tk;
    tvt = tv;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  FwdParams p;
  p.q_tiles = a.q_tiles;
  p.entries = a.entries;
  p.text_valid = a.text_valid;
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.lse = a.lse;
  p.nq = int(a.nq);
  p.nk = int(a.nk);
  p.text_len = int(a.text_len);
  p.hq = a.hq;
  p.group = a.hq / a.hkv;
  p.heads_per_cta = (p.group % 2 == 0) ? 2 : 1;
  p.base_tiles = a.key_splits > 1 ? a.num_q_tiles / a.key_splits : a.num_q_tiles;
  p.out_rows = int(a.nq) * (a.key_splits > 1 ? a.key_splits : 1);
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.status = a.status;
  dim3 grid(a.num_q_tiles, a.hq / p.heads_per_cta, unsigned(a.batch));
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, stream>>>(tq, tkt, tvt, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace agb
