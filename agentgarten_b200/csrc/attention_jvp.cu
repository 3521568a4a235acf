// Flash attention with forward-mode tangents on tcgen05 (head_dim 128, grouped KV heads).
//
// For q, k, v and tangents tq, tk, tv (all bf16) one pass over the keys produces
//   O  = softmax(q k^T * scale) v
//   tO = sum_j P_ij (tS_ij - mu_i) v_j + sum_j P_ij tv_j,   tS = (tq k^T + q tk^T) * scale,
//        mu_i = sum_j P_ij tS_ij
// and the log-sum-exp.  Per tile of 64 keys the tensor core runs six products:
//   S  = Q K^T                     T  = tQ K^T + Q tK^T          (operands in shared memory)
//   O += P V                       A += W V + P tV,  W = P o T   (P, W read from TMEM)
// and the softmax warps keep, per row, the running maximum, l = sum P and r = sum W; at the
// end O/l and A/l - (O/l)(r/l) are written in fp32.
//
// One CTA per (128 query rows, query head, sample): warps 0-3 softmax (a row per thread),
// warp 4 TMA producer, warp 5 MMA issuer.  S and T are double buffered (the next tile's
// scores are computed while the softmax works); P and W overwrite the first 32 columns of
// their own S and T buffer, which the tensor core may refill only after the products that
// read them have completed.
//
// TMEM columns: S0 [0,64) S1 [64,128) T0 [128,192) T1 [192,256) O [256,384) A [384,512).
// Keys: optional text prefix [0, text_len) of which the first text_valid[b] are visible,
// everything after it visible; rows past nk are masked.
#include "agb.h"
#include "attention_common.cuh"
#include "tensormap.h"

namespace agb {
bool make_rows_map(CUtensorMap* map, const void* base, int heads, int64_t rows, int64_t batch,
                   int64_t row_stride, int64_t batch_stride);
namespace {

constexpr int JBN = 64;                      // keys per tile
constexpr int Q_BYTES = 128 * 128 * 2;       // 32 KiB, two atoms of 16 KiB
constexpr int Q_HALF = Q_BYTES / 2;
constexpr int K_BYTES = JBN * 128 * 2;       // 16 KiB, two atoms of 8 KiB
constexpr int K_HALF = K_BYTES / 2;
constexpr int JSTAGES = 2;
constexpr int JVP_THREADS = 192;
constexpr int JVP_SMEM = 2 * Q_BYTES + 4 * JSTAGES * K_BYTES + 1024 + 512;
constexpr uint32_t CS = 0, CT = 128, CO = 256, CA = 384;
constexpr float RESCALE = 8.0f;

struct JvpParams {
  float* out;       // [B, NQ, Hq, 128]
  float* tangent;   // [B, NQ, Hq, 128]
  float* lse;       // [B, Hq, NQ] or null
  const int* text_valid;
  int nq, nk, hq, group, text_len;
  float scale, scale_log2;
  int* status;
};

bool make_key_map(CUtensorMap* map, const void* base, int heads, int64_t rows, int64_t batch,
                  int64_t row_stride, int64_t batch_stride) {
  const uint64_t dims[3] = {uint64_t(heads) * ATT_D, uint64_t(rows), uint64_t(batch)};
  const uint64_t strides[2] = {uint64_t(row_stride) * 2, uint64_t(batch_stride) * 2};
  const uint32_t box[3] = {64, JBN, 1};
  return make_tensor_map_bf16(map, base, 3, dims, strides, box);
}

__global__ void __launch_bounds__(JVP_THREADS, 1)
attn_jvp_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_tq,
                const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_tk,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_tv,
                const JvpParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sTQ = sQ + Q_BYTES;
  uint8_t* sK = sTQ + Q_BYTES;                 // [stage][K | tK]
  uint8_t* sV = sK + 2 * JSTAGES * K_BYTES;    // [stage][V | tV]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * JSTAGES * K_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2] MMA -> softmax: S and T of the buffer are complete
  uint64_t* p_ready = bars + 11;    // [2] softmax -> MMA: P and W are in TMEM
  uint64_t* pv_done = bars + 13;    // [2] MMA -> softmax/MMA: products of the buffer completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / p.group;
  const int q_row = blockIdx.x * ATT_BM;
  const int n_tiles = (p.nk + JBN - 1) / JBN;
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
      mbar_init(&pv_done[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(q_full, 2 * Q_BYTES);
      tma_load_3d(sQ, &tm_q, q_full, head * ATT_D, q_row, batch);
      tma_load_3d(sQ + Q_HALF, &tm_q, q_full, head * ATT_D + 64, q_row, batch);
      tma_load_3d(sTQ, &tm_tq, q_full, head * ATT_D, q_row, batch);
      tma_load_3d(sTQ + Q_HALF, &tm_tq, q_full, head * ATT_D + 64, q_row, batch);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % JSTAGES;
        const uint32_t ph = (j / JSTAGES) & 1;
        const int row = j * JBN;
        const int x = kv_head * ATT_D;
        if (!mbar_wait(&k_empty[st], ph ^ 1, guard, kTimeoutProducer)) { ok = false; break; }
        uint8_t* k = sK + st * 2 * K_BYTES;
        mbar_expect_tx(&k_full[st], 2 * K_BYTES);
        tma_load_3d(k, &tm_k, &k_full[st], x, row, batch);
        tma_load_3d(k + K_HALF, &tm_k, &k_full[st], x + 64, row, batch);
        tma_load_3d(k + K_BYTES, &tm_tk, &k_full[st], x, row, batch);
        tma_load_3d(k + K_BYTES + K_HALF, &tm_tk, &k_full[st], x + 64, row, batch);
        if (!mbar_wait(&v_empty[st], ph ^ 1, guard, kTimeoutProducer)) { ok = false; break; }
        uint8_t* v = sV + st * 2 * K_BYTES;
        mbar_expect_tx(&v_full[st], 2 * K_BYTES);
        tma_load_3d(v, &tm_v, &v_full[st], x, row, batch);
        tma_load_3d(v + K_HALF, &tm_v, &v_full[st], x + 64, row, batch);
        tma_load_3d(v + K_BYTES, &tm_tv, &v_full[st], x, row, batch);
        tma_load_3d(v + K_BYTES + K_HALF, &tm_tv, &v_full[st], x + 64, row, batch);
      }
      if (!ok || *abort_flag) {
        const uint64_t start = global_timer_ns();  // let copies in flight land
        while (global_timer_ns() - start < 100000ull) {}
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------------- MMA issuer
    if (n_tiles > 0) {  // the whole warp runs the loop; one elected lane issues
      constexpr uint32_t idesc_s = make_idesc_bf16(128, JBN, 0, 0);   // both K-major over d
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, 0, 1);   // P from TMEM, V MN-major
      const uint32_t q_addr = smem_u32(sQ), tq_addr = smem_u32(sTQ);
      bool ok = mbar_wait_w(q_full, 0, guard, kTimeoutMma);
      auto scores = [&](int j) -> bool {
        const int st = j % JSTAGES, buf = j & 1;
        if (!mbar_wait_w(&k_full[st], (j / JSTAGES) & 1, guard, kTimeoutMma)) return false;
        // P and W of tile j-2 live in this buffer until their products have completed.
        if (j >= 2 && !mbar_wait_w(&pv_done[buf], ((j - 2) >> 1) & 1, guard, kTimeoutMma)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(sK + st * 2 * K_BYTES);
        const uint32_t tk_addr = k_addr + K_BYTES;
        const uint32_t s_col = tmem_base + CS + buf * JBN, t_col = tmem_base + CT + buf * JBN;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t qo = (kk >> 2) * Q_HALF + (kk & 3) * 32;
          const uint32_t ko = (kk >> 2) * K_HALF + (kk & 3) * 32;
          tc_mma_ss_w(s_col, make_smem_desc(q_addr + qo, 16, 1024), make_smem_desc(k_addr + ko, 16, 1024),
                    idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t qo = (kk >> 2) * Q_HALF + (kk & 3) * 32;
          const uint32_t ko = (kk >> 2) * K_HALF + (kk & 3) * 32;
          tc_mma_ss_w(t_col, make_smem_desc(tq_addr + qo, 16, 1024), make_smem_desc(k_addr + ko, 16, 1024),
                    idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t qo = (kk >> 2) * Q_HALF + (kk & 3) * 32;
          const uint32_t ko = (kk >> 2) * K_HALF + (kk & 3) * 32;
          tc_mma_ss_w(t_col, make_smem_desc(q_addr + qo, 16, 1024), make_smem_desc(tk_addr + ko, 16, 1024),
                    idesc_s, true);
        }
        tc_commit_w(&k_empty[st]);
        tc_commit_w(&s_full[buf]);
        return true;
      };
      if (ok) ok = scores(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles && !scores(j + 1)) { ok = false; break; }
        const int st = j % JSTAGES, buf = j & 1;
        if (!mbar_wait_w(&v_full[st], (j / JSTAGES) & 1, guard, kTimeoutMma)) { ok = false; break; }
        if (!mbar_wait_w(&p_ready[buf], (j >> 1) & 1, guard, kTimeoutMma)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(sV + st * 2 * K_BYTES);
        const uint32_t tv_addr = v_addr + K_BYTES;
        const uint32_t p_col = tmem_base + CS + buf * JBN, w_col = tmem_base + CT + buf * JBN;
#pragma unroll
        for (int kk = 0; kk < JBN / 16; ++kk)  // 16 keys per step: 8 packed columns, 16 V rows
          tc_mma_ts_w(tmem_base + CO, p_col + kk * 8, make_smem_desc(v_addr + kk * 2048, K_HALF, 1024),
                    idesc_o, (j | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < JBN / 16; ++kk)
          tc_mma_ts_w(tmem_base + CA, w_col + kk * 8, make_smem_desc(v_addr + kk * 2048, K_HALF, 1024),
                    idesc_o, (j | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < JBN / 16; ++kk)
          tc_mma_ts_w(tmem_base + CA, p_col + kk * 8, make_smem_desc(tv_addr + kk * 2048, K_HALF, 1024),
                    idesc_o, true);
        tc_commit_w(&v_empty[st]);
        tc_commit_w(&pv_done[buf]);
      }
    }
  } else {
    // ----------------------------------------------------------------------- softmax
    const uint32_t lane_base = uint32_t(warp * 32) << 16;
    const int my_row = warp * 32 + lane;
    const int visible_text = p.text_valid ? min(p.text_len, p.text_valid[batch]) : p.text_len;
    float m_ref = -INFINITY, l_sum = 0.f, r_sum = 0.f;
    bool ok = n_tiles > 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int buf = j & 1;
      if (!mbar_wait(&s_full[buf], (j >> 1) & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s[2][32], t[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tmem_ld_32x32(tmem_base + lane_base + CS + buf * JBN + c * 32, s[c]);
        tmem_ld_32x32(tmem_base + lane_base + CT + buf * JBN + c * 32, t[c]);
      }
      tmem_ld_wait();
      float m_tile = -INFINITY;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = j * JBN + c * 32 + i;
          const bool seen = key < p.nk && (key >= p.text_len || key < visible_text);
          const float v = seen ? __uint_as_float(s[c][i]) * p.scale_log2 : -INFINITY;
          s[c][i] = __float_as_uint(v);
          m_tile = fmaxf(m_tile, v);
        }
      const bool grow = m_tile > m_ref + RESCALE;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
        if (j > 0) {
          if (!mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, guard, kTimeoutSoftmax)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {  // O then A: 256 consecutive columns
            uint32_t o[32];
            tmem_ld_32x32(tmem_base + lane_base + CO + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_base + lane_base + CO + c * 32, o);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        r_sum *= alpha;
        m_ref = m_new;
      }
      const float shift = (m_ref == -INFINITY) ? 0.f : m_ref;
      uint32_t pp[32], ww[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int c = i >> 4, e = (2 * i) & 31;
        const float a = exp2f(__uint_as_float(s[c][e]) - shift);
        const float b = exp2f(__uint_as_float(s[c][e + 1]) - shift);
        const float wa = a * (__uint_as_float(t[c][e]) * p.scale);
        const float wb = b * (__uint_as_float(t[c][e + 1]) * p.scale);
        l_sum += a + b;
        r_sum += wa + wb;
        pp[i] = pack_bf16(a, b);
        ww[i] = pack_bf16(wa, wb);
      }
      // S and T of this buffer are in registers: their first 32 columns become P and W.
      tmem_st_32x32(tmem_base + lane_base + CS + buf * JBN, pp);
      tmem_st_32x32(tmem_base + lane_base + CT + buf * JBN, ww);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[buf]);
    }
    // ---------------------------------------------------------------------- epilogue
    if (ok) {
      const int last = n_tiles - 1;
      ok = mbar_wait(&pv_done[last & 1], (last >> 1) & 1, guard, kTimeoutEpilogue);
    }
    if (n_tiles == 0 || ok) {
      tc_fence_after_sync();
      const float inv = (l_sum > 0.f) ? 1.f / l_sum : 0.f;
      const float mu = r_sum * inv;
      const bool row_ok = q_row + my_row < p.nq;
      const int64_t at = ((int64_t(batch) * p.nq + q_row + my_row) * p.hq + head) * ATT_D;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32], a[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem_base + lane_base + CO + c * 32, o);
          tmem_ld_32x32(tmem_base + lane_base + CA + c * 32, a);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = a[i] = 0;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 ov, tv;
            float* op = reinterpret_cast<float*>(&ov);
            float* tp = reinterpret_cast<float*>(&tv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float value = __uint_as_float(o[g * 4 + i]) * inv;
              op[i] = value;
              tp[i] = __uint_as_float(a[g * 4 + i]) * inv - value * mu;
            }
            *reinterpret_cast<float4*>(p.out + at + c * 32 + g * 4) = ov;
            *reinterpret_cast<float4*>(p.tangent + at + c * 32 + g * 4) = tv;
          }
        }
      }
      if (row_ok && p.lse) {
        const float lse = (l_sum > 0.f) ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
        p.lse[(int64_t(batch) * p.hq + head) * p.nq + q_row + my_row] = lse;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

cudaError_t attention_jvp(const AttnJvpArgs& a, cudaStream_t stream) {
  if (a.batch == 0 || a.nq == 0) return cudaSuccess;
  if (a.hq % a.hkv || a.nk <= 0) {
    set_error_detail("attention_jvp: heads must group evenly and there must be keys");
    return cudaErrorInvalidValue;
  }
  CUtensorMap tq, ttq, tk, ttk, tv, ttv;
  if (!make_rows_map(&tq, a.q, a.hq, a.nq, a.batch, a.q_row_stride, a.q_batch_stride) ||
      !make_rows_map(&ttq, a.tq, a.hq, a.nq, a.batch, a.q_row_stride, a.q_batch_stride) ||
      !make_key_map(&tk, a.k, a.hkv, a.nk, a.batch, a.kv_row_stride, a.kv_batch_stride) ||
      !make_key_map(&ttk, a.tk, a.hkv, a.nk, a.batch, a.kv_row_stride, a.kv_batch_stride) ||
      !make_key_map(&tv, a.v, a.hkv, a.nk, a.batch, a.kv_row_stride, a.kv_batch_stride) ||
      !make_key_map(&ttv, a.tv, a.hkv, a.nk, a.batch, a.kv_row_stride, a.kv_batch_stride))
    return cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_jvp_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, JVP_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  JvpParams p;
  p.out = a.out;
  p.tangent = a.tangent;
  p.lse = a.lse;
  p.text_valid = a.text_valid;
  p.nq = int(a.nq);
  p.nk = int(a.nk);
  p.hq = a.hq;
  p.group = a.hq / a.hkv;
  p.text_len = int(a.text_len);
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.status = a.status;
  dim3 grid(unsigned((a.nq + ATT_BM - 1) / ATT_BM), a.hq, unsigned(a.batch));
  (void)cudaGetLastError();
  attn_jvp_kernel<<<grid, JVP_THREADS, JVP_SMEM, stream>>>(tq, ttq, tk, ttk, tv, ttv, p);
  return cudaGetLastError();
}

}  // namespace agb
