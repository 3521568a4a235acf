// Stride-1 convolution of channels-last 16-bit float volumes as an implicit GEMM on tcgen05.
//
// The GEMM view: rows = output positions, columns = output channels, K = taps x input
// channels.  A row tile is a TH x TW patch of one output frame (TH * TW = 128).  For every tap
// (dt, dh, dw) and every block of 64 input channels the TMA producer loads the patch shifted
// by the tap straight from the 5-D tensor (C, W, H, T, B): positions outside the frame read
// as zero, which is the spatial zero padding, so no im2col buffer and no padded copy exists.
// The matching weight block [BN output channels x 64 input channels] of the same tap comes
// from the 3-D tensor (Cin, taps, Cout).  Both land in 128-byte-swizzled K-major tiles and
// feed the same pipeline as the dense GEMM of this library:
//   warp 4 (one lane)  TMA producer -> 4-stage ring
//   warp 5 (one lane)  tcgen05.mma into one of two TMEM accumulators
//   warps 0-3          epilogue: TMEM -> registers -> + bias + residual (-> ReLU) -> channels-last
// Operands and result are bf16 or fp16 (one type per call); accumulation is fp32.
// Persistent, one CTA per SM.  The innermost TMA coordinate is always a multiple of 64
// channels (128 bytes).
#include "agb.h"
#include "sm100.cuh"
#include "tensormap.h"

#include <cuda_fp16.h>

namespace agb {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int MAX_BN = 256;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + MAX_BN * BK * 2;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct Params {
  uint16_t* out;             // bf16 or fp16, like the operands
  const uint16_t* bias;
  const uint16_t* residual;
  int relu;
  int batch, frames_out, height, width, cin, cout;
  int kt, kh, kw, pad_h, pad_w;
  int lead, hist;            // implicit leading frames of a causal call; how many of them are history
  int tile_w, tile_w_shift;  // patch width (a power of two) and its log2; patch height = 128 / width
  int tiles_w, tiles_h, tiles_n;
  int bn;                    // output channels per tile, a multiple of 32
  uint32_t idesc;
  int* status;
};

// Two 16-bit floats of the activation type <-> two fp32 values.
template <bool HALF>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if (HALF) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  return make_float2(bf16_lo(w), bf16_hi(w));
}
template <bool HALF>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (HALF) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  return pack_bf16(lo, hi);
}

struct TileAt {
  int b, t, h0, w0, n0;
};

__device__ __forceinline__ TileAt decode(int tile, const Params& p) {
  TileAt at;
  at.n0 = (tile % p.tiles_n) * p.bn;
  tile /= p.tiles_n;
  at.w0 = (tile % p.tiles_w) * p.tile_w;
  tile /= p.tiles_w;
  at.h0 = (tile % p.tiles_h) * (BM >> p.tile_w_shift);
  tile /= p.tiles_h;
  at.t = tile % p.frames_out;
  at.b = tile / p.frames_out;
  return at;
}

template <bool HALF>
__global__ void __launch_bounds__(NUM_THREADS, 1)
conv3d_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
              const __grid_constant__ CUtensorMap tm_h, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
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
      mbar_init(&acc_empty[a], 4);
    }
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_h);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.batch * p.frames_out * p.tiles_h * p.tiles_w * p.tiles_n;
  const int c_blocks = (p.cin + BK - 1) / BK;
  const int taps = p.kt * p.kh * p.kw;
  const int k_blocks = taps * c_blocks;
  const uint32_t stage_tx = A_BYTES + p.bn * BK * 2;

  if (warp == 4) {
    // -------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileAt at = decode(tile, p);
        int tap = 0;
        for (int dt = 0; dt < p.kt && ok; ++dt) {
          // Frame dt of the window of output frame t.  A causal call sees `lead` implicit
          // frames before x: the last `hist` of them come from the history tensor, the ones
          // before read as zero (a coordinate in front of the tensor).
          const int frame = at.t + dt;
          const CUtensorMap* source = &tm_x;
          int frame_at = frame - p.lead;
          if (frame < p.lead) {
            if (frame >= p.lead - p.hist) {
              source = &tm_h;
              frame_at = frame - (p.lead - p.hist);
            } else {
              frame_at = -1;
            }
          }
          for (int dh = 0; dh < p.kh && ok; ++dh)
            for (int dw = 0; dw < p.kw && ok; ++dw, ++tap)
              for (int cb = 0; cb < c_blocks; ++cb) {
                if (!mbar_wait(&empty[stage], phase ^ 1, guard, kTimeoutProducer)) {
                  ok = false;
                  break;
                }
                uint8_t* sa = smem + stage * STAGE_BYTES;
                mbar_expect_tx(&full[stage], stage_tx);
                armed |= 1u << stage;
                tma_load_5d(sa, source, &full[stage], cb * BK, at.w0 + dw - p.pad_w,
                            at.h0 + dh - p.pad_h, frame_at, at.b);
                tma_load_3d(sa + A_BYTES, &tm_w, &full[stage], cb * BK, tap, at.n0);
                if (++stage == STAGES) {
                  stage = 0;
                  phase ^= 1;
                }
              }
        }
      }
      if (!ok || *abort_flag) {
        // Abort path: let this thread's copies land before the CTA's shared memory dies.
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
    // ---------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, guard, kTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * MAX_BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, guard, kTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            tc_mma_ss(d_tmem, make_smem_desc(sa + kk * 32, 16, 1024),
                      make_smem_desc(sb + kk * 32, 16, 1024), p.idesc, (kb | kk) != 0);
          tc_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------------ epilogue
    int local = 0;
    bool ok = true;
    const int r = warp * 32 + lane;
    const int hi = r >> p.tile_w_shift, wi = r & (p.tile_w - 1);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      const TileAt at = decode(tile, p);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, guard, kTimeoutEpilogue)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int h = at.h0 + hi, w = at.w0 + wi;
      const bool row_ok = h < p.height && w < p.width;
      const int64_t position = ((int64_t(at.b) * p.frames_out + at.t) * p.height + h) * p.width + w;
      uint16_t* out_row = p.out + position * p.cout;
      const uint16_t* res_row = p.residual ? p.residual + position * p.cout : nullptr;
      const uint32_t t_row = tmem_base + (uint32_t(warp * 32) << 16) + acc * MAX_BN;
#pragma unroll 1
      for (int c = 0; c < p.bn / 32; ++c) {
        const int col0 = at.n0 + c * 32;
        if (col0 >= p.cout) break;  // uniform across the CTA
        uint32_t acc_regs[32];
        tmem_ld_32x32(t_row + c * 32, acc_regs);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col >= p.cout) break;  // Cout is a multiple of 8
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc_regs[g * 8 + i]);
            if (p.bias) {
              const uint4 b = *reinterpret_cast<const uint4*>(p.bias + col);
              const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = unpack2<HALF>(bw[i]);
                v[2 * i] += f.x;
                v[2 * i + 1] += f.y;
              }
            }
            if (res_row) {
              const uint4 b = *reinterpret_cast<const uint4*>(res_row + col);
              const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = unpack2<HALF>(bw[i]);
                v[2 * i] += f.x;
                v[2 * i + 1] += f.y;
              }
            }
            if (p.relu) {
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.0f);
            }
            *reinterpret_cast<uint4*>(out_row + col) =
                make_uint4(pack2<HALF>(v[0], v[1]), pack2<HALF>(v[2], v[3]), pack2<HALF>(v[4], v[5]),
                           pack2<HALF>(v[6], v[7]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
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

// --------------------------------------------------------------------------------- host
cudaError_t conv3d_bf16(const ConvArgs& g, int sm_count, cudaStream_t stream) {
  const int lead = g.causal ? g.kt - 1 : 0;
  const int frames_out = g.frames_in + lead - g.kt + 1;
  if (g.batch <= 0 || frames_out <= 0 || g.height <= 0 || g.width <= 0) return cudaSuccess;
  if ((g.cin % 8) || (g.cout % 8) || !(g.kh & 1) || !(g.kw & 1) || g.kt < 1 ||
      (reinterpret_cast<uintptr_t>(g.x) & 15) || (reinterpret_cast<uintptr_t>(g.weight) & 15) ||
      (reinterpret_cast<uintptr_t>(g.out) & 15) || (reinterpret_cast<uintptr_t>(g.bias) & 15) ||
      (reinterpret_cast<uintptr_t>(g.residual) & 15)) {
    set_error_detail("conv3d: channels must be multiples of 8, spatial kernel sizes odd, pointers 16-byte aligned");
    return cudaErrorInvalidValue;
  }
  if (g.history_frames < 0 || g.history_frames > lead || (g.history_frames > 0 && !g.history) ||
      (reinterpret_cast<uintptr_t>(g.history) & 15)) {
    set_error_detail("conv3d: history holds at most kt - 1 frames of a causal call");
    return cudaErrorInvalidValue;
  }

  Params p{};
  // Patch shape: the power-of-two width whose 128-position patches waste the fewest positions.
  int64_t best = -1;
  for (int shift = 3; shift <= 7; ++shift) {
    const int tw = 1 << shift, th = BM / tw;
    const int64_t covered = int64_t((g.width + tw - 1) / tw) * tw * ((g.height + th - 1) / th) * th;
    if (best < 0 || covered < best) {
      best = covered;
      p.tile_w = tw;
      p.tile_w_shift = shift;
    }
  }
  const int tile_h = BM / p.tile_w;
  p.tiles_w = (g.width + p.tile_w - 1) / p.tile_w;
  p.tiles_h = (g.height + tile_h - 1) / tile_h;
  // Output channels per tile: a multiple of 32, at most 256, with the least padding.
  {
    int best_pad = 1 << 30;
    const int least = (g.cout + MAX_BN - 1) / MAX_BN;
    for (int tiles = least; tiles <= least + 3; ++tiles) {
      const int bn = (((g.cout + tiles - 1) / tiles) + 31) / 32 * 32;
      if (bn > MAX_BN) continue;
      const int pad = bn * tiles - g.cout;
      if (pad < best_pad) {
        best_pad = pad;
        p.tiles_n = tiles;
        p.bn = bn;
      }
    }
  }
  const int64_t tiles = int64_t(g.batch) * frames_out * p.tiles_h * p.tiles_w * p.tiles_n;
  if (tiles > (int64_t(1) << 30)) {
    set_error_detail("conv3d: too many output tiles for one launch");
    return cudaErrorInvalidValue;
  }

  CUtensorMap tx, tw, th;
  {
    const uint64_t dims[5] = {uint64_t(g.cin), uint64_t(g.width), uint64_t(g.height),
                              uint64_t(g.frames_in), uint64_t(g.batch)};
    const uint64_t c = uint64_t(g.cin) * 2;
    const uint64_t strides[4] = {c, c * g.width, c * g.width * g.height,
                                 c * g.width * g.height * g.frames_in};
    const uint32_t box[5] = {64, uint32_t(p.tile_w), uint32_t(tile_h), 1, 1};
    if (!make_tensor_map_bf16(&tx, g.x, 5, dims, strides, box)) return cudaErrorInvalidValue;
    th = tx;
    if (g.history_frames > 0) {
      const uint64_t hdims[5] = {dims[0], dims[1], dims[2], uint64_t(g.history_frames), dims[4]};
      const uint64_t hstrides[4] = {c, c * g.width, c * g.width * g.height,
                                    c * g.width * g.height * g.history_frames};
      if (!make_tensor_map_bf16(&th, g.history, 5, hdims, hstrides, box)) return cudaErrorInvalidValue;
    }
  }
  {
    const int taps = g.kt * g.kh * g.kw;
    const uint64_t dims[3] = {uint64_t(g.cin), uint64_t(taps), uint64_t(g.cout)};
    const uint64_t strides[2] = {uint64_t(g.cin) * 2, uint64_t(g.cin) * 2 * taps};
    const uint32_t box[3] = {64, 1, uint32_t(p.bn)};
    if (!make_tensor_map_bf16(&tw, g.weight, 3, dims, strides, box)) return cudaErrorInvalidValue;
  }

  p.out = static_cast<uint16_t*>(g.out);
  p.bias = static_cast<const uint16_t*>(g.bias);
  p.residual = static_cast<const uint16_t*>(g.residual);
  p.relu = g.relu;
  p.batch = g.batch;
  p.frames_out = frames_out;
  p.height = g.height;
  p.width = g.width;
  p.cin = g.cin;
  p.cout = g.cout;
  p.kt = g.kt;
  p.kh = g.kh;
  p.kw = g.kw;
  p.pad_h = g.kh / 2;
  p.pad_w = g.kw / 2;
  p.lead = lead;
  p.hist = g.history_frames;
  // fp16 operands: the A and B format fields of the descriptor are 0 instead of 1 (bf16)
  p.idesc = make_idesc_bf16(BM, p.bn, 0, 0) & (g.fp16 ? ~((1u << 7) | (1u << 10)) : ~0u);
  p.status = g.status;

  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(conv3d_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(conv3d_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               SMEM_BYTES);
    if (e != cudaSuccess) {
      set_error_detail("conv3d: cudaFuncSetAttribute(max dynamic shared memory) failed");
      return e;
    }
    configured = true;
  }
  (void)cudaGetLastError();
  const int grid = tiles < sm_count ? int(tiles) : sm_count;
  if (g.fp16)
    conv3d_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tx, tw, th, p);
  else
    conv3d_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tx, tw, th, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_error_detail("conv3d: kernel launch failed");
  return e;
}

}  // namespace agb
