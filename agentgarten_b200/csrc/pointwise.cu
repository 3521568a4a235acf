// Row-wise and element-wise kernels of the transformer layers (all HBM-bound):
// RMSNorm (optionally fused with the residual add) forward/backward, per-head RMSNorm +
// rotate-half RoPE forward/backward, SiLU*mul forward/backward, rectified-flow combine.
//
// Rounding contract: statistics in fp32; a value is rounded to bf16 wherever an eager bf16
// program would store it (normalised value, weight product, each rotary product, sums).
#include "agb.h"
#include "sm100.cuh"

namespace agb {
namespace {

constexpr int NT = 256;  // threads per CTA of the row kernels

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) total += scratch[w];
  return total;
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

// ------------------------------------------------------------------------ RMSNorm fwd
// One CTA per row.  With `addend`, total = bf16(x + addend) is stored and normalised.
template <bool ADD>
__global__ void __launch_bounds__(NT) rms_norm_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ addend,
    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ total_out,
    __nv_bfloat16* __restrict__ out, float* __restrict__ rstd_out, int width, float eps) {
  __shared__ float scratch[NT / 32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * width;
  float sumsq = 0.f;
  for (int c = threadIdx.x * 8; c < width; c += NT * 8) {
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
    if (ADD) {
      float a[8];
      unpack8(*reinterpret_cast<const uint4*>(addend + row * width + c), a);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = round_bf16(v[i] + a[i]);
      *reinterpret_cast<uint4*>(total_out + row * width + c) = pack8(v);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sumsq += v[i] * v[i];
  }
  const float rstd = rsqrtf(block_sum(sumsq, scratch) / float(width) + eps);
  if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
  const __nv_bfloat16* src = ADD ? total_out + row * width : xr;
  for (int c = threadIdx.x * 8; c < width; c += NT * 8) {
    float v[8], g[8];
    unpack8(*reinterpret_cast<const uint4*>(src + c), v);
    unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = g[i] * round_bf16(v[i] * rstd);
    *reinterpret_cast<uint4*>(out + row * width + c) = pack8(v);
  }
}

// ------------------------------------------------------------------------ RMSNorm bwd
// Each CTA walks ROWS_PER_CTA rows; dx per row, dw partial per CTA (fp32 [grid, width]).
constexpr int ROWS_PER_CTA = 32;
constexpr int MAX_CHUNKS = 4;  // width <= NT * 8 * MAX_CHUNKS = 8192

__global__ void __launch_bounds__(NT) rms_norm_bwd_kernel(
    const __nv_bfloat16* __restrict__ grad, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
    __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows, int width,
    const __nv_bfloat16* __restrict__ extra) {
  // extra (may be null): a gradient that reaches the same tensor on another path (the residual
  // branch); it is added in FP32 before the one rounding of dx.
  __shared__ float scratch[NT / 32];
  float dw[MAX_CHUNKS][8];
#pragma unroll
  for (int k = 0; k < MAX_CHUNKS; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) dw[k][i] = 0.f;
  const int row0 = blockIdx.x * ROWS_PER_CTA;
  const int row1 = min(rows, row0 + ROWS_PER_CTA);
  for (int64_t row = row0; row < row1; ++row) {
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_CHUNKS; ++k) {
      const int c = (k * NT + threadIdx.x) * 8;
      if (c < width) {
        float g[8], xv[8], wv[8];
        unpack8(*reinterpret_cast<const uint4*>(grad + row * width + c), g);
        unpack8(*reinterpret_cast<const uint4*>(x + row * width + c), xv);
        unpack8(*reinterpret_cast<const uint4*>(w + c), wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dot += g[i] * wv[i] * xv[i];
          dw[k][i] += g[i] * round_bf16(xv[i] * r);
        }
      }
    }
    dot = block_sum(dot, scratch);
    const float coef = dot * r * r * r / float(width);
#pragma unroll
    for (int k = 0; k < MAX_CHUNKS; ++k) {
      const int c = (k * NT + threadIdx.x) * 8;
      if (c < width) {
        float g[8], xv[8], wv[8], o[8];
        unpack8(*reinterpret_cast<const uint4*>(grad + row * width + c), g);
        unpack8(*reinterpret_cast<const uint4*>(x + row * width + c), xv);
        unpack8(*reinterpret_cast<const uint4*>(w + c), wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = g[i] * wv[i] * r - xv[i] * coef;
        if (extra) {
          float e[8];
          unpack8(*reinterpret_cast<const uint4*>(extra + row * width + c), e);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += e[i];
        }
        *reinterpret_cast<uint4*>(dx + row * width + c) = pack8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < MAX_CHUNKS; ++k) {
    const int c = (k * NT + threadIdx.x) * 8;
    if (c < width) {
      float* dst = dw_partial + int64_t(blockIdx.x) * width + c;
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[i] = dw[k][i];
    }
  }
}

// -------------------------------------------------------------- head norm + RoPE (D=128)
// One warp per (token, head).  Lane l owns elements {2l, 2l+1, 64+2l, 65+2l}: both members
// of every rotate-half pair (i, i+64) live in the same lane.
__global__ void __launch_bounds__(NT) head_norm_rope_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    const __nv_bfloat16* __restrict__ cosv, const __nv_bfloat16* __restrict__ sinv,
    __nv_bfloat16* __restrict__ out, float* __restrict__ rstd_out, int64_t rows, int heads,
    int64_t row_stride, float eps) {
  const int64_t unit = int64_t(blockIdx.x) * (NT / 32) + (threadIdx.x >> 5);
  if (unit >= rows * heads) return;
  const int lane = threadIdx.x & 31;
  const int64_t token = unit / heads;
  // the input may be a column block of a wider matrix (e.g. the q part of a fused qkv product)
  const __nv_bfloat16* xr = x + token * row_stride + (unit - token * heads) * 128;
  const uint32_t a = *reinterpret_cast<const uint32_t*>(xr + 2 * lane);
  const uint32_t b = *reinterpret_cast<const uint32_t*>(xr + 64 + 2 * lane);
  float v[4] = {bf16_lo(a), bf16_hi(a), bf16_lo(b), bf16_hi(b)};
  float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rstd = rsqrtf(ss / 128.f + eps);
  if (rstd_out && lane == 0) rstd_out[unit] = rstd;
  const uint32_t wa = *reinterpret_cast<const uint32_t*>(w + 2 * lane);
  const uint32_t wb = *reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane);
  const float wv[4] = {bf16_lo(wa), bf16_hi(wa), bf16_lo(wb), bf16_hi(wb)};
  float y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) y[i] = round_bf16(wv[i] * round_bf16(v[i] * rstd));
  const uint32_t ca = *reinterpret_cast<const uint32_t*>(cosv + token * 128 + 2 * lane);
  const uint32_t cb = *reinterpret_cast<const uint32_t*>(cosv + token * 128 + 64 + 2 * lane);
  const uint32_t sa = *reinterpret_cast<const uint32_t*>(sinv + token * 128 + 2 * lane);
  const uint32_t sb = *reinterpret_cast<const uint32_t*>(sinv + token * 128 + 64 + 2 * lane);
  const float c[4] = {bf16_lo(ca), bf16_hi(ca), bf16_lo(cb), bf16_hi(cb)};
  const float s[4] = {bf16_lo(sa), bf16_hi(sa), bf16_lo(sb), bf16_hi(sb)};
  // rotate_half(y)[i] = -y[i+64] (i < 64), y[i-64] (i >= 64)
  const float o0 = round_bf16(y[0] * c[0]) + round_bf16(-y[2] * s[0]);
  const float o1 = round_bf16(y[1] * c[1]) + round_bf16(-y[3] * s[1]);
  const float o2 = round_bf16(y[2] * c[2]) + round_bf16(y[0] * s[2]);
  const float o3 = round_bf16(y[3] * c[3]) + round_bf16(y[1] * s[3]);
  __nv_bfloat16* dst = out + unit * 128;
  *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16(o0, o1);
  *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = pack_bf16(o2, o3);
}

constexpr int HEAD_UNITS_PER_WARP = 64;  // (token, head) units walked by one warp in bwd

__global__ void __launch_bounds__(NT) head_norm_rope_bwd_kernel(
    const __nv_bfloat16* __restrict__ grad, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ cosv,
    const __nv_bfloat16* __restrict__ sinv, const float* __restrict__ rstd,
    __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int64_t rows, int heads,
    int64_t x_row_stride, int64_t dx_row_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = int64_t(blockIdx.x) * (NT / 32) + (threadIdx.x >> 5);
  const int64_t u0 = warp_global * HEAD_UNITS_PER_WARP;
  const int64_t u1 = min(rows * heads, u0 + HEAD_UNITS_PER_WARP);
  const uint32_t wa = *reinterpret_cast<const uint32_t*>(w + 2 * lane);
  const uint32_t wb = *reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane);
  const float wv[4] = {bf16_lo(wa), bf16_hi(wa), bf16_lo(wb), bf16_hi(wb)};
  float dw[4] = {0.f, 0.f, 0.f, 0.f};
  for (int64_t unit = u0; unit < u1; ++unit) {
    const int64_t token = unit / heads;
    // x and dx may be column slices of wider matrices (the q or k part of a fused q|k|v product)
    const int64_t x_at = token * x_row_stride + (unit - token * heads) * 128;
    const int64_t dx_at = token * dx_row_stride + (unit - token * heads) * 128;
    const uint32_t ga = *reinterpret_cast<const uint32_t*>(grad + unit * 128 + 2 * lane);
    const uint32_t gb = *reinterpret_cast<const uint32_t*>(grad + unit * 128 + 64 + 2 * lane);
    const float g[4] = {bf16_lo(ga), bf16_hi(ga), bf16_lo(gb), bf16_hi(gb)};
    const uint32_t ca = *reinterpret_cast<const uint32_t*>(cosv + token * 128 + 2 * lane);
    const uint32_t cb = *reinterpret_cast<const uint32_t*>(cosv + token * 128 + 64 + 2 * lane);
    const uint32_t sa = *reinterpret_cast<const uint32_t*>(sinv + token * 128 + 2 * lane);
    const uint32_t sb = *reinterpret_cast<const uint32_t*>(sinv + token * 128 + 64 + 2 * lane);
    const float c[4] = {bf16_lo(ca), bf16_hi(ca), bf16_lo(cb), bf16_hi(cb)};
    const float s[4] = {bf16_lo(sa), bf16_hi(sa), bf16_lo(sb), bf16_hi(sb)};
    // out_i = y_i c_i - y_{i+64} s_i ; out_{i+64} = y_{i+64} c_{i+64} + y_i s_{i+64}
    const float dy[4] = {g[0] * c[0] + g[2] * s[2], g[1] * c[1] + g[3] * s[3],
                         g[2] * c[2] - g[0] * s[0], g[3] * c[3] - g[1] * s[1]};
    const uint32_t xa = *reinterpret_cast<const uint32_t*>(x + x_at + 2 * lane);
    const uint32_t xb = *reinterpret_cast<const uint32_t*>(x + x_at + 64 + 2 * lane);
    const float xv[4] = {bf16_lo(xa), bf16_hi(xa), bf16_lo(xb), bf16_hi(xb)};
    const float r = rstd[unit];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dot += dy[i] * wv[i] * xv[i];
      dw[i] += dy[i] * round_bf16(xv[i] * r);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float coef = dot * r * r * r / 128.f;
    float o4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o4[i] = dy[i] * wv[i] * r - xv[i] * coef;
    *reinterpret_cast<uint32_t*>(dx + dx_at + 2 * lane) = pack_bf16(o4[0], o4[1]);
    *reinterpret_cast<uint32_t*>(dx + dx_at + 64 + 2 * lane) = pack_bf16(o4[2], o4[3]);
  }
  float* dst = dw_partial + warp_global * 128;
  dst[2 * lane] = dw[0];
  dst[2 * lane + 1] = dw[1];
  dst[64 + 2 * lane] = dw[2];
  dst[65 + 2 * lane] = dw[3];
}

// --------------------------------------------------------------------------- SiLU * mul
__global__ void __launch_bounds__(NT) silu_mul_fwd_kernel(const __nv_bfloat16* __restrict__ gate,
                                                          const __nv_bfloat16* __restrict__ up,
                                                          __nv_bfloat16* __restrict__ out,
                                                          int64_t vecs) {
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < vecs; i += int64_t(gridDim.x) * NT) {
    float g[8], u[8];
    unpack8(reinterpret_cast<const uint4*>(gate)[i], g);
    unpack8(reinterpret_cast<const uint4*>(up)[i], u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = round_bf16(g[k] / (1.f + __expf(-g[k]))) * u[k];
    reinterpret_cast<uint4*>(out)[i] = pack8(g);
  }
}

__global__ void __launch_bounds__(NT) silu_mul_bwd_kernel(const __nv_bfloat16* __restrict__ grad,
                                                          const __nv_bfloat16* __restrict__ gate,
                                                          const __nv_bfloat16* __restrict__ up,
                                                          __nv_bfloat16* __restrict__ dgate,
                                                          __nv_bfloat16* __restrict__ dup,
                                                          int64_t vecs) {
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < vecs; i += int64_t(gridDim.x) * NT) {
    float d[8], g[8], u[8], dg[8], du[8];
    unpack8(reinterpret_cast<const uint4*>(grad)[i], d);
    unpack8(reinterpret_cast<const uint4*>(gate)[i], g);
    unpack8(reinterpret_cast<const uint4*>(up)[i], u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * sig;
      du[k] = d[k] * round_bf16(silu);
      dg[k] = d[k] * u[k] * sig * (1.f + g[k] * (1.f - sig));
    }
    reinterpret_cast<uint4*>(dgate)[i] = pack8(dg);
    reinterpret_cast<uint4*>(dup)[i] = pack8(du);
  }
}

// ------------------------------------------------------------------ rectified-flow combine
// mode 0: (1 - s) * a + s * b      mode 1: a - s * b
// sigma is [B] (sigma_frames == 1) or [B, T]; tensors are [B, C, T, HW] contiguous.
template <typename T>
__global__ void __launch_bounds__(NT) rf_combine_kernel(const T* __restrict__ a,
                                                        const T* __restrict__ b,
                                                        const float* __restrict__ sigma,
                                                        T* __restrict__ out, int64_t total,
                                                        int64_t per_sample, int frames, int hw,
                                                        int sigma_frames, int mode) {
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int64_t sample = i / per_sample;
    const int frame = sigma_frames == 1 ? 0 : int((i / hw) % frames);
    // sigma is rounded to the tensor dtype first, as the eager expression does.
    const float s = float(T(sigma[sample * sigma_frames + frame]));
    const float av = float(a[i]), bv = float(b[i]);
    float r;
    if (mode == 0) {
      r = float(T(float(T(1.f - s)) * av)) + float(T(s * bv));
    } else {
      r = av - float(T(s * bv));
    }
    out[i] = T(r);
  }
}

// ------------------------------------------------------ distribution-matching target
// For each sample (row of `per` elements), all arithmetic in FP64 as the eager expression:
//   spread = max(mean |estimate - teacher|, 1e-5)
//   step   = (fake - teacher) / spread,   target = estimate - step
// Pass one leaves per-block partial sums of |estimate - teacher| (no atomics: the sum has a
// fixed order); pass two adds a sample's partials, writes the target and leaves per-block
// partial sums of float(step)^2 for the reported root mean square.
constexpr int DMD_BLOCKS = 32;  // blocks per sample in both passes

__device__ __forceinline__ double block_sum(double v, double* shared) {
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) shared[threadIdx.x >> 5] = v;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < NT / 32; ++i) total += shared[i];
  __syncthreads();
  return total;
}

__global__ void __launch_bounds__(NT) dmd_spread_kernel(const float* __restrict__ estimate,
                                                        const float* __restrict__ teacher,
                                                        double* __restrict__ partial, int64_t per) {
  __shared__ double shared[NT / 32];
  const int64_t base = int64_t(blockIdx.y) * per;
  double sum = 0.0;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < per; i += int64_t(DMD_BLOCKS) * NT)
    sum += fabs(double(estimate[base + i]) - double(teacher[base + i]));
  sum = block_sum(sum, shared);
  if (threadIdx.x == 0) partial[blockIdx.y * DMD_BLOCKS + blockIdx.x] = sum;
}

__global__ void __launch_bounds__(NT) dmd_target_kernel(const float* __restrict__ estimate,
                                                        const float* __restrict__ fake,
                                                        const float* __restrict__ teacher,
                                                        const double* __restrict__ partial,
                                                        double* __restrict__ target,
                                                        double* __restrict__ squares, int64_t per) {
  __shared__ double shared[NT / 32];
  double total = 0.0;
  for (int i = 0; i < DMD_BLOCKS; ++i) total += partial[blockIdx.y * DMD_BLOCKS + i];
  const double spread = fmax(total / double(per), 1e-5);
  const int64_t base = int64_t(blockIdx.y) * per;
  double sum = 0.0;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < per; i += int64_t(DMD_BLOCKS) * NT) {
    const double step = (double(fake[base + i]) - double(teacher[base + i])) / spread;
    target[base + i] = double(estimate[base + i]) - step;
    const float narrow = float(step);
    sum += double(narrow * narrow);
  }
  sum = block_sum(sum, shared);
  if (threadIdx.x == 0) squares[blockIdx.y * DMD_BLOCKS + blockIdx.x] = sum;
}

int grid_for(int64_t work_items) {
  const int64_t blocks = (work_items + NT - 1) / NT;
  return int(blocks < 148 * 16 ? (blocks > 0 ? blocks : 1) : 148 * 16);
}

// --------------------------------------------------------------- AdaLN modulation
// out = bf16(rms_norm(x) * w) * (1 + scale) + shift, one CTA per row.  scale and shift are rows
// of a wider matrix (the six-way modulation projection), `mod_stride` elements apart.
__global__ void __launch_bounds__(NT) norm_modulate_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    const __nv_bfloat16* __restrict__ scale, const __nv_bfloat16* __restrict__ shift,
    __nv_bfloat16* __restrict__ out, int width, int64_t mod_stride, float eps) {
  __shared__ float scratch[NT / 32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * width;
  float sumsq = 0.f;
  for (int c = threadIdx.x * 8; c < width; c += NT * 8) {
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) sumsq += v[i] * v[i];
  }
  const float rstd = rsqrtf(block_sum(sumsq, scratch) / float(width) + eps);
  for (int c = threadIdx.x * 8; c < width; c += NT * 8) {
    float v[8], g[8], sc[8], sh[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
    unpack8(*reinterpret_cast<const uint4*>(w + c), g);
    unpack8(*reinterpret_cast<const uint4*>(scale + row * mod_stride + c), sc);
    unpack8(*reinterpret_cast<const uint4*>(shift + row * mod_stride + c), sh);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float normed = round_bf16(g[i] * round_bf16(v[i] * rstd));
      v[i] = round_bf16(normed * round_bf16(1.f + sc[i])) + sh[i];
    }
    *reinterpret_cast<uint4*>(out + row * width + c) = pack8(v);
  }
}

// out = hidden + gate * y (gate a row of the modulation matrix, `gate_stride` elements apart).
__global__ void __launch_bounds__(NT) gated_residual_kernel(
    const __nv_bfloat16* __restrict__ hidden, const __nv_bfloat16* __restrict__ gate,
    const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ out, int64_t rows, int width,
    int64_t gate_stride) {
  const int per_row = width / 8;
  const int64_t total = rows * per_row;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < total; i += int64_t(gridDim.x) * NT) {
    const int64_t row = i / per_row;
    const int c = int(i % per_row) * 8;
    float h[8], g[8], v[8];
    unpack8(*reinterpret_cast<const uint4*>(hidden + row * width + c), h);
    unpack8(*reinterpret_cast<const uint4*>(gate + row * gate_stride + c), g);
    unpack8(*reinterpret_cast<const uint4*>(y + row * width + c), v);
#pragma unroll
    for (int k = 0; k < 8; ++k) h[k] += round_bf16(g[k] * v[k]);
    *reinterpret_cast<uint4*>(out + row * width + c) = pack8(h);
  }
}

}  // namespace

cudaError_t rms_norm_fwd(const void* x, const void* addend, const void* w, void* total_out,
                         void* out, float* rstd, int64_t rows, int width, float eps,
                         cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if (width % 8) return cudaErrorInvalidValue;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto A = static_cast<const __nv_bfloat16*>(addend);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto TO = static_cast<__nv_bfloat16*>(total_out);
  auto O = static_cast<__nv_bfloat16*>(out);
  if (addend)
    rms_norm_fwd_kernel<true><<<unsigned(rows), NT, 0, stream>>>(X, A, W, TO, O, rstd, width, eps);
  else
    rms_norm_fwd_kernel<false><<<unsigned(rows), NT, 0, stream>>>(X, A, W, TO, O, rstd, width, eps);
  return cudaGetLastError();
}

cudaError_t norm_modulate(const void* x, const void* w, const void* scale, const void* shift,
                          void* out, int64_t rows, int width, int64_t mod_stride, float eps,
                          cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if ((width % 8) || (mod_stride % 8)) return cudaErrorInvalidValue;
  norm_modulate_kernel<<<unsigned(rows), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(scale), static_cast<const __nv_bfloat16*>(shift),
      static_cast<__nv_bfloat16*>(out), width, mod_stride, eps);
  return cudaGetLastError();
}

cudaError_t gated_residual(const void* hidden, const void* gate, const void* y, void* out,
                           int64_t rows, int width, int64_t gate_stride, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if ((width % 8) || (gate_stride % 8)) return cudaErrorInvalidValue;
  const int64_t blocks = (rows * (width / 8) + NT - 1) / NT;
  gated_residual_kernel<<<unsigned(blocks < 148 * 16 ? blocks : 148 * 16), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(hidden), static_cast<const __nv_bfloat16*>(gate),
      static_cast<const __nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(out), rows, width,
      gate_stride);
  return cudaGetLastError();
}

int rms_norm_bwd_partials(int64_t rows) { return int((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA); }

cudaError_t rms_norm_bwd(const void* grad, const void* x, const void* w, const float* rstd,
                         void* dx, float* dw_partial, int64_t rows, int width,
                         cudaStream_t stream, const void* extra) {
  if (rows == 0) return cudaSuccess;
  if (width % 8 || width > NT * 8 * MAX_CHUNKS) return cudaErrorInvalidValue;
  rms_norm_bwd_kernel<<<rms_norm_bwd_partials(rows), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(grad), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), dw_partial,
      int(rows), width, static_cast<const __nv_bfloat16*>(extra));
  return cudaGetLastError();
}

cudaError_t head_norm_rope_fwd(const void* x, const void* w, const void* cosv, const void* sinv,
                               void* out, float* rstd, int64_t rows, int heads, int64_t row_stride,
                               float eps, cudaStream_t stream) {
  const int64_t units = rows * heads;
  if (units == 0) return cudaSuccess;
  const unsigned grid = unsigned((units + NT / 32 - 1) / (NT / 32));
  head_norm_rope_fwd_kernel<<<grid, NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(cosv), static_cast<const __nv_bfloat16*>(sinv),
      static_cast<__nv_bfloat16*>(out), rstd, rows, heads, row_stride, eps);
  return cudaGetLastError();
}

int head_norm_rope_bwd_partials(int64_t rows, int heads) {
  const int64_t warps = (rows * heads + HEAD_UNITS_PER_WARP - 1) / HEAD_UNITS_PER_WARP;
  const int64_t blocks = (warps + NT / 32 - 1) / (NT / 32);
  return int(blocks * (NT / 32));
}

cudaError_t head_norm_rope_bwd(const void* grad, const void* x, const void* w, const void* cosv,
                               const void* sinv, const float* rstd, void* dx, float* dw_partial,
                               int64_t rows, int heads, int64_t x_row_stride, int64_t dx_row_stride,
                               cudaStream_t stream) {
  if (rows * heads == 0) return cudaSuccess;
  const int partial_rows = head_norm_rope_bwd_partials(rows, heads);
  head_norm_rope_bwd_kernel<<<partial_rows / (NT / 32), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(grad), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(cosv),
      static_cast<const __nv_bfloat16*>(sinv), rstd, static_cast<__nv_bfloat16*>(dx), dw_partial,
      rows, heads, x_row_stride, dx_row_stride);
  return cudaGetLastError();
}

cudaError_t silu_mul_fwd(const void* gate, const void* up, void* out, int64_t elements,
                         cudaStream_t stream) {
  if (elements == 0) return cudaSuccess;
  if (elements % 8) return cudaErrorInvalidValue;
  silu_mul_fwd_kernel<<<grid_for(elements / 8), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
      static_cast<__nv_bfloat16*>(out), elements / 8);
  return cudaGetLastError();
}

// gate and up are the two column halves of one [rows, 2 * width] matrix (one GEMM produced both).
__global__ void __launch_bounds__(NT) silu_mul_pair_kernel(const __nv_bfloat16* __restrict__ both,
                                                           __nv_bfloat16* __restrict__ out,
                                                           int64_t rows, int width) {
  const int per_row = width / 8;
  const int64_t vecs = rows * per_row;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < vecs; i += int64_t(gridDim.x) * NT) {
    const int64_t row = i / per_row;
    const int col = int(i - row * per_row) * 8;
    float g[8], u[8];
    unpack8(*reinterpret_cast<const uint4*>(both + row * 2 * width + col), g);
    unpack8(*reinterpret_cast<const uint4*>(both + row * 2 * width + width + col), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = round_bf16(g[k] / (1.f + __expf(-g[k]))) * u[k];
    *reinterpret_cast<uint4*>(out + row * width + col) = pack8(g);
  }
}

cudaError_t silu_mul_pair(const void* both, void* out, int64_t rows, int width, cudaStream_t stream) {
  if (rows == 0 || width == 0) return cudaSuccess;
  if (width % 8) return cudaErrorInvalidValue;
  silu_mul_pair_kernel<<<grid_for(rows * (width / 8)), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(both), static_cast<__nv_bfloat16*>(out), rows, width);
  return cudaGetLastError();
}

// Backward of silu_mul_pair: grad [rows, width], both = [gate | up], dboth = [dgate | dup].
// With `act` given it also writes the forward value silu(gate) * up (bit for bit what
// silu_mul_pair gives), which the caller needs for the next weight gradient: one pass over
// `both` instead of two.
__global__ void __launch_bounds__(NT) silu_mul_pair_bwd_kernel(const __nv_bfloat16* __restrict__ grad,
                                                               const __nv_bfloat16* __restrict__ both,
                                                               __nv_bfloat16* __restrict__ dboth,
                                                               __nv_bfloat16* __restrict__ act,
                                                               int64_t rows, int width) {
  const int per_row = width / 8;
  const int64_t vecs = rows * per_row;
  for (int64_t i = int64_t(blockIdx.x) * NT + threadIdx.x; i < vecs; i += int64_t(gridDim.x) * NT) {
    const int64_t row = i / per_row;
    const int col = int(i - row * per_row) * 8;
    float d[8], g[8], u[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(grad + row * width + col), d);
    unpack8(*reinterpret_cast<const uint4*>(both + row * 2 * width + col), g);
    unpack8(*reinterpret_cast<const uint4*>(both + row * 2 * width + width + col), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * sig;
      du[k] = d[k] * round_bf16(silu);
      dg[k] = d[k] * u[k] * sig * (1.f + g[k] * (1.f - sig));
    }
    *reinterpret_cast<uint4*>(dboth + row * 2 * width + col) = pack8(dg);
    *reinterpret_cast<uint4*>(dboth + row * 2 * width + width + col) = pack8(du);
    if (act) {
#pragma unroll
      for (int k = 0; k < 8; ++k) d[k] = round_bf16(g[k] / (1.f + __expf(-g[k]))) * u[k];
      *reinterpret_cast<uint4*>(act + row * width + col) = pack8(d);
    }
  }
}

cudaError_t silu_mul_pair_bwd(const void* grad, const void* both, void* dboth, int64_t rows,
                              int width, cudaStream_t stream, void* act) {
  if (rows == 0 || width == 0) return cudaSuccess;
  if (width % 8) return cudaErrorInvalidValue;
  silu_mul_pair_bwd_kernel<<<grid_for(rows * (width / 8)), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(grad), static_cast<const __nv_bfloat16*>(both),
      static_cast<__nv_bfloat16*>(dboth), static_cast<__nv_bfloat16*>(act), rows, width);
  return cudaGetLastError();
}

cudaError_t silu_mul_bwd(const void* grad, const void* gate, const void* up, void* dgate,
                         void* dup, int64_t elements, cudaStream_t stream) {
  if (elements == 0) return cudaSuccess;
  if (elements % 8) return cudaErrorInvalidValue;
  silu_mul_bwd_kernel<<<grid_for(elements / 8), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(grad), static_cast<const __nv_bfloat16*>(gate),
      static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(dgate),
      static_cast<__nv_bfloat16*>(dup), elements / 8);
  return cudaGetLastError();
}

// ------------------------------------------------- channel RMS norm (+ SiLU), channels last
// y = x / max(||x||_2, 1e-12) * sqrt(C) * gamma over the C contiguous channels of a pixel,
// optionally followed by SiLU: the norm / activation pair in front of every convolution of
// the video VAE, in one pass (one warp per pixel, C <= 1024, a multiple of 8).
template <bool SILU>
__global__ void __launch_bounds__(NT) channel_norm_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ gamma,
                                                          __nv_bfloat16* __restrict__ out,
                                                          int64_t pixels, int channels) {
  const int lane = threadIdx.x & 31;
  const int chunks = channels >> 3;
  const float gain = sqrtf(float(channels));
  for (int64_t pixel = (int64_t(blockIdx.x) * NT + threadIdx.x) >> 5; pixel < pixels;
       pixel += (int64_t(gridDim.x) * NT) >> 5) {
    const __nv_bfloat16* row = x + pixel * channels;
    float v[4][8];
    float sumsq = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = k * 32 + lane;
      if (c < chunks) {
        unpack8(*reinterpret_cast<const uint4*>(row + c * 8), v[k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) sumsq += v[k][i] * v[k][i];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
    const float scale = gain / fmaxf(sqrtf(sumsq), 1e-12f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = k * 32 + lane;
      if (c < chunks) {
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + c * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(gamma + c * 8 + 4);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float n = v[k][i] * scale * g[i];
          y[i] = SILU ? n / (1.f + __expf(-n)) : n;
        }
        *reinterpret_cast<uint4*>(out + pixel * channels + c * 8) = pack8(y);
      }
    }
  }
}

cudaError_t channel_norm(const void* x, const float* gamma, void* out, int64_t pixels, int channels,
                         int silu, cudaStream_t stream) {
  if (pixels == 0) return cudaSuccess;
  if (channels % 8 || channels > 1024 || channels <= 0) {
    set_error_detail("channel_norm: channels must be a multiple of 8 up to 1024");
    return cudaErrorInvalidValue;
  }
  const int64_t warps_per_cta = NT / 32;
  const int64_t ctas = (pixels + warps_per_cta - 1) / warps_per_cta;
  const unsigned grid = unsigned(ctas < 148 * 32 ? ctas : 148 * 32);
  auto xs = static_cast<const __nv_bfloat16*>(x);
  auto os = static_cast<__nv_bfloat16*>(out);
  if (silu) channel_norm_kernel<true><<<grid, NT, 0, stream>>>(xs, gamma, os, pixels, channels);
  else channel_norm_kernel<false><<<grid, NT, 0, stream>>>(xs, gamma, os, pixels, channels);
  return cudaGetLastError();
}

// One warp per (sample, query row, head): 128 bf16 values = 4 per lane.
__global__ void __launch_bounds__(NT) attn_combine_kernel(const __nv_bfloat16* __restrict__ partial,
                                                          const float* __restrict__ lse,
                                                          __nv_bfloat16* __restrict__ out,
                                                          int64_t rows_total, int64_t nq, int hq,
                                                          int splits) {
  const int64_t item = (int64_t(blockIdx.x) * NT + threadIdx.x) >> 5;  // (b, q, h) flattened
  if (item >= rows_total) return;
  const int lane = threadIdx.x & 31;
  const int h = int(item % hq);
  const int64_t q = (item / hq) % nq, b = item / (int64_t(hq) * nq);
  const int64_t lse_base = (b * hq + h) * (int64_t(splits) * nq) + q;
  float top = -INFINITY;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, lse[lse_base + s * nq]);
  float total = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < splits; ++s) {
    const float v = lse[lse_base + s * nq];
    const float w = (v == -INFINITY) ? 0.f : __expf(v - top);
    if (w == 0.f) continue;  // an empty split may hold anything
    total += w;
    const uint2 raw = *reinterpret_cast<const uint2*>(
        partial + ((b * (int64_t(splits) * nq) + s * nq + q) * hq + h) * 128 + lane * 4);
    acc[0] += w * bf16_lo(raw.x);
    acc[1] += w * bf16_hi(raw.x);
    acc[2] += w * bf16_lo(raw.y);
    acc[3] += w * bf16_hi(raw.y);
  }
  const float inv = total > 0.f ? 1.f / total : 0.f;
  *reinterpret_cast<uint2*>(out + ((b * nq + q) * hq + h) * 128 + lane * 4) =
      make_uint2(pack_bf16(acc[0] * inv, acc[1] * inv), pack_bf16(acc[2] * inv, acc[3] * inv));
}

cudaError_t attention_combine(const void* partial, const float* lse, void* out, int64_t batch,
                              int64_t nq, int hq, int splits, cudaStream_t stream) {
  const int64_t items = batch * nq * hq;
  if (items == 0) return cudaSuccess;
  const int64_t threads = items * 32;
  attn_combine_kernel<<<unsigned((threads + NT - 1) / NT), NT, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(partial), lse, static_cast<__nv_bfloat16*>(out), items, nq,
      hq, splits);
  return cudaGetLastError();
}

cudaError_t rf_combine(const void* a, const void* b, const float* sigma, void* out, int64_t batch,
                       int64_t channels, int frames, int hw, int sigma_frames, int mode,
                       int is_bf16, cudaStream_t stream) {
  const int64_t per_sample = channels * frames * hw;
  const int64_t total = batch * per_sample;
  if (total == 0) return cudaSuccess;
  if (is_bf16)
    rf_combine_kernel<__nv_bfloat16><<<grid_for(total), NT, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), sigma,
        static_cast<__nv_bfloat16*>(out), total, per_sample, frames, hw, sigma_frames, mode);
  else
    rf_combine_kernel<float><<<grid_for(total), NT, 0, stream>>>(
        static_cast<const float*>(a), static_cast<const float*>(b), sigma,
        static_cast<float*>(out), total, per_sample, frames, hw, sigma_frames, mode);
  return cudaGetLastError();
}

int dmd_target_blocks() { return DMD_BLOCKS; }

cudaError_t dmd_target(const float* estimate, const float* fake, const float* teacher, double* partial,
                       double* target, double* squares, int64_t batch, int64_t per, cudaStream_t stream) {
  if (batch == 0 || per == 0) return cudaSuccess;
  if (batch > 65535) return cudaErrorInvalidValue;
  const dim3 grid(DMD_BLOCKS, unsigned(batch));
  dmd_spread_kernel<<<grid, NT, 0, stream>>>(estimate, teacher, partial, per);
  dmd_target_kernel<<<grid, NT, 0, stream>>>(estimate, fake, teacher, partial, target, squares, per);
  return cudaGetLastError();
}

}  // namespace agb
