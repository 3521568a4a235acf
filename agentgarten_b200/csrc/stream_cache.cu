// KV-cache maintenance for streaming inference: FIFO eviction with RoPE re-rotation.
//
// A cache tensor holds rows [token][kv_head][128] (bf16).  After a commit that overflows
// the frame budget, the rows behind the permanent sink move `shift` rows towards the front
// and — for keys — are rotated by the phase difference between their old and new temporal
// positions (cos/sin of the difference, fp32 [kept_tokens, 128], rotate-half convention).
// One pass: every retained row is read once from `src` and written once to `dst` (a second
// buffer, so no row is overwritten before it is read).
#include "agb.h"
#include "sm100.cuh"

namespace agb {
namespace {

// One warp per (token, head) row; lane l owns elements {2l, 2l+1, 64+2l, 65+2l}.
__global__ void __launch_bounds__(256) relocate_kernel(const __nv_bfloat16* __restrict__ src,
                                                       __nv_bfloat16* __restrict__ dst,
                                                       const float* __restrict__ cosv,
                                                       const float* __restrict__ sinv,
                                                       int64_t kept_tokens, int sink_tokens,
                                                       int shift_tokens, int heads) {
  const int64_t unit = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (unit >= kept_tokens * heads) return;
  const int lane = threadIdx.x & 31;
  const int64_t token = unit / heads;
  const int head = int(unit % heads);
  const int64_t from = token < sink_tokens ? token : token + shift_tokens;
  const __nv_bfloat16* s = src + (from * heads + head) * 128;
  __nv_bfloat16* d = dst + unit * 128;
  const uint32_t a = *reinterpret_cast<const uint32_t*>(s + 2 * lane);
  const uint32_t b = *reinterpret_cast<const uint32_t*>(s + 64 + 2 * lane);
  if (!cosv || token < sink_tokens) {
    *reinterpret_cast<uint32_t*>(d + 2 * lane) = a;
    *reinterpret_cast<uint32_t*>(d + 64 + 2 * lane) = b;
    return;
  }
  const float x0 = bf16_lo(a), x1 = bf16_hi(a), y0 = bf16_lo(b), y1 = bf16_hi(b);
  const float* c = cosv + token * 128;
  const float* sn = sinv + token * 128;
  const float2 c_lo = *reinterpret_cast<const float2*>(c + 2 * lane);
  const float2 c_hi = *reinterpret_cast<const float2*>(c + 64 + 2 * lane);
  const float2 s_lo = *reinterpret_cast<const float2*>(sn + 2 * lane);
  const float2 s_hi = *reinterpret_cast<const float2*>(sn + 64 + 2 * lane);
  // rotate_half(v)[i] = -v[i+64] (i < 64), v[i-64] (i >= 64)
  *reinterpret_cast<uint32_t*>(d + 2 * lane) =
      pack_bf16(x0 * c_lo.x - y0 * s_lo.x, x1 * c_lo.y - y1 * s_lo.y);
  *reinterpret_cast<uint32_t*>(d + 64 + 2 * lane) =
      pack_bf16(y0 * c_hi.x + x0 * s_hi.x, y1 * c_hi.y + x1 * s_hi.y);
}

}  // namespace

cudaError_t relocate_rows(const void* src, void* dst, const float* cosv, const float* sinv,
                          int64_t kept_tokens, int sink_tokens, int shift_tokens, int heads,
                          cudaStream_t stream) {
  const int64_t units = kept_tokens * heads;
  if (units == 0) return cudaSuccess;
  relocate_kernel<<<unsigned((units + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), cosv, sinv,
      kept_tokens, sink_tokens, shift_tokens, heads);
  return cudaGetLastError();
}

}  // namespace agb
