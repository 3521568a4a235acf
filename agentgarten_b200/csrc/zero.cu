// Sharded optimizer step over peer memory (NVLink P2P loads and stores from inside the
// kernels): gradient reduce-scatter + norm/finite side outputs, then Adam on the FP32
// shard fused with the bf16 parameter all-gather.
//
// Every rank keeps the whole bf16 parameter buffer and the whole bf16 gradient buffer of an
// optimizer in two flat allocations that all ranks of the node map (peer pointers).  A rank
// owns a list of "units": (flat offset, state offset, count) ranges, at most UNIT elements
// each, that follow the FSDP2 rule (chunk `rank` of dim 0 of every parameter).
//
//   zero_reduce:  for every owned unit, load the unit from each rank's gradient buffer
//                 (plain ld.global on peer pointers), sum in FP32 in rank order, scale by
//                 1/world, store the FP32 result locally, and emit per-CTA partial sums of
//                 squares and a non-finite flag.  zero_reduce_finish folds the partials in
//                 a fixed order (deterministic norm).
//                 With several ranks the bf16 average is written back over this rank's own
//                 gradient of the range (no peer reads that range), so the peers' gradients
//                 cross NVLink once and no FP32 gradient shard is allocated -- the reduced
//                 gradient is bf16, as it is after FSDP2's reduce-scatter.
//   zero_adam:    Adam/AdamW on the owned units with FP32 master weights and moments (the
//                 averaged gradient is read from an FP32 shard, from this rank's own buffer
//                 after the write-back, or summed again from the peers); the
//                 gradient is multiplied by a device-resident factor (the clip coefficient)
//                 on the fly; the new bf16 values are stored into every rank's parameter
//                 buffer (st.global on peer pointers): the all-gather costs no extra pass.
//
// Cross-rank ordering uses monotonic system-scope counters in symmetric memory instead of
// library collectives: a rank announces "my gradients of bucket b are complete" by adding 1 to
// slot b on every peer (zero_signal); the bucket's reduce kernel waits (bounded) until its own
// slot has reached world * epoch before it loads the peers' gradients, so a bucket can be
// reduced on a side stream while the backward pass of earlier layers is still running.
// zero_stats folds the per-CTA partial sums in a fixed order, stores this rank's two numbers
// into every peer's slot table and sums all ranks' entries in rank order: the global gradient
// norm without an all-reduce, and at the same time the point after which every rank has
// finished reading its peers' gradients.  After Adam a "done" counter tells the peers that
// the stores into their parameter buffers are complete (zero_signal / zero_wait).
#include "agb.h"
#include "sm100.cuh"

namespace agb {
namespace {

constexpr int ZT = 256;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = bf16_lo(w[i]);
    f[2 * i + 1] = bf16_hi(w[i]);
  }
}

// Bounded wait (system scope) until a monotonic counter reaches `target`; false on timeout.
__device__ bool wait_reached(const int* counter, int target, int* status, uint64_t limit_ns) {
  const uint64_t start = global_timer_ns();
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if (counter_reached(seen, target)) return true;
    if (status && *reinterpret_cast<volatile int*>(status) != 0) return false;  // step already lost
    if (global_timer_ns() - start > limit_ns) {
      if (status) atomicCAS(status, 0, kTimeoutPeer);
      return false;
    }
    __nanosleep(256);
  }
}

__global__ void __launch_bounds__(ZT) zero_reduce_kernel(ZeroPeers grads, const int64_t* units,
                                                         int unit_begin, int num_units, float* gshard,
                                                         float* partial_sumsq, int* partial_bad,
                                                         float inv_world, const int* ready,
                                                         int ready_target, int* status,
                                                         uint64_t limit_ns, int write_back_rank) {
  __shared__ float red[ZT / 32];
  __shared__ int bad_any;
  __shared__ int go;
  if (threadIdx.x == 0) {
    bad_any = 0;
    // every rank has finished writing the gradients of this bucket
    go = ready ? (wait_reached(ready, ready_target, status, limit_ns) ? 1 : 0) : 1;
  }
  __syncthreads();
  float sumsq = 0.f;
  int bad = 0;
  if (!go) {  // a peer never arrived: report through the status word, poison the norm
    if (threadIdx.x == 0) {
      partial_sumsq[blockIdx.x] = 0.f;
      partial_bad[blockIdx.x] = 1;
    }
    return;
  }
  for (int u = unit_begin + blockIdx.x; u < num_units; u += gridDim.x) {
    const int64_t flat = units[4 * u], state = units[4 * u + 1];
    const int count = int(units[4 * u + 2]);
    if (((flat | state) & 7) == 0 && (count & 7) == 0) {
      for (int i = threadIdx.x * 8; i < count; i += ZT * 8) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        // All peers' loads of this chunk are issued before the first sum (an NVLink load takes
        // microseconds; one at a time would leave the links idle), the sums stay in rank order.
        uint4 raw[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          if (r < grads.world)
            raw[r] = *reinterpret_cast<const uint4*>(
                static_cast<const __nv_bfloat16*>(grads.ptr[r]) + flat + i);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < grads.world) {
            float v[8];
            unpack8(raw[r], v);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += v[k];
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          acc[k] *= inv_world;
          sumsq += acc[k] * acc[k];
          bad |= !isfinite(acc[k]);
        }
        if (gshard) {
          float4* dst = reinterpret_cast<float4*>(gshard + state + i);
          dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
          dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
        if (write_back_rank >= 0) {
          // the average replaces this rank's own gradient of the range it owns (no peer reads it)
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(grads.ptr[write_back_rank]) + flat + i) =
              make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]),
                         pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
        }
      }
    } else {
      for (int i = threadIdx.x; i < count; i += ZT) {
        float acc = 0.f;
        for (int r = 0; r < grads.world; ++r)
          acc += __bfloat162float(static_cast<const __nv_bfloat16*>(grads.ptr[r])[flat + i]);
        acc *= inv_world;
        sumsq += acc * acc;
        bad |= !isfinite(acc);
        if (gshard) gshard[state + i] = acc;
        if (write_back_rank >= 0)
          static_cast<__nv_bfloat16*>(grads.ptr[write_back_rank])[flat + i] = __float2bfloat16_rn(acc);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sumsq;
  if (bad) bad_any = 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < ZT / 32; ++w) total += red[w];
    partial_sumsq[blockIdx.x] = total;
    partial_bad[blockIdx.x] = bad_any;
  }
}

__global__ void zero_reduce_finish_kernel(const float* partial_sumsq, const int* partial_bad,
                                          int parts, float* sumsq_out, float* bad_out) {
  // one warp, fixed summation order
  float s = 0.f;
  int bad = 0;
  for (int i = threadIdx.x; i < parts; i += 32) {
    s += partial_sumsq[i];
    bad |= partial_bad[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  if (threadIdx.x == 0) {
    *sumsq_out = s;
    *bad_out = bad ? 1.f : 0.f;
  }
}

// counters.ptr[r] + slot on every rank r is advanced by one (release, system scope).
__global__ void zero_signal_kernel(ZeroPeers counters, int slot) {
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < counters.world; ++r) {
      int* c = static_cast<int*>(counters.ptr[r]) + slot;
      asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(c) : "memory");
    }
  }
}

__global__ void zero_wait_kernel(const int* counter, int target, int* status, uint64_t limit_ns) {
  if (threadIdx.x == 0) wait_reached(counter, target, status, limit_ns);
}

// One warp.  Folds `parts` partials in index order, then (world > 1) publishes this rank's
// (sum of squares, non-finite flag) in slot `rank` of every peer's table -- three 32-bit words
// per rank: sum, flag, epoch tag written last with release -- waits for all ranks' entries of
// this epoch and adds them in rank order.
__global__ void zero_stats_kernel(const float* partial_sumsq, const int* partial_bad, int parts,
                                  ZeroPeers tables, int rank, int epoch, float* sumsq_out,
                                  float* bad_out, int* status, uint64_t limit_ns) {
  float s = 0.f;
  int bad = 0;
  for (int i = threadIdx.x; i < parts; i += 32) {
    s += partial_sumsq[i];
    bad |= partial_bad[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  if (threadIdx.x != 0) return;
  if (tables.world > 1) {
    for (int r = 0; r < tables.world; ++r) {
      int* entry = static_cast<int*>(tables.ptr[r]) + 4 * rank;
      reinterpret_cast<volatile float*>(entry)[0] = s;
      reinterpret_cast<volatile int*>(entry)[1] = bad;
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(entry + 2), "r"(epoch) : "memory");
    }
    const int* mine = static_cast<const int*>(tables.ptr[rank]);
    float total = 0.f;
    int any = 0;
    for (int r = 0; r < tables.world; ++r) {
      if (!wait_reached(mine + 4 * r + 2, epoch, status, limit_ns)) {
        any = 1;
        break;
      }
      total += reinterpret_cast<const volatile float*>(mine + 4 * r)[0];
      any |= reinterpret_cast<const volatile int*>(mine + 4 * r)[1];
    }
    s = total;
    bad = any;
  }
  *sumsq_out = s;
  *bad_out = bad ? 1.f : 0.f;
}

struct Hyper {  // one row of the hyper-parameter table (8 floats)
  float lr, beta1, beta2, eps, weight_decay, corr1, corr2_sqrt, adam_w;
};

__device__ __forceinline__ float adam_one(float g, float& m, float& v, float& w, const Hyper& h) {
  if (h.adam_w == 0.f && h.weight_decay != 0.f) g += h.weight_decay * w;
  float numer = g;
  if (h.beta1 > 0.f) {
    m += (g - m) * (1.f - h.beta1);
    numer = m;
  }
  float denom;
  if (h.beta2 > 0.f) {
    v = v * h.beta2 + (1.f - h.beta2) * g * g;
    denom = sqrtf(v) / h.corr2_sqrt + h.eps;
  } else {
    denom = fabsf(g) + h.eps;
  }
  if (h.adam_w != 0.f && h.weight_decay != 0.f) w *= 1.f - h.lr * h.weight_decay;
  w -= (h.lr / h.corr1) * (numer / denom);
  return w;
}

__global__ void __launch_bounds__(ZT) zero_adam_kernel(ZeroPeers params, ZeroPeers grads,
                                                       const int64_t* units,
                                                       int num_units, const float* gshard,
                                                       float* master, float* exp_avg,
                                                       float* exp_avg_sq, const float* hyper,
                                                       const float* grad_scale,
                                                       const float* skip_flag) {
  if (skip_flag && *skip_flag != 0.f) return;  // non-finite gradients: leave everything as is
  const float scale = grad_scale ? *grad_scale : 1.f;
  const float inv_world = 1.f / float(grads.world);
  for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
    const int64_t flat = units[4 * u], state = units[4 * u + 1];
    const int count = int(units[4 * u + 2]);
    const Hyper h = *reinterpret_cast<const Hyper*>(hyper + 8 * units[4 * u + 3]);
    const bool has_m = h.beta1 > 0.f, has_v = h.beta2 > 0.f;
    if (((flat | state) & 7) == 0 && (count & 7) == 0) {
      for (int i = threadIdx.x * 8; i < count; i += ZT * 8) {
        float g[8], m[8], v[8], w[8];
        const float4* wp = reinterpret_cast<const float4*>(master + state + i);
        const float4 w0 = wp[0], w1 = wp[1];
        if (gshard) {
          const float4* gp = reinterpret_cast<const float4*>(gshard + state + i);
          const float4 g0 = gp[0], g1 = gp[1];
          g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w;
          g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
        } else {
          // same summation order as zero_reduce: rank 0 first
#pragma unroll
          for (int k = 0; k < 8; ++k) g[k] = 0.f;
          for (int r = 0; r < grads.world; ++r) {
            float t[8];
            unpack8(*reinterpret_cast<const uint4*>(
                        static_cast<const __nv_bfloat16*>(grads.ptr[r]) + flat + i), t);
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] += t[k];
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) g[k] *= inv_world;
        }
        w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
        w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
        if (has_m) {
          const float4* mp = reinterpret_cast<const float4*>(exp_avg + state + i);
          const float4 m0 = mp[0], m1 = mp[1];
          m[0] = m0.x; m[1] = m0.y; m[2] = m0.z; m[3] = m0.w;
          m[4] = m1.x; m[5] = m1.y; m[6] = m1.z; m[7] = m1.w;
        }
        if (has_v) {
          const float4* vp = reinterpret_cast<const float4*>(exp_avg_sq + state + i);
          const float4 v0 = vp[0], v1 = vp[1];
          v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w;
          v[4] = v1.x; v[5] = v1.y; v[6] = v1.z; v[7] = v1.w;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) adam_one(g[k] * scale, m[k], v[k], w[k], h);
        float4* wo = reinterpret_cast<float4*>(master + state + i);
        wo[0] = make_float4(w[0], w[1], w[2], w[3]);
        wo[1] = make_float4(w[4], w[5], w[6], w[7]);
        if (has_m) {
          float4* mo = reinterpret_cast<float4*>(exp_avg + state + i);
          mo[0] = make_float4(m[0], m[1], m[2], m[3]);
          mo[1] = make_float4(m[4], m[5], m[6], m[7]);
        }
        if (has_v) {
          float4* vo = reinterpret_cast<float4*>(exp_avg_sq + state + i);
          vo[0] = make_float4(v[0], v[1], v[2], v[3]);
          vo[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
        const uint4 packed = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]),
                                        pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
        for (int r = 0; r < params.world; ++r)
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.ptr[r]) + flat + i) = packed;
      }
    } else {
      for (int i = threadIdx.x; i < count; i += ZT) {
        float m = has_m ? exp_avg[state + i] : 0.f;
        float v = has_v ? exp_avg_sq[state + i] : 0.f;
        float w = master[state + i];
        float g;
        if (gshard) {
          g = gshard[state + i];
        } else {
          g = 0.f;
          for (int r = 0; r < grads.world; ++r)
            g += __bfloat162float(static_cast<const __nv_bfloat16*>(grads.ptr[r])[flat + i]);
          g *= inv_world;
        }
        adam_one(g * scale, m, v, w, h);
        master[state + i] = w;
        if (has_m) exp_avg[state + i] = m;
        if (has_v) exp_avg_sq[state + i] = v;
        const __nv_bfloat16 bw = __float2bfloat16_rn(w);
        for (int r = 0; r < params.world; ++r)
          static_cast<__nv_bfloat16*>(params.ptr[r])[flat + i] = bw;
      }
    }
  }
}

}  // namespace

int zero_reduce_parts(int num_units, int sm_count) {
  const int cap = sm_count * 8;
  return num_units < cap ? (num_units > 0 ? num_units : 1) : cap;
}

cudaError_t zero_reduce(const ZeroPeers& grads, const int64_t* units, int num_units,
                        float* gshard, float* partial_sumsq, int* partial_bad, float* sumsq_out,
                        float* bad_out, int sm_count, cudaStream_t stream) {
  const int parts = zero_reduce_parts(num_units, sm_count);
  zero_reduce_kernel<<<parts, ZT, 0, stream>>>(grads, units, 0, num_units, gshard, partial_sumsq,
                                               partial_bad, 1.f / float(grads.world), nullptr, 0,
                                               nullptr, 0, -1);
  zero_reduce_finish_kernel<<<1, 32, 0, stream>>>(partial_sumsq, partial_bad, parts, sumsq_out,
                                                  bad_out);
  return cudaGetLastError();
}

cudaError_t zero_reduce_range(const ZeroPeers& grads, const int64_t* units, int unit_begin,
                              int unit_end, float* gshard, float* partial_sumsq, int* partial_bad,
                              int parts, const int* ready, int ready_target, int* status,
                              uint64_t limit_ns, int write_back_rank, cudaStream_t stream) {
  if (parts <= 0) return cudaSuccess;
  zero_reduce_kernel<<<parts, ZT, 0, stream>>>(grads, units, unit_begin, unit_end, gshard,
                                               partial_sumsq, partial_bad, 1.f / float(grads.world),
                                               ready, ready_target, status, limit_ns,
                                               write_back_rank);
  return cudaGetLastError();
}

cudaError_t zero_signal(const ZeroPeers& counters, int slot, cudaStream_t stream) {
  zero_signal_kernel<<<1, 32, 0, stream>>>(counters, slot);
  return cudaGetLastError();
}

cudaError_t zero_wait(const int* counter, int target, int* status, uint64_t limit_ns,
                      cudaStream_t stream) {
  zero_wait_kernel<<<1, 32, 0, stream>>>(counter, target, status, limit_ns);
  return cudaGetLastError();
}

cudaError_t zero_stats(const float* partial_sumsq, const int* partial_bad, int parts,
                       const ZeroPeers& tables, int rank, int epoch, float* sumsq_out,
                       float* bad_out, int* status, uint64_t limit_ns, cudaStream_t stream) {
  zero_stats_kernel<<<1, 32, 0, stream>>>(partial_sumsq, partial_bad, parts, tables, rank, epoch,
                                          sumsq_out, bad_out, status, limit_ns);
  return cudaGetLastError();
}

cudaError_t zero_adam(const ZeroPeers& params, const ZeroPeers& grads, const int64_t* units,
                      int num_units,
                      const float* gshard, float* master, float* exp_avg, float* exp_avg_sq,
                      const float* hyper, const float* grad_scale, const float* skip_flag,
                      int sm_count, cudaStream_t stream) {
  if (num_units == 0) return cudaSuccess;
  const int parts = zero_reduce_parts(num_units, sm_count);
  zero_adam_kernel<<<parts, ZT, 0, stream>>>(params, grads, units, num_units, gshard, master, exp_avg,
                                             exp_avg_sq, hyper, grad_scale, skip_flag);
  return cudaGetLastError();
}

}  // namespace agb
