// Python bindings of the sm_100a kernels (torch tensors in, torch tensors out).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>

#include "agb.h"

namespace {

using torch::Tensor;

cudaStream_t stream_of(const Tensor& t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e), " (", agb::error_detail(), ")");
}

// One int32 status word per device; kernels write a non-zero code when a bounded wait
// ran out or an argument was rejected on the device.
Tensor status_word(int device) {
  static std::map<int, Tensor> words;
  auto it = words.find(device);
  if (it == words.end()) {
    auto w = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
    it = words.emplace(device, w).first;
  }
  return it->second;
}

int sm_count(int device) { return at::cuda::getDeviceProperties(device)->multiProcessorCount; }

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16, name, " must be a bf16 CUDA tensor");
}

// out = op(a) @ op(b) (+ bias) (+ residual) (+ out)
Tensor gemm(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b,
            c10::optional<Tensor> out_opt, bool accumulate, c10::optional<Tensor> bias,
            c10::optional<Tensor> residual, torch::ScalarType out_dtype) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm operands must be 2-D");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "gemm operands must have unit inner stride");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t m = trans_a ? a.size(1) : a.size(0);
  const int64_t k = trans_a ? a.size(0) : a.size(1);
  const int64_t n = trans_b ? b.size(0) : b.size(1);
  TORCH_CHECK((trans_b ? b.size(1) : b.size(0)) == k, "gemm inner dimensions differ");
  Tensor out;
  if (out_opt.has_value()) {
    out = *out_opt;
    TORCH_CHECK(out.dim() == 2 && out.size(0) == m && out.size(1) == n && out.stride(1) == 1,
                "gemm out has the wrong shape");
  } else {
    TORCH_CHECK(!accumulate, "accumulate needs out");
    out = torch::empty({m, n}, a.options().dtype(out_dtype));
  }
  TORCH_CHECK(out.scalar_type() == torch::kBFloat16 || out.scalar_type() == torch::kFloat32,
              "gemm out must be bf16 or fp32");
  agb::GemmArgs g{};
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.out = out.data_ptr();
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  g.ldo = out.stride(0);
  if (bias.has_value()) {
    check_bf16(*bias, "bias");
    TORCH_CHECK(bias->numel() == n && bias->is_contiguous(), "bias must be [N]");
    g.bias = bias->data_ptr();
  }
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    TORCH_CHECK(residual->dim() == 2 && residual->size(0) == m && residual->size(1) == n &&
                    residual->stride(1) == 1, "residual must be [M, N]");
    g.residual = residual->data_ptr();
    g.ldr = residual->stride(0);
  }
  g.m = int(m);
  g.n = int(n);
  g.k = int(k);
  g.a_mn_major = trans_a ? 1 : 0;
  g.b_mn_major = trans_b ? 0 : 1;
  g.out_fp32 = out.scalar_type() == torch::kFloat32;
  g.accumulate = accumulate;
  g.status = status_word(a.device().index()).data_ptr<int>();
  check(agb::gemm_bf16(g, sm_count(a.device().index()), stream_of(a)), "gemm_bf16");
  return out;
}

std::tuple<Tensor, Tensor> rms_norm_fwd(const Tensor& x, const Tensor& w, double eps) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  auto rstd = torch::empty({x.size(0)}, x.options().dtype(torch::kFloat32));
  check(agb::rms_norm_fwd(x.data_ptr(), nullptr, w.data_ptr(), nullptr, out.data_ptr(),
                          rstd.data_ptr<float>(), x.size(0), int(x.size(1)), float(eps),
                          stream_of(x)), "rms_norm_fwd");
  return {out, rstd};
}

std::tuple<Tensor, Tensor> rms_norm_add_fwd(const Tensor& x, const Tensor& addend, const Tensor& w,
                                            double eps) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  auto total = torch::empty_like(x);
  auto out = torch::empty_like(x);
  check(agb::rms_norm_fwd(x.data_ptr(), addend.data_ptr(), w.data_ptr(), total.data_ptr(),
                          out.data_ptr(), nullptr, x.size(0), int(x.size(1)), float(eps),
                          stream_of(x)), "rms_norm_add_fwd");
  return {total, out};
}

std::tuple<Tensor, Tensor> rms_norm_bwd(const Tensor& grad, const Tensor& x, const Tensor& w,
                                        const Tensor& rstd) {
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  const int parts = agb::rms_norm_bwd_partials(x.size(0));
  auto partial = torch::empty({parts, x.size(1)}, x.options().dtype(torch::kFloat32));
  check(agb::rms_norm_bwd(grad.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                          dx.data_ptr(), partial.data_ptr<float>(), x.size(0), int(x.size(1)),
                          stream_of(x)), "rms_norm_bwd");
  return {dx, partial.sum(0)};
}

// The same with `extra` (a gradient reaching x on another path) added before dx is rounded.
std::tuple<Tensor, Tensor> rms_norm_bwd_add(const Tensor& grad, const Tensor& x, const Tensor& w,
                                            const Tensor& rstd, const Tensor& extra) {
  check_bf16(extra, "extra");
  TORCH_CHECK(extra.is_contiguous() && extra.sizes() == x.sizes() && grad.is_contiguous() && x.is_contiguous(),
              "rms_norm_bwd_add: contiguous tensors of one shape");
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  const int parts = agb::rms_norm_bwd_partials(x.size(0));
  auto partial = torch::empty({parts, x.size(1)}, x.options().dtype(torch::kFloat32));
  check(agb::rms_norm_bwd(grad.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                          dx.data_ptr(), partial.data_ptr<float>(), x.size(0), int(x.size(1)),
                          stream_of(x), extra.data_ptr()), "rms_norm_bwd_add");
  return {dx, partial.sum(0)};
}

std::tuple<Tensor, Tensor> head_norm_rope_fwd(const Tensor& x, const Tensor& w, const Tensor& cosv,
                                              const Tensor& sinv, double eps) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 4 && x.size(3) == 128 && x.stride(3) == 1 && x.stride(2) == 128 &&
                  (x.size(0) == 1 || x.stride(0) == x.size(1) * x.stride(1)) && x.stride(1) % 8 == 0,
              "x must be [B, N, H, 128], dense over (H, 128), rows at a constant stride");
  TORCH_CHECK(cosv.is_contiguous() && sinv.is_contiguous() && cosv.numel() == x.size(0) * x.size(1) * 128,
              "cos/sin must be contiguous [B, N, 128]");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0) * x.size(1);
  const int heads = int(x.size(2));
  auto out = torch::empty(x.sizes(), x.options());
  auto rstd = torch::empty({rows, heads}, x.options().dtype(torch::kFloat32));
  check(agb::head_norm_rope_fwd(x.data_ptr(), w.data_ptr(), cosv.data_ptr(), sinv.data_ptr(),
                                out.data_ptr(), rstd.data_ptr<float>(), rows, heads, x.stride(1),
                                float(eps), stream_of(x)), "head_norm_rope_fwd");
  return {out, rstd};
}

// x may be a column slice of a wider matrix (rows at a constant stride); `out`, when given,
// receives dx and may be such a slice too.
std::tuple<Tensor, Tensor> head_norm_rope_bwd(const Tensor& grad, const Tensor& x, const Tensor& w,
                                              const Tensor& cosv, const Tensor& sinv,
                                              const Tensor& rstd, c10::optional<Tensor> out) {
  auto sliced = [](const Tensor& t) {
    return t.dim() == 4 && t.size(3) == 128 && t.stride(3) == 1 && t.stride(2) == 128 &&
           (t.size(0) == 1 || t.stride(0) == t.size(1) * t.stride(1)) && t.stride(1) % 8 == 0;
  };
  TORCH_CHECK(grad.is_contiguous() && sliced(x), "grad is contiguous, x is [B, N, H, 128] with rows at a constant stride");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0) * x.size(1);
  const int heads = int(x.size(2));
  Tensor dx = out.has_value() ? *out : torch::empty({x.size(0), x.size(1), x.size(2), 128}, x.options());
  TORCH_CHECK(sliced(dx) && dx.sizes() == x.sizes(), "out must have the shape of x and rows at a constant stride");
  const int parts = agb::head_norm_rope_bwd_partials(rows, heads);
  auto partial = torch::zeros({parts, 128}, x.options().dtype(torch::kFloat32));
  check(agb::head_norm_rope_bwd(grad.data_ptr(), x.data_ptr(), w.data_ptr(), cosv.data_ptr(),
                                sinv.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                                partial.data_ptr<float>(), rows, heads, x.stride(1), dx.stride(1),
                                stream_of(x)),
        "head_norm_rope_bwd");
  return {dx, partial.sum(0)};
}

Tensor silu_mul_fwd(const Tensor& gate, const Tensor& up) {
  check_bf16(gate, "gate");
  c10::cuda::CUDAGuard guard(gate.device());
  auto out = torch::empty_like(gate);
  check(agb::silu_mul_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(),
                          stream_of(gate)), "silu_mul_fwd");
  return out;
}

Tensor silu_mul_pair(const Tensor& both) {
  check_bf16(both, "both");
  TORCH_CHECK(both.dim() == 2 && both.is_contiguous() && both.size(1) % 16 == 0,
              "silu_mul_pair takes a contiguous [rows, 2 * width] matrix");
  c10::cuda::CUDAGuard guard(both.device());
  auto out = torch::empty({both.size(0), both.size(1) / 2}, both.options());
  check(agb::silu_mul_pair(both.data_ptr(), out.data_ptr(), both.size(0), int(both.size(1) / 2),
                           stream_of(both)), "silu_mul_pair");
  return out;
}

Tensor silu_mul_pair_bwd(const Tensor& grad, const Tensor& both) {
  check_bf16(both, "both");
  TORCH_CHECK(both.dim() == 2 && both.is_contiguous() && grad.is_contiguous() &&
                  grad.size(0) == both.size(0) && 2 * grad.size(1) == both.size(1) && grad.size(1) % 8 == 0,
              "silu_mul_pair_bwd takes grad [rows, width] and both [rows, 2 * width]");
  c10::cuda::CUDAGuard guard(both.device());
  auto dboth = torch::empty_like(both);
  check(agb::silu_mul_pair_bwd(grad.data_ptr(), both.data_ptr(), dboth.data_ptr(), both.size(0),
                               int(grad.size(1)), stream_of(both)), "silu_mul_pair_bwd");
  return dboth;
}

// (dboth, act): the gradient of both = [gate | up] and the forward activation, in one pass.
std::tuple<Tensor, Tensor> silu_mul_pair_bwd_act(const Tensor& grad, const Tensor& both) {
  check_bf16(both, "both");
  TORCH_CHECK(both.dim() == 2 && both.is_contiguous() && grad.is_contiguous() &&
                  grad.size(0) == both.size(0) && 2 * grad.size(1) == both.size(1) && grad.size(1) % 8 == 0,
              "silu_mul_pair_bwd_act takes grad [rows, width] and both [rows, 2 * width]");
  c10::cuda::CUDAGuard guard(both.device());
  auto dboth = torch::empty_like(both);
  auto act = torch::empty_like(grad);
  check(agb::silu_mul_pair_bwd(grad.data_ptr(), both.data_ptr(), dboth.data_ptr(), both.size(0),
                               int(grad.size(1)), stream_of(both), act.data_ptr()), "silu_mul_pair_bwd_act");
  return {dboth, act};
}

std::tuple<Tensor, Tensor> silu_mul_bwd(const Tensor& grad, const Tensor& gate, const Tensor& up) {
  c10::cuda::CUDAGuard guard(gate.device());
  auto dgate = torch::empty_like(gate);
  auto dup = torch::empty_like(gate);
  check(agb::silu_mul_bwd(grad.data_ptr(), gate.data_ptr(), up.data_ptr(), dgate.data_ptr(),
                          dup.data_ptr(), gate.numel(), stream_of(gate)), "silu_mul_bwd");
  return {dgate, dup};
}

Tensor rf_combine(const Tensor& a, const Tensor& b, const Tensor& sigma, int64_t mode) {
  TORCH_CHECK(a.dim() == 5 && a.is_contiguous() && b.is_contiguous(), "expected [B,C,T,H,W]");
  c10::cuda::CUDAGuard guard(a.device());
  auto out = torch::empty_like(a);
  const int sigma_frames = sigma.dim() == 1 ? 1 : int(sigma.size(1));
  check(agb::rf_combine(a.data_ptr(), b.data_ptr(), sigma.data_ptr<float>(), out.data_ptr(),
                        a.size(0), a.size(1), int(a.size(2)), int(a.size(3) * a.size(4)),
                        sigma_frames, int(mode), a.scalar_type() == torch::kBFloat16, stream_of(a)),
        "rf_combine");
  return out;
}

// q [B,NQ,Hq,128]; k/v [B,NK,Hkv,128]; optional text k/v [B,NT,Hkv,128]; returns (out, lse)
std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v,
                                    c10::optional<Tensor> text_k, c10::optional<Tensor> text_v,
                                    c10::optional<Tensor> text_valid, const Tensor& q_tiles,
                                    const Tensor& entries, double scale, int64_t key_splits) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_bf16(v, "v");
  TORCH_CHECK(q.dim() == 4 && q.size(3) == 128 && k.dim() == 4 && k.size(3) == 128, "head_dim must be 128");
  TORCH_CHECK(q.stride(3) == 1 && q.stride(2) == 128 && k.stride(3) == 1 && k.stride(2) == 128 &&
                  v.stride(3) == 1 && v.stride(2) == 128 && k.sizes() == v.sizes() &&
                  v.stride(1) % 8 == 0 && v.stride(0) % 8 == 0,
              "q/k/v must be dense over (head, dim)");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t splits = key_splits > 1 ? key_splits : 1;
  TORCH_CHECK(q_tiles.size(0) % splits == 0, "the tile list must hold key_splits copies of the query tiles");
  auto out = torch::empty({q.size(0), splits * q.size(1), q.size(2), 128}, q.options());
  auto lse = torch::empty({q.size(0), q.size(2), splits * q.size(1)}, q.options().dtype(torch::kFloat32));
  agb::AttnArgs a{};
  a.key_splits = int(splits);
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.out = out.data_ptr(); a.lse = lse.data_ptr<float>();
  a.q_tiles = q_tiles.data_ptr<int>(); a.entries = entries.data_ptr<int>();
  a.nq = q.size(1); a.nk = k.size(1); a.batch = q.size(0);
  a.q_row_stride = q.stride(1); a.q_batch_stride = q.stride(0);
  a.kv_row_stride = k.stride(1); a.kv_batch_stride = k.stride(0);
  a.v_row_stride = v.stride(1); a.v_batch_stride = v.stride(0);
  if (text_k.has_value()) {
    check_bf16(*text_k, "text_k");
    TORCH_CHECK(text_k->strides() == text_v->strides() && text_k->stride(2) == 128, "text k/v layout");
    a.text_k = text_k->data_ptr(); a.text_v = text_v->data_ptr();
    a.text_len = text_k->size(1);
    a.text_row_stride = text_k->stride(1); a.text_batch_stride = text_k->stride(0);
  }
  if (text_valid.has_value()) a.text_valid = text_valid->data_ptr<int>();
  a.hq = int(q.size(2)); a.hkv = int(k.size(2)); a.num_q_tiles = int(q_tiles.size(0));
  a.scale = float(scale);
  a.status = status_word(q.device().index()).data_ptr<int>();
  check(agb::attention_fwd(a, stream_of(q)), "attention_fwd");
  if (splits == 1) return {out, lse};
  auto merged = torch::empty({q.size(0), q.size(1), q.size(2), 128}, q.options());
  check(agb::attention_combine(out.data_ptr(), lse.data_ptr<float>(), merged.data_ptr(), q.size(0),
                               q.size(1), int(q.size(2)), int(splits), stream_of(q)),
        "attention_combine");
  return {merged, lse};
}

std::tuple<Tensor, Tensor, Tensor> attn_bwd(
    const Tensor& grad, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
    const Tensor& lse, c10::optional<Tensor> text_k, c10::optional<Tensor> text_v,
    c10::optional<Tensor> text_valid, const Tensor& q_tiles, const Tensor& entries,
    const Tensor& k_tiles, const Tensor& q_lists, double scale, c10::optional<Tensor> dv_out) {
  check_bf16(grad, "grad");
  TORCH_CHECK(grad.is_contiguous() && out.is_contiguous(), "grad/out must be contiguous");
  TORCH_CHECK(q.stride(2) == 128 && k.stride(2) == 128 && v.stride(2) == 128 && v.stride(3) == 1 &&
                  k.sizes() == v.sizes() && v.stride(1) % 8 == 0 && v.stride(0) % 8 == 0, "q/k/v layout");
  c10::cuda::CUDAGuard guard(q.device());
  auto dq = torch::empty({q.size(0), q.size(1), q.size(2), 128}, q.options());
  auto dk = torch::zeros({k.size(0), k.size(1), k.size(2), 128}, k.options());
  // dv_out: a caller-zeroed [B, NK, Hkv, 128] view (for example the v columns of a fused
  // gradient matrix); rows of keys that nothing attends to are left untouched.
  Tensor dv = dv_out.has_value() ? *dv_out : torch::zeros({k.size(0), k.size(1), k.size(2), 128}, k.options());
  TORCH_CHECK(dv.sizes() == k.sizes() && dv.stride(3) == 1 && dv.stride(2) == 128, "dv_out layout");
  auto delta = torch::empty({q.size(0), q.size(2), q.size(1)}, q.options().dtype(torch::kFloat32));
  agb::AttnBwdArgs b{};
  agb::AttnArgs& a = b.fwd;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.out = out.data_ptr(); a.lse = lse.data_ptr<float>();
  a.q_tiles = q_tiles.data_ptr<int>(); a.entries = entries.data_ptr<int>();
  a.nq = q.size(1); a.nk = k.size(1); a.batch = q.size(0);
  a.q_row_stride = q.stride(1); a.q_batch_stride = q.stride(0);
  a.kv_row_stride = k.stride(1); a.kv_batch_stride = k.stride(0);
  a.v_row_stride = v.stride(1); a.v_batch_stride = v.stride(0);
  if (text_k.has_value()) {
    a.text_k = text_k->data_ptr(); a.text_v = text_v->data_ptr();
    a.text_len = text_k->size(1);
    a.text_row_stride = text_k->stride(1); a.text_batch_stride = text_k->stride(0);
  }
  if (text_valid.has_value()) a.text_valid = text_valid->data_ptr<int>();
  a.hq = int(q.size(2)); a.hkv = int(k.size(2)); a.num_q_tiles = int(q_tiles.size(0));
  a.scale = float(scale);
  a.status = status_word(q.device().index()).data_ptr<int>();
  b.grad_out = grad.data_ptr();
  b.dq = dq.data_ptr(); b.dk = dk.data_ptr(); b.dv = dv.data_ptr();
  b.dv_row_stride = dv.stride(1); b.dv_batch_stride = dv.stride(0);
  b.delta = delta.data_ptr<float>();
  b.k_tiles = k_tiles.data_ptr<int>(); b.q_lists = q_lists.data_ptr<int>();
  b.num_k_tiles = int(k_tiles.size(0));
  check(agb::attention_bwd(b, stream_of(q)), "attention_bwd");
  return {dq, dk, dv};
}

// The same gradients from the one-pass kernel.  k_tiles_f / blocks_f come from the schedule
// (ops/attention.py::AttentionSchedule.fused); nq_pad is the query count rounded up to 128.
std::tuple<Tensor, Tensor, Tensor> attn_bwd_fused(
    const Tensor& grad, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
    const Tensor& lse, c10::optional<Tensor> text_k, c10::optional<Tensor> text_v,
    c10::optional<Tensor> text_valid, const Tensor& k_tiles_f, const Tensor& blocks_f, double scale,
    c10::optional<Tensor> dv_out) {
  check_bf16(grad, "grad");
  TORCH_CHECK(grad.is_contiguous() && out.is_contiguous(), "grad/out must be contiguous");
  TORCH_CHECK(q.stride(2) == 128 && k.stride(2) == 128 && v.stride(2) == 128 && v.stride(3) == 1 &&
                  k.sizes() == v.sizes() && v.stride(1) % 8 == 0 && v.stride(0) % 8 == 0, "q/k/v layout");
  TORCH_CHECK(k_tiles_f.dim() == 2 && k_tiles_f.size(1) == 5 && blocks_f.dim() == 2 && blocks_f.size(1) == 4 &&
                  k_tiles_f.is_contiguous() && blocks_f.is_contiguous(), "fused schedule layout");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t nq_pad = (q.size(1) + 127) / 128 * 128;
  auto dq = torch::empty({q.size(0), q.size(1), q.size(2), 128}, q.options());
  auto dk = torch::zeros({k.size(0), k.size(1), k.size(2), 128}, k.options());
  Tensor dv = dv_out.has_value() ? *dv_out : torch::zeros({k.size(0), k.size(1), k.size(2), 128}, k.options());
  TORCH_CHECK(dv.sizes() == k.sizes() && dv.stride(3) == 1 && dv.stride(2) == 128, "dv_out layout");
  auto delta = torch::empty({q.size(0), q.size(2), q.size(1)}, q.options().dtype(torch::kFloat32));
  auto dq_acc = torch::zeros({q.size(0), nq_pad, q.size(2), 128}, q.options().dtype(torch::kFloat32));
  auto turns = torch::zeros({1 + q.size(0) * q.size(2) * (nq_pad / 128)}, q.options().dtype(torch::kInt32));
  agb::AttnBwdArgs b{};
  agb::AttnArgs& a = b.fwd;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.out = out.data_ptr(); a.lse = lse.data_ptr<float>();
  a.nq = q.size(1); a.nk = k.size(1); a.batch = q.size(0);
  a.q_row_stride = q.stride(1); a.q_batch_stride = q.stride(0);
  a.kv_row_stride = k.stride(1); a.kv_batch_stride = k.stride(0);
  a.v_row_stride = v.stride(1); a.v_batch_stride = v.stride(0);
  if (text_k.has_value()) {
    a.text_k = text_k->data_ptr(); a.text_v = text_v->data_ptr();
    a.text_len = text_k->size(1);
    a.text_row_stride = text_k->stride(1); a.text_batch_stride = text_k->stride(0);
  }
  if (text_valid.has_value()) a.text_valid = text_valid->data_ptr<int>();
  a.hq = int(q.size(2)); a.hkv = int(k.size(2));
  a.scale = float(scale);
  a.status = status_word(q.device().index()).data_ptr<int>();
  b.grad_out = grad.data_ptr();
  b.dq = dq.data_ptr(); b.dk = dk.data_ptr(); b.dv = dv.data_ptr();
  b.dv_row_stride = dv.stride(1); b.dv_batch_stride = dv.stride(0);
  b.delta = delta.data_ptr<float>();
  b.num_k_tiles = int(k_tiles_f.size(0));
  check(agb::attention_bwd_fused(b, k_tiles_f.data_ptr<int>(), blocks_f.data_ptr<int>(),
                                 dq_acc.data_ptr<float>(), turns.data_ptr<int>(), nq_pad, stream_of(q)),
        "attention_bwd_fused");
  return {dq, dk, dv};
}

// Stride-1 convolution of a channels-last volume: x [B, Tin, H, W, Cin], weight
// [Cout, kt * kh * kw, Cin] -> [B, Tin - kt + 1, H, W, Cout] (+ bias [Cout], + residual like out,
// then ReLU when asked); bf16 or fp16 throughout.
Tensor conv3d(const Tensor& x, const Tensor& weight, c10::optional<Tensor> bias,
              c10::optional<Tensor> residual, int64_t kt, int64_t kh, int64_t kw, bool relu,
              c10::optional<Tensor> history, bool causal) {
  const auto dtype = x.scalar_type();
  TORCH_CHECK(x.is_cuda() && (dtype == torch::kBFloat16 || dtype == torch::kFloat16),
              "conv3d: x is a bf16 or fp16 CUDA tensor");
  auto same = [&](const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == dtype, "conv3d: ", name, " has the dtype of x");
  };
  same(weight, "weight");
  TORCH_CHECK(x.dim() == 5 && x.is_contiguous(), "conv3d: x is contiguous [B, T, H, W, Cin]");
  TORCH_CHECK(weight.dim() == 3 && weight.is_contiguous() && weight.size(1) == kt * kh * kw &&
                  weight.size(2) == x.size(4), "conv3d: weight is contiguous [Cout, taps, Cin]");
  TORCH_CHECK(causal || x.size(1) >= kt, "conv3d: fewer frames than the kernel is deep");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t frames_out = causal ? x.size(1) : x.size(1) - kt + 1;
  Tensor out = torch::empty({x.size(0), frames_out, x.size(2), x.size(3), weight.size(0)}, x.options());
  agb::ConvArgs a{};
  a.x = x.data_ptr();
  a.weight = weight.data_ptr();
  a.out = out.data_ptr();
  if (bias.has_value()) {
    same(*bias, "bias");
    TORCH_CHECK(bias->numel() == weight.size(0) && bias->is_contiguous(), "conv3d: bias is [Cout]");
    a.bias = bias->data_ptr();
  }
  if (residual.has_value()) {
    same(*residual, "residual");
    TORCH_CHECK(residual->sizes() == out.sizes() && residual->is_contiguous(),
                "conv3d: residual has the shape of the result, contiguous");
    a.residual = residual->data_ptr();
  }
  a.batch = int(x.size(0)); a.frames_in = int(x.size(1)); a.height = int(x.size(2));
  a.width = int(x.size(3)); a.cin = int(x.size(4)); a.cout = int(weight.size(0));
  a.kt = int(kt); a.kh = int(kh); a.kw = int(kw);
  a.relu = relu ? 1 : 0;
  a.fp16 = dtype == torch::kFloat16 ? 1 : 0;
  a.causal = causal ? 1 : 0;
  if (history.has_value() && history->size(1) > 0) {
    same(*history, "history");
    TORCH_CHECK(causal && history->dim() == 5 && history->is_contiguous() && history->size(0) == x.size(0) &&
                    history->size(2) == x.size(2) && history->size(3) == x.size(3) &&
                    history->size(4) == x.size(4) && history->size(1) <= kt - 1,
                "conv3d: history is contiguous [B, <= kt - 1, H, W, Cin] of a causal call");
    a.history = history->data_ptr();
    a.history_frames = int(history->size(1));
  }
  a.status = status_word(x.device().index()).data_ptr<int>();
  check(agb::conv3d_bf16(a, sm_count(x.device().index()), stream_of(x)), "conv3d");
  return out;
}

// AdaLN: rows of x [rows, H]; scale / shift / gate are [rows, H] column blocks (unit inner stride).
namespace {
void check_block(const Tensor& t, const Tensor& like, const char* name) {
  check_bf16(t, name);
  TORCH_CHECK(t.dim() == 2 && t.sizes() == like.sizes() && t.stride(1) == 1 && t.stride(0) % 8 == 0 &&
                  (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0,
              name, " must be a [rows, H] column block with 16-byte aligned rows");
}
}  // namespace

Tensor norm_modulate(const Tensor& x, const Tensor& w, const Tensor& scale, const Tensor& shift, double eps) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && w.numel() == x.size(1) && w.is_contiguous(),
              "norm_modulate: x [rows, H] contiguous, w [H]");
  check_block(scale, x, "scale");
  check_block(shift, x, "shift");
  TORCH_CHECK(scale.stride(0) == shift.stride(0), "scale and shift come from the same projection");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(x);
  check(agb::norm_modulate(x.data_ptr(), w.data_ptr(), scale.data_ptr(), shift.data_ptr(), out.data_ptr(),
                           x.size(0), int(x.size(1)), scale.stride(0), float(eps), stream_of(x)),
        "norm_modulate");
  return out;
}

Tensor gated_residual(const Tensor& hidden, const Tensor& gate, const Tensor& y) {
  check_bf16(hidden, "hidden");
  check_bf16(y, "y");
  TORCH_CHECK(hidden.dim() == 2 && hidden.is_contiguous() && y.is_contiguous() && y.sizes() == hidden.sizes(),
              "gated_residual: hidden and y are contiguous [rows, H]");
  check_block(gate, hidden, "gate");
  c10::cuda::CUDAGuard guard(hidden.device());
  Tensor out = torch::empty_like(hidden);
  check(agb::gated_residual(hidden.data_ptr(), gate.data_ptr(), y.data_ptr(), out.data_ptr(), hidden.size(0),
                            int(hidden.size(1)), gate.stride(0), stream_of(hidden)), "gated_residual");
  return out;
}

// Geometry preprocessing: depth [B, 1, T, H, W] fp32 -> RGB [B, 3, T, H, W]; uint8 normals -> unit vectors.
Tensor colorize_depth(const Tensor& depth, const Tensor& scale) {
  TORCH_CHECK(depth.is_cuda() && depth.scalar_type() == torch::kFloat32 && depth.dim() == 5 &&
                  depth.size(1) == 1 && depth.is_contiguous(), "colorize_depth: depth is contiguous fp32 [B, 1, T, H, W]");
  TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == torch::kFloat32 && scale.is_contiguous() &&
                  (scale.numel() == 1 || scale.numel() == depth.size(0)), "colorize_depth: scale is fp32 [B] or [1]");
  c10::cuda::CUDAGuard guard(depth.device());
  Tensor out = torch::empty({depth.size(0), 3, depth.size(2), depth.size(3), depth.size(4)}, depth.options());
  check(agb::colorize_depth(depth.data_ptr<float>(), scale.data_ptr<float>(), out.data_ptr<float>(),
                            depth.size(0), depth.numel() / depth.size(0), int(scale.numel()), stream_of(depth)),
        "colorize_depth");
  return out;
}

static void check_frames(const Tensor& t, int64_t dims, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous() && t.dim() == dims, what,
              ": contiguous fp32 CUDA tensor of ", dims, " dimensions");
}

// [..., H, W] -> [..., H / factor, W / factor]: window means, non-finite inputs as zero.
Tensor pool_frames(const Tensor& video, int64_t factor) {
  TORCH_CHECK(video.dim() >= 2, "pool_frames: at least [H, W]");
  check_frames(video, video.dim(), "pool_frames");
  const int64_t h = video.size(-2), w = video.size(-1);
  TORCH_CHECK(factor >= 1 && h >= factor && w >= factor, "pool_frames: the window does not fit the frame");
  c10::cuda::CUDAGuard guard(video.device());
  auto shape = video.sizes().vec();
  shape[shape.size() - 2] = h / factor;
  shape[shape.size() - 1] = w / factor;
  auto out = torch::empty(shape, video.options());
  check(agb::pool_frames(video.data_ptr<float>(), out.data_ptr<float>(), video.numel() / (h * w), int(h), int(w),
                         int(factor), stream_of(video)), "pool_frames");
  return out;
}

// Separable blur of [..., H, W] with the odd-length `taps` and replicated borders.
Tensor blur_frames(const Tensor& images, const Tensor& taps) {
  TORCH_CHECK(images.dim() >= 2, "blur_frames: at least [H, W]");
  check_frames(images, images.dim(), "blur_frames");
  TORCH_CHECK(taps.is_cuda() && taps.scalar_type() == torch::kFloat32 && taps.is_contiguous() &&
                  taps.numel() % 2 == 1, "blur_frames: taps is a contiguous fp32 vector of odd length");
  c10::cuda::CUDAGuard guard(images.device());
  const int64_t h = images.size(-2), w = images.size(-1);
  auto scratch = torch::empty_like(images), out = torch::empty_like(images);
  check(agb::blur_frames(images.data_ptr<float>(), scratch.data_ptr<float>(), out.data_ptr<float>(),
                         taps.data_ptr<float>(), int(taps.numel() / 2), images.numel() / std::max<int64_t>(h * w, 1),
                         int(h), int(w), stream_of(images)), "blur_frames");
  return out;
}

// [B, C, T, H, W] warped frame by frame: params [B, T, 8] fp32, copy [B, T] uint8.
Tensor warp_frames(const Tensor& video, const Tensor& params, const Tensor& copy) {
  check_frames(video, 5, "warp_frames");
  const int64_t b = video.size(0), t = video.size(2);
  TORCH_CHECK(params.is_cuda() && params.scalar_type() == torch::kFloat32 && params.is_contiguous() &&
                  params.numel() == b * t * 8, "warp_frames: params is contiguous fp32 [B, T, 8]");
  TORCH_CHECK(copy.is_cuda() && copy.scalar_type() == torch::kUInt8 && copy.is_contiguous() &&
                  copy.numel() == b * t, "warp_frames: copy is contiguous uint8 [B, T]");
  c10::cuda::CUDAGuard guard(video.device());
  auto out = torch::empty_like(video);
  check(agb::warp_frames(video.data_ptr<float>(), out.data_ptr<float>(), params.data_ptr<float>(),
                         copy.data_ptr<uint8_t>(), b, int(video.size(1)), int(t), int(video.size(3)),
                         int(video.size(4)), stream_of(video)), "warp_frames");
  return out;
}

// [..., H, W] -> [..., OH, OW]: mean over source bins (area = true) or bilinear sampling.
Tensor resize_frames(const Tensor& images, int64_t oh, int64_t ow, bool area) {
  TORCH_CHECK(images.dim() >= 2, "resize_frames: at least [H, W]");
  check_frames(images, images.dim(), "resize_frames");
  const int64_t h = images.size(-2), w = images.size(-1);
  TORCH_CHECK(h >= 1 && w >= 1 && oh >= 1 && ow >= 1, "resize_frames: empty extent");
  c10::cuda::CUDAGuard guard(images.device());
  auto shape = images.sizes().vec();
  shape[shape.size() - 2] = oh;
  shape[shape.size() - 1] = ow;
  auto out = torch::empty(shape, images.options());
  check(agb::resize_frames(images.data_ptr<float>(), out.data_ptr<float>(), images.numel() / (h * w), int(h),
                           int(w), int(oh), int(ow), area ? 1 : 0, stream_of(images)), "resize_frames");
  return out;
}

// [B, ..., H, W] -> [B, ..., TH, TW]: quadrant stretch; top / left are int32 [B] on the device.
Tensor stretch_frames(const Tensor& video, const Tensor& top, const Tensor& left, int64_t th, int64_t tw) {
  TORCH_CHECK(video.dim() >= 3, "stretch_frames: at least [B, H, W]");
  check_frames(video, video.dim(), "stretch_frames");
  const int64_t b = video.size(0), h = video.size(-2), w = video.size(-1);
  TORCH_CHECK(h >= 2 && w >= 2 && th >= h && tw >= w, "stretch_frames: the target is smaller than the frame");
  for (const Tensor* t : {&top, &left})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kInt32 && t->is_contiguous() && t->numel() == b,
                "stretch_frames: top and left are contiguous int32 [B] on the device");
  c10::cuda::CUDAGuard guard(video.device());
  auto shape = video.sizes().vec();
  shape[shape.size() - 2] = th;
  shape[shape.size() - 1] = tw;
  auto out = torch::empty(shape, video.options());
  check(agb::stretch_frames(video.data_ptr<float>(), out.data_ptr<float>(), top.data_ptr<int>(),
                            left.data_ptr<int>(), b, b ? video.numel() / (b * h * w) : 0, int(h), int(w), int(th),
                            int(tw), stream_of(video)), "stretch_frames");
  return out;
}

// Distribution-matching target: fp32 [B, ...] inputs -> (fp64 target, fp64 [B, blocks] sums of
// float(step)^2 whose total over the element count is the mean square of the step).
std::tuple<Tensor, Tensor> dmd_target(const Tensor& estimate, const Tensor& fake, const Tensor& teacher) {
  for (const Tensor* t : {&estimate, &fake, &teacher})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous() &&
                    t->sizes() == estimate.sizes() && t->dim() >= 2,
                "dmd_target: three contiguous fp32 CUDA tensors of one shape [B, ...]");
  c10::cuda::CUDAGuard guard(estimate.device());
  const int64_t b = estimate.size(0), per = b ? estimate.numel() / b : 0;
  const auto wide = estimate.options().dtype(torch::kFloat64);
  auto target = torch::empty(estimate.sizes(), wide);
  auto partial = torch::empty({b, agb::dmd_target_blocks()}, wide);
  auto squares = torch::zeros({b, agb::dmd_target_blocks()}, wide);
  check(agb::dmd_target(estimate.data_ptr<float>(), fake.data_ptr<float>(), teacher.data_ptr<float>(),
                        partial.data_ptr<double>(), target.data_ptr<double>(), squares.data_ptr<double>(), b, per,
                        stream_of(estimate)), "dmd_target");
  return {target, squares};
}

Tensor decode_normal(const Tensor& normal) {
  TORCH_CHECK(normal.is_cuda() && normal.scalar_type() == torch::kUInt8 && normal.dim() == 5 &&
                  normal.size(1) == 3 && normal.is_contiguous(), "decode_normal: normal is contiguous uint8 [B, 3, T, H, W]");
  c10::cuda::CUDAGuard guard(normal.device());
  Tensor out = torch::empty(normal.sizes(), normal.options().dtype(torch::kFloat32));
  check(agb::decode_normal(normal.data_ptr(), out.data_ptr<float>(), normal.size(0),
                           normal.numel() / normal.size(0) / 3, stream_of(normal)), "decode_normal");
  return out;
}

// Depthwise k x k convolution of channels-last frames: x [N, H, W, C], weight [k * k, C].
Tensor depthwise(const Tensor& x, const Tensor& weight, c10::optional<Tensor> bias, int64_t kernel) {
  const auto dtype = x.scalar_type();
  TORCH_CHECK(x.is_cuda() && (dtype == torch::kBFloat16 || dtype == torch::kFloat16) && x.dim() == 4 &&
                  x.is_contiguous(), "depthwise: x is a contiguous bf16 or fp16 CUDA tensor [N, H, W, C]");
  TORCH_CHECK(weight.is_cuda() && weight.scalar_type() == dtype && weight.is_contiguous() &&
                  weight.dim() == 2 && weight.size(0) == kernel * kernel && weight.size(1) == x.size(3),
              "depthwise: weight is [k * k, C] in the dtype of x");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(x);
  agb::DepthwiseArgs a{};
  a.x = x.data_ptr();
  a.weight = weight.data_ptr();
  a.out = out.data_ptr();
  if (bias.has_value()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == dtype && bias->is_contiguous() &&
                    bias->numel() == x.size(3), "depthwise: bias is [C] in the dtype of x");
    a.bias = bias->data_ptr();
  }
  a.frames = int(x.size(0)); a.height = int(x.size(1)); a.width = int(x.size(2));
  a.channels = int(x.size(3)); a.kernel = int(kernel);
  a.fp16 = dtype == torch::kFloat16 ? 1 : 0;
  check(agb::depthwise_conv(a, stream_of(x)), "depthwise");
  return out;
}

// Channel RMS norm (+ SiLU) of a channels-last activation; x is [..., C] with C contiguous.
Tensor channel_norm(const Tensor& x, const Tensor& gamma, bool silu) {
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && gamma.scalar_type() == torch::kFloat32 && gamma.is_contiguous() &&
                  gamma.numel() == x.size(-1), "channel_norm: x [..., C] contiguous, gamma fp32 [C]");
  c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  const int64_t channels = x.size(-1);
  check(agb::channel_norm(x.data_ptr(), gamma.data_ptr<float>(), out.data_ptr(), x.numel() / channels,
                          int(channels), silu ? 1 : 0, stream_of(x)), "channel_norm");
  return out;
}

// (O, tangent of O, LSE) of dense attention under forward-mode differentiation.
std::tuple<Tensor, Tensor, Tensor> attn_jvp(const Tensor& q, const Tensor& k, const Tensor& v,
                                            const Tensor& tq, const Tensor& tk, const Tensor& tv,
                                            double scale, int64_t text_len,
                                            c10::optional<Tensor> text_valid) {
  for (const Tensor* t : {&q, &k, &v, &tq, &tk, &tv}) {
    check_bf16(*t, "attn_jvp operand");
    TORCH_CHECK(t->dim() == 4 && t->size(3) == 128 && t->is_contiguous(),
                "attn_jvp operands are contiguous [B, N, H, 128]");
  }
  TORCH_CHECK(tq.sizes() == q.sizes() && tk.sizes() == k.sizes() && tv.sizes() == v.sizes() &&
                  k.sizes() == v.sizes() && k.size(0) == q.size(0), "attn_jvp shapes disagree");
  c10::cuda::CUDAGuard guard(q.device());
  auto f32 = q.options().dtype(torch::kFloat32);
  Tensor out = torch::empty(q.sizes(), f32), tangent = torch::empty(q.sizes(), f32);
  Tensor lse = torch::empty({q.size(0), q.size(2), q.size(1)}, f32);
  agb::AttnJvpArgs a{};
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.tq = tq.data_ptr(); a.tk = tk.data_ptr(); a.tv = tv.data_ptr();
  a.out = out.data_ptr<float>(); a.tangent = tangent.data_ptr<float>(); a.lse = lse.data_ptr<float>();
  if (text_valid.has_value()) {
    TORCH_CHECK(text_valid->scalar_type() == torch::kInt32 && text_valid->numel() == q.size(0) &&
                    text_valid->is_cuda(), "text_valid must be int32 [B] on the device");
    a.text_valid = text_valid->data_ptr<int>();
  }
  a.nq = q.size(1); a.nk = k.size(1); a.text_len = text_len; a.batch = q.size(0);
  a.q_row_stride = q.stride(1); a.q_batch_stride = q.stride(0);
  a.kv_row_stride = k.stride(1); a.kv_batch_stride = k.stride(0);
  a.hq = int(q.size(2)); a.hkv = int(k.size(2));
  a.scale = float(scale);
  a.status = status_word(q.device().index()).data_ptr<int>();
  check(agb::attention_jvp(a, stream_of(q)), "attention_jvp");
  return {out, tangent, lse};
}

// ---------------------------------------------------------------- tensor-parallel serving
// out = a @ b^T coupled to the peers (see agb::TpLink).  With a_ready the producer waits for
// pushed rows of `a`; with slot_ptrs the output goes to the owners' partial-sum slots and
// `out` is not used.
void tp_gemm(const Tensor& a, const Tensor& b, c10::optional<Tensor> out, int64_t rank, int64_t world,
             c10::optional<Tensor> a_ready, c10::optional<Tensor> a_seen, c10::optional<Tensor> ticket,
             std::vector<int64_t> slot_ptrs, std::vector<int64_t> arrive_ptrs, int64_t tiles_owned) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 &&
                  a.size(1) == b.size(1), "tp_gemm operands must be [M, K] and [N, K]");
  c10::cuda::CUDAGuard guard(a.device());
  agb::TpLink link{};
  link.rank = int(rank);
  link.world = int(world);
  if (a_ready.has_value()) {
    TORCH_CHECK(a_seen.has_value(), "a_ready needs a_seen");
    TORCH_CHECK(a_ready->numel() >= (a.size(0) + 127) / 128 && a_seen->numel() >= (a.size(0) + 127) / 128,
                "a_ready / a_seen are too short");
    link.wait_a = 1;
    link.a_ready = a_ready->data_ptr<int>();
    link.a_seen = a_seen->data_ptr<int>();
    link.ticket = ticket.has_value() ? ticket->data_ptr<int>() : nullptr;  // null: use stays open
  }
  agb::GemmArgs g{};
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  g.m = int(a.size(0));
  g.n = int(b.size(0));
  g.k = int(a.size(1));
  if (!slot_ptrs.empty()) {
    TORCH_CHECK(int64_t(slot_ptrs.size()) == world && int64_t(arrive_ptrs.size()) == world,
                "one slot and one arrival pointer per rank");
    link.push = 1;
    link.tiles_owned = int(tiles_owned);
    for (int64_t i = 0; i < world; ++i) {
      link.slot[i] = reinterpret_cast<void*>(slot_ptrs[i]);
      link.arrive[i] = reinterpret_cast<int*>(arrive_ptrs[i]);
    }
    g.ldo = g.n;
  } else {
    TORCH_CHECK(out.has_value() && out->dim() == 2 && out->size(0) == a.size(0) &&
                    out->size(1) == b.size(0) && out->stride(1) == 1, "tp_gemm out has the wrong shape");
    check_bf16(*out, "out");
    g.out = out->data_ptr();
    g.ldo = out->stride(0);
  }
  g.status = status_word(a.device().index()).data_ptr<int>();
  g.tp = &link;
  check(agb::gemm_bf16(g, sm_count(a.device().index()), stream_of(a)), "tp_gemm");
}

void tp_reduce_norm(int64_t rank, int64_t world, int64_t m, const Tensor& slot, const Tensor& arrive,
                    const Tensor& arrive_seen, const Tensor& ticket, int64_t arrivals_per_source,
                    const Tensor& hidden_own, c10::optional<Tensor> seed, const Tensor& weight,
                    double eps, std::vector<int64_t> xbuf_ptrs, std::vector<int64_t> ready_ptrs,
                    int64_t tiles_owned, const Tensor& done, const Tensor& done_uses,
                    int64_t rows_per_cta) {
  check_bf16(hidden_own, "hidden_own");
  check_bf16(weight, "weight");
  c10::cuda::CUDAGuard guard(hidden_own.device());
  TORCH_CHECK(int64_t(xbuf_ptrs.size()) == world && int64_t(ready_ptrs.size()) == world,
              "one buffer and one counter pointer per rank");
  TORCH_CHECK(hidden_own.dim() == 2 && hidden_own.size(0) >= tiles_owned * 128 &&
                  hidden_own.is_contiguous(), "hidden_own must be [tiles_owned * 128, width]");
  agb::TpReduceArgs a{};
  a.rank = int(rank);
  a.world = int(world);
  a.m = int(m);
  a.width = int(hidden_own.size(1));
  a.tiles_owned = int(tiles_owned);
  a.slot = slot.data_ptr();
  a.arrive = arrive.data_ptr<int>();
  TORCH_CHECK(arrive_seen.numel() >= tiles_owned, "arrive_seen is too short");
  a.arrive_seen = arrive_seen.data_ptr<int>();
  a.ticket = ticket.data_ptr<int>();
  a.arrivals_per_source = int(arrivals_per_source);
  a.hidden_own = hidden_own.data_ptr();
  if (seed.has_value()) {
    check_bf16(*seed, "seed");
    TORCH_CHECK(seed->is_contiguous() && seed->numel() == m * hidden_own.size(1), "seed must be [m, width]");
    a.seed = seed->data_ptr();
  }
  a.rows_per_cta = int(rows_per_cta);
  a.done = done.data_ptr<int>();
  a.done_uses = done_uses.data_ptr<int>();
  a.weight = weight.data_ptr();
  a.eps = float(eps);
  for (int64_t i = 0; i < world; ++i) {
    a.xbuf[i] = reinterpret_cast<void*>(xbuf_ptrs[i]);
    a.ready[i] = reinterpret_cast<int*>(ready_ptrs[i]);
  }
  a.status = status_word(hidden_own.device().index()).data_ptr<int>();
  check(agb::tp_reduce_norm(a, stream_of(hidden_own)), "tp_reduce_norm");
}

void tp_signal_done(std::vector<int64_t> done_ptrs, const Tensor& anchor) {
  c10::cuda::CUDAGuard guard(anchor.device());
  TORCH_CHECK(!done_ptrs.empty() && done_ptrs.size() <= 8, "1..8 ranks");
  int* done[8] = {};
  for (size_t i = 0; i < done_ptrs.size(); ++i) done[i] = reinterpret_cast<int*>(done_ptrs[i]);
  check(agb::tp_signal_done(done, int(done_ptrs.size()), stream_of(anchor)), "tp_signal_done");
}

// All-to-all over peer memory: out[s] = send_of_rank_s[rank]; send / out are [world, ...] contiguous.
void exchange(const Tensor& send, const Tensor& out, std::vector<int64_t> recv_ptrs,
              std::vector<int64_t> arrive_ptrs, const Tensor& state, int64_t half_bytes, int64_t rank) {
  TORCH_CHECK(send.is_cuda() && out.is_cuda() && send.is_contiguous() && out.is_contiguous() &&
                  send.nbytes() == out.nbytes() && send.dim() >= 1,
              "exchange: send and out are contiguous CUDA tensors of one size");
  const int64_t world = int64_t(recv_ptrs.size());
  TORCH_CHECK(world >= 1 && world <= 8 && arrive_ptrs.size() == recv_ptrs.size() && send.size(0) == world,
              "exchange: 1..8 ranks, dim 0 of send is the destination rank");
  TORCH_CHECK(state.is_cuda() && state.scalar_type() == torch::kInt32 && state.numel() >= 2 &&
                  state.is_contiguous(), "exchange: state is int32 [2] (count, ticket)");
  c10::cuda::CUDAGuard guard(send.device());
  agb::ExchangeArgs a{};
  a.send = send.data_ptr();
  a.out = out.data_ptr();
  for (int64_t i = 0; i < world; ++i) {
    a.recv[i] = reinterpret_cast<void*>(recv_ptrs[i]);
    a.arrive[i] = reinterpret_cast<int*>(arrive_ptrs[i]);
  }
  a.count = state.data_ptr<int>();
  a.ticket = state.data_ptr<int>() + 1;
  a.bytes_per_rank = int64_t(send.nbytes()) / world;
  a.half_bytes = half_bytes;
  a.rank = int(rank);
  a.world = int(world);
  a.status = status_word(send.device().index()).data_ptr<int>();
  check(agb::exchange_all_to_all(a, sm_count(send.device().index()), stream_of(send)), "exchange");
}

agb::ZeroPeers peers_of(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(!ptrs.empty() && ptrs.size() <= 8, "1..8 peers supported");
  agb::ZeroPeers p{};
  p.world = int(ptrs.size());
  for (size_t i = 0; i < ptrs.size(); ++i) p.ptr[i] = reinterpret_cast<void*>(ptrs[i]);
  return p;
}

// gshard <- mean over ranks of the owned gradient ranges; stats[0] = sum of squares,
// stats[1] = 1 if any value is not finite.
void zero_reduce(std::vector<int64_t> grad_ptrs, const Tensor& units,
                 c10::optional<Tensor> gshard_opt, const Tensor& stats) {
  c10::cuda::CUDAGuard guard(stats.device());
  const int dev = stats.device().index();
  float* gshard_ptr = gshard_opt.has_value() ? gshard_opt->data_ptr<float>() : nullptr;
  const int n = int(units.size(0));
  const int parts = agb::zero_reduce_parts(n, sm_count(dev));
  auto psum = torch::empty({parts}, stats.options());
  auto pbad = torch::empty({parts}, stats.options().dtype(torch::kInt32));
  check(agb::zero_reduce(peers_of(grad_ptrs), units.data_ptr<int64_t>(), n, gshard_ptr,
                         psum.data_ptr<float>(), pbad.data_ptr<int>(), stats.data_ptr<float>(),
                         stats.data_ptr<float>() + 1, sm_count(dev), stream_of(stats)),
        "zero_reduce");
}

constexpr uint64_t kGradientWaitNs = 30ull * 1000000000ull;  // ranks may be seconds apart in a step

// One bucket of the reduce: units [begin, end), partials written at [part_offset, part_offset + parts).
void zero_reduce_range(std::vector<int64_t> grad_ptrs, const Tensor& units, int64_t begin, int64_t end,
                       c10::optional<Tensor> gshard_opt, const Tensor& psum, const Tensor& pbad,
                       int64_t part_offset, int64_t parts, c10::optional<Tensor> ready,
                       int64_t ready_slot, int64_t ready_target, int64_t write_back_rank) {
  c10::cuda::CUDAGuard guard(psum.device());
  TORCH_CHECK(part_offset + parts <= psum.numel() && psum.numel() == pbad.numel(), "partial buffers too small");
  const int dev = psum.device().index();
  check(agb::zero_reduce_range(
            peers_of(grad_ptrs), units.data_ptr<int64_t>(), int(begin), int(end),
            gshard_opt.has_value() ? gshard_opt->data_ptr<float>() : nullptr,
            psum.data_ptr<float>() + part_offset, pbad.data_ptr<int>() + part_offset, int(parts),
            ready.has_value() ? ready->data_ptr<int>() + ready_slot : nullptr, int(ready_target),
            status_word(dev).data_ptr<int>(), kGradientWaitNs, int(write_back_rank), stream_of(psum)),
        "zero_reduce_range");
}

void zero_signal(std::vector<int64_t> counter_ptrs, int64_t slot, const Tensor& anchor) {
  c10::cuda::CUDAGuard guard(anchor.device());
  check(agb::zero_signal(peers_of(counter_ptrs), int(slot), stream_of(anchor)), "zero_signal");
}

void zero_wait(const Tensor& counters, int64_t slot, int64_t target) {
  c10::cuda::CUDAGuard guard(counters.device());
  check(agb::zero_wait(counters.data_ptr<int>() + slot, int(target),
                       status_word(counters.device().index()).data_ptr<int>(), kGradientWaitNs,
                       stream_of(counters)), "zero_wait");
}

void zero_stats(const Tensor& psum, const Tensor& pbad, int64_t parts, std::vector<int64_t> table_ptrs,
                int64_t rank, int64_t epoch, const Tensor& stats) {
  c10::cuda::CUDAGuard guard(stats.device());
  agb::ZeroPeers tables = table_ptrs.empty() ? agb::ZeroPeers{} : peers_of(table_ptrs);
  if (table_ptrs.empty()) tables.world = 1;
  check(agb::zero_stats(psum.data_ptr<float>(), pbad.data_ptr<int>(), int(parts), tables, int(rank),
                        int(epoch), stats.data_ptr<float>(), stats.data_ptr<float>() + 1,
                        status_word(stats.device().index()).data_ptr<int>(), kGradientWaitNs,
                        stream_of(stats)), "zero_stats");
}

void zero_adam(std::vector<int64_t> param_ptrs, std::vector<int64_t> grad_ptrs,
               const Tensor& units, c10::optional<Tensor> gshard, const Tensor& master, const Tensor& exp_avg, const Tensor& exp_avg_sq,
               const Tensor& hyper, c10::optional<Tensor> grad_scale,
               c10::optional<Tensor> skip_flag) {
  c10::cuda::CUDAGuard guard(master.device());
  const int dev = master.device().index();
  check(agb::zero_adam(peers_of(param_ptrs), peers_of(grad_ptrs), units.data_ptr<int64_t>(),
                       int(units.size(0)),
                       gshard.has_value() ? gshard->data_ptr<float>() : nullptr,
                       master.data_ptr<float>(),
                       exp_avg.data_ptr<float>(), exp_avg_sq.data_ptr<float>(),
                       hyper.data_ptr<float>(),
                       grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr,
                       skip_flag.has_value() ? skip_flag->data_ptr<float>() : nullptr,
                       sm_count(dev), stream_of(master)), "zero_adam");
}

// src/dst: [tokens, heads, 128] bf16 views (dst may be larger); cos/sin fp32 [kept, 128].
void relocate(const Tensor& src, const Tensor& dst, int64_t kept_tokens, int64_t sink_tokens,
              int64_t shift_tokens, c10::optional<Tensor> cosv, c10::optional<Tensor> sinv) {
  check_bf16(src, "src");
  check_bf16(dst, "dst");
  TORCH_CHECK(src.dim() == 3 && src.size(2) == 128 && src.is_contiguous() && dst.is_contiguous(),
              "cache rows must be contiguous [tokens, heads, 128]");
  TORCH_CHECK(kept_tokens <= dst.size(0) && kept_tokens + shift_tokens <= src.size(0) + 0,
              "relocate range exceeds the cache");
  c10::cuda::CUDAGuard guard(src.device());
  const float* c = nullptr;
  const float* s = nullptr;
  if (cosv.has_value()) {
    TORCH_CHECK(cosv->scalar_type() == torch::kFloat32 && cosv->is_contiguous() &&
                    cosv->size(0) >= kept_tokens && cosv->size(1) == 128, "cos must be fp32 [kept,128]");
    c = cosv->data_ptr<float>();
    s = sinv->data_ptr<float>();
  }
  check(agb::relocate_rows(src.data_ptr(), dst.data_ptr(), c, s, kept_tokens, int(sink_tokens),
                           int(shift_tokens), int(src.size(1)), stream_of(src)), "relocate_rows");
}

Tensor status(int64_t device) { return status_word(int(device)); }

}  // namespace

// cos / sin tables of the 3-axis RoPE: positions [..., 3] fp32, inverse [64] fp32, axis [64] int32.
std::tuple<Tensor, Tensor> rope_tables(const Tensor& positions, const Tensor& inverse, const Tensor& axis,
                                       bool bf16_out) {
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == torch::kFloat32 && positions.is_contiguous() &&
                  positions.size(-1) == 3, "positions: contiguous fp32 [..., 3]");
  TORCH_CHECK(inverse.scalar_type() == torch::kFloat32 && inverse.numel() == 64 && inverse.is_contiguous() &&
                  axis.scalar_type() == torch::kInt32 && axis.numel() == 64 && axis.is_contiguous(),
              "inverse fp32 [64], axis int32 [64]");
  c10::cuda::CUDAGuard guard(positions.device());
  auto shape = positions.sizes().vec();
  shape.back() = 128;
  auto options = positions.options().dtype(bf16_out ? torch::kBFloat16 : torch::kFloat32);
  auto cosine = torch::empty(shape, options), sine = torch::empty(shape, options);
  check(agb::rope_tables(positions.data_ptr<float>(), inverse.data_ptr<float>(), axis.data_ptr<int>(),
                         cosine.data_ptr(), sine.data_ptr(), positions.numel() / 3, bf16_out,
                         stream_of(positions)), "rope_tables");
  return {cosine, sine};
}

// [B, C, T, H, W] -> [B, T, (H/p)(W/p), p*p*C] (to_patches) or back, fp32 / bf16 on either side.
Tensor patch_layout(const Tensor& src, int64_t channels, int64_t height, int64_t width, int64_t patch,
                    bool to_patches, bool bf16_out) {
  const auto in = src.scalar_type();
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && (in == torch::kFloat32 || in == torch::kBFloat16),
              "patch_layout: contiguous fp32 or bf16 CUDA tensor");
  TORCH_CHECK(patch >= 1 && height % patch == 0 && width % patch == 0, "patch does not divide the frame");
  c10::cuda::CUDAGuard guard(src.device());
  int64_t batch, frames;
  Tensor dst;
  auto options = src.options().dtype(bf16_out ? torch::kBFloat16 : torch::kFloat32);
  if (to_patches) {
    TORCH_CHECK(src.dim() == 5 && src.size(1) == channels && src.size(3) == height && src.size(4) == width,
                "patch_layout: latent is [B, C, T, H, W]");
    batch = src.size(0); frames = src.size(2);
    dst = torch::empty({batch, frames, (height / patch) * (width / patch), patch * patch * channels}, options);
  } else {
    TORCH_CHECK(src.dim() == 4 && src.size(2) == (height / patch) * (width / patch) &&
                    src.size(3) == patch * patch * channels, "patch_layout: patches are [B, T, N, p*p*C]");
    batch = src.size(0); frames = src.size(1);
    dst = torch::empty({batch, channels, frames, height, width}, options);
  }
  check(agb::patch_layout(src.data_ptr(), dst.data_ptr(), batch, channels, frames, height, width, int(patch),
                          to_patches, in == torch::kBFloat16, bf16_out, stream_of(src)), "patch_layout");
  return dst;
}

// Element-wise maximum of a few int32 values over the GPUs of a node through the switch.
void multimem_max(const Tensor& buffer, int64_t multicast_ptr, const Tensor& state, const Tensor& values,
                  const Tensor& out, int64_t world, int64_t rank, int64_t limit_ns) {
  TORCH_CHECK(buffer.is_cuda() && buffer.scalar_type() == torch::kInt32 && buffer.numel() >= 65 &&
                  state.scalar_type() == torch::kInt32 && values.scalar_type() == torch::kInt32 &&
                  out.scalar_type() == torch::kInt32 && values.is_contiguous() && out.is_contiguous() &&
                  values.numel() == out.numel() && values.numel() >= 1 && values.numel() <= 32,
              "multimem_max: int32 buffers, 1..32 values");
  TORCH_CHECK(multicast_ptr != 0, "multimem_max: no multicast mapping");
  c10::cuda::CUDAGuard guard(buffer.device());
  check(agb::multimem_max(buffer.data_ptr(), reinterpret_cast<void*>(multicast_ptr), state.data_ptr<int>(),
                          reinterpret_cast<const uint32_t*>(values.data_ptr<int>()),
                          reinterpret_cast<uint32_t*>(out.data_ptr<int>()), int(values.numel()), int(world),
                          int(rank), status_word(buffer.device().index()).data_ptr<int>(), uint64_t(limit_ns),
                          stream_of(buffer)), "multimem_max");
}

// All-gather / broadcast through multicast stores: `part` (uint8, may be empty) lands at `offset`
// of a payload of out.numel() bytes on every GPU; `out` receives the whole payload.
void multimem_share(const Tensor& buffer, int64_t multicast_ptr, const Tensor& state, const Tensor& part,
                    int64_t offset, const Tensor& out, int64_t world, int64_t limit_ns) {
  TORCH_CHECK(buffer.is_cuda() && buffer.is_contiguous() && state.is_cuda() &&
                  state.scalar_type() == torch::kInt32 && state.numel() >= 2 &&
                  part.scalar_type() == torch::kUInt8 && out.scalar_type() == torch::kUInt8 &&
                  part.is_contiguous() && out.is_contiguous() && out.is_cuda(),
              "multimem_share: contiguous byte tensors on the device");
  TORCH_CHECK(multicast_ptr != 0, "multimem_share: no multicast mapping");
  c10::cuda::CUDAGuard guard(buffer.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  check(agb::multimem_share(buffer.data_ptr(), reinterpret_cast<void*>(multicast_ptr),
                            int64_t(buffer.numel()) * int64_t(buffer.element_size()), state.data_ptr<int>(),
                            part.numel() ? part.data_ptr() : nullptr, part.numel(), offset, out.data_ptr(),
                            out.numel(), int(world), sms, status_word(buffer.device().index()).data_ptr<int>(),
                            uint64_t(limit_ns), stream_of(buffer)), "multimem_share");
}
int64_t multimem_share_capacity(int64_t buffer_bytes) { return agb::multimem_share_capacity(buffer_bytes); }

// A few FP32 rows through a wide linear layer in FP32, weights read as they are (bf16 or fp32).
Tensor rows_linear_fwd(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias) {
  const auto wt = w.scalar_type();
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kFloat32 && x.dim() == 2 && x.is_contiguous() &&
                  w.dim() == 2 && w.is_contiguous() && w.size(1) == x.size(1) &&
                  (wt == torch::kBFloat16 || wt == torch::kFloat32), "rows_linear: x fp32 [m, k], w [n, k]");
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == wt && bias->is_contiguous() && bias->numel() == w.size(0), "rows_linear: bias");
  }
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({x.size(0), w.size(0)}, x.options());
  check(agb::rows_linear_fwd(x.data_ptr<float>(), w.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr,
                             y.data_ptr<float>(), int(x.size(0)), int(w.size(0)), int(x.size(1)),
                             wt == torch::kBFloat16, stream_of(x)), "rows_linear_fwd");
  return y;
}

std::tuple<Tensor, Tensor, Tensor> rows_linear_bwd(const Tensor& dy, const Tensor& x, const Tensor& w,
                                                   bool need_dx, bool need_dw) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == torch::kFloat32 && dy.is_contiguous() && dy.dim() == 2 &&
                  x.scalar_type() == torch::kFloat32 && x.is_contiguous() && x.size(0) == dy.size(0) &&
                  w.is_contiguous() && w.size(0) == dy.size(1) && w.size(1) == x.size(1), "rows_linear_bwd shapes");
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor dx, dw, db, partial;
  TORCH_CHECK(x.size(1) % 8 == 0, "rows_linear: the input width must be a multiple of 8");
  if (need_dx) {
    dx = torch::empty_like(x);
    partial = torch::empty({agb::rows_linear_slices(int(dy.size(1))), x.size(0), x.size(1)}, x.options());
  }
  if (need_dw) {
    dw = torch::empty({w.size(0), w.size(1)}, dy.options());
    db = torch::empty({w.size(0)}, dy.options());
  }
  check(agb::rows_linear_bwd(dy.data_ptr<float>(), x.data_ptr<float>(), w.data_ptr(),
                             need_dx ? dx.data_ptr<float>() : nullptr,
                             need_dx ? partial.data_ptr<float>() : nullptr, need_dw ? dw.data_ptr<float>() : nullptr,
                             need_dw ? db.data_ptr<float>() : nullptr, int(dy.size(0)), int(dy.size(1)),
                             int(x.size(1)), w.scalar_type() == torch::kBFloat16, stream_of(dy)), "rows_linear_bwd");
  return {dx, dw, db};
}

// Cycles per tcgen05.mma (M 128, K 16) issued back to back; see csrc/mma_rate.cu.
double mma_issue_rate(int64_t columns, bool a_from_tmem, int64_t iterations) {
  const int device = c10::cuda::current_device();
  c10::cuda::CUDAGuard guard(device);
  auto cycles = torch::zeros({1}, torch::dtype(torch::kInt64).device(torch::kCUDA, device));
  auto stream = c10::cuda::getCurrentCUDAStream(device).stream();
  check(agb::mma_issue_rate(int(columns), a_from_tmem, int(iterations), sm_count(device),
                            reinterpret_cast<long long*>(cycles.data_ptr<int64_t>()),
                            status_word(device).data_ptr<int>(), stream), "mma_issue_rate");
  const int64_t total = cycles.item<int64_t>();
  TORCH_CHECK(total >= 0, "mma_issue_rate: the bounded wait gave up");
  return double(total) / double(iterations * 8);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("mma_issue_rate", &mma_issue_rate);
  m.def("rows_linear_fwd", &rows_linear_fwd);
  m.def("rows_linear_bwd", &rows_linear_bwd);
  m.def("multimem_max", &multimem_max);
  m.def("multimem_share", &multimem_share);
  m.def("multimem_share_capacity", &multimem_share_capacity);
  m.def("rope_tables", &rope_tables);
  m.def("patch_layout", &patch_layout);
  m.def("gemm", &gemm);
  m.def("rms_norm_fwd", &rms_norm_fwd);
  m.def("rms_norm_add_fwd", &rms_norm_add_fwd);
  m.def("rms_norm_bwd", &rms_norm_bwd);
  m.def("rms_norm_bwd_add", &rms_norm_bwd_add);
  m.def("head_norm_rope_fwd", &head_norm_rope_fwd);
  m.def("head_norm_rope_bwd", &head_norm_rope_bwd);
  m.def("silu_mul_fwd", &silu_mul_fwd);
  m.def("silu_mul_bwd", &silu_mul_bwd);
  m.def("silu_mul_pair", &silu_mul_pair);
  m.def("silu_mul_pair_bwd", &silu_mul_pair_bwd);
  m.def("silu_mul_pair_bwd_act", &silu_mul_pair_bwd_act);
  m.def("rf_combine", &rf_combine);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("attn_bwd_fused", &attn_bwd_fused);
  m.def("relocate", &relocate);
  m.def("zero_reduce", &zero_reduce);
  m.def("zero_adam", &zero_adam);
  m.def("zero_reduce_range", &zero_reduce_range);
  m.def("zero_signal", &zero_signal);
  m.def("zero_wait", &zero_wait);
  m.def("zero_stats", &zero_stats);
  m.def("channel_norm", &channel_norm);
  m.def("conv3d", &conv3d);
  m.def("depthwise", &depthwise);
  m.def("colorize_depth", &colorize_depth);
  m.def("decode_normal", &decode_normal);
  m.def("pool_frames", &pool_frames);
  m.def("blur_frames", &blur_frames);
  m.def("warp_frames", &warp_frames);
  m.def("resize_frames", &resize_frames);
  m.def("stretch_frames", &stretch_frames);
  m.def("dmd_target", &dmd_target);
  m.def("norm_modulate", &norm_modulate);
  m.def("gated_residual", &gated_residual);
  m.def("attn_jvp", &attn_jvp);
  m.def("tp_gemm", &tp_gemm);
  m.def("tp_reduce_norm", &tp_reduce_norm);
  m.def("tp_signal_done", &tp_signal_done);
  m.def("exchange", &exchange);
  m.def("status", &status);
}
