// Host-callable launchers of the sm_100a kernels (plain C++ interface, no torch types).
// Every launcher enqueues on the given stream and returns a cudaError_t; none allocates.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace agb {

// Human-readable reason of the last failure reported by a launcher on this host thread.
void set_error_detail(const char* text);
const char* error_detail();

// ------------------------------------------------------------------------------- GEMM
// out[M, N] (+)= op(A) * op(B)^T-style product with bf16 inputs and fp32 accumulation.
//   a_mn_major = 0: A stored [M, K] (K contiguous);  1: A stored [K, M] (M contiguous)
//   b_mn_major = 0: B stored [N, K] (K contiguous);  1: B stored [K, N] (N contiguous)
// Strides (lda, ldb) are in elements of the stored row.  Epilogue, in this order:
//   acc (+ bias[n]) (+ residual[m, n]) (+ out[m, n] if accumulate) -> out (bf16 or fp32)
struct GemmArgs {
  const void* a;
  const void* b;
  void* out;
  const void* bias;      // bf16 [N] or null
  const void* residual;  // bf16 [M, N] (ld = ldr) or null
  int64_t lda, ldb, ldo, ldr;
  int m, n, k;
  int a_mn_major, b_mn_major;
  int out_fp32;    // 1: out is float, 0: out is bf16
  int accumulate;  // 1: add the previous contents of out
  int* status;     // device status word (0 = ok) or null
  const struct TpLink* tp;  // tensor-parallel coupling of this GEMM to its peers, or null
};

// Tensor-parallel coupling of one GEMM (bf16 output, K-major operands).
//
// Rows are grouped in tiles of 128; tile t is owned by rank t % world and is that rank's
// local tile t / world.  Counters are monotonic and never reset: the consumer keeps, in its
// own device memory, how much of each counter it has already consumed (`*_seen`, one entry
// per tile) and the last CTA of the consuming kernel advances it, so the same captured launch
// sequence can be replayed and steps with different row counts can be mixed.
//
//   wait_a:  the TMA producer loads rows of A tile t only after a_ready[t] (local counter,
//            incremented by the peers that push rows of A into this GPU's memory) shows that
//            all valid rows of the tile have arrived for the current use.
//   push:    the epilogue stores output tile t into the owner's partial-sum slot
//            slot[owner][(rank * tiles_owned + t / world) * 128 + row][n] with plain stores
//            through the peer mapping, then adds 1 (release, system scope) per epilogue warp
//            to arrive[owner][t / world].
struct TpLink {
  int rank, world;
  int wait_a;
  const int* a_ready;  // [ceil(m / 128)] rows received so far, per tile
  int* a_seen;         // [ceil(m / 128)] rows consumed so far, per tile
  int* ticket;         // scratch for last-CTA detection, zero between launches; null: this
                       // GEMM does not close the use (another GEMM on the same rows follows)
  int push;
  int tiles_owned;     // local tiles per rank: ceil(ceil(m / 128) / world)
  void* slot[8];       // bf16 [world, tiles_owned, 128, n] on every rank
  int* arrive[8];      // int32 [tiles_owned] on every rank
};
cudaError_t gemm_bf16(const GemmArgs& args, int sm_count, cudaStream_t stream);
// The same product on CTA pairs (tcgen05.mma.cta_group::2, 256x256 tiles); g.tp must be null.
cudaError_t gemm_bf16_pairs(const GemmArgs& g, int sm_count, cudaStream_t stream);

// Owner side of the tensor-parallel residual stream, one CTA per owned row or per four owned rows:
//   h = bf16(residual_row + sum over source ranks (in rank order) of slot[src][row])
//   hidden_own[row] = h;  x = weight * bf16(h * rsqrt(mean(h^2) + eps))
//   x is stored into xbuf[peer][global_row] on every rank (peer stores), then ready[peer][tile]
//   is advanced by one row (release, system scope).
// With seed != null the slots are not read and residual_row = seed[global_row] (first layer).
// The kernel waits (bounded) until arrive[local tile] exceeds arrive_seen[local tile] by
// world * arrivals_per_source.
struct TpReduceArgs {
  int rank, world;
  int m, width;            // rows of the full activation, hidden size (multiple of 8, <= 8192)
  int tiles_owned;
  const void* slot;        // local bf16 [world, tiles_owned, 128, width]
  const int* arrive;       // local int32 [tiles_owned]
  int* arrive_seen;        // local int32 [tiles_owned]
  int* ticket;
  int arrivals_per_source; // 4 * ceil(width / 256): one per epilogue warp and column tile
  void* hidden_own;        // local bf16 [tiles_owned * 128, width], in/out
  const void* seed;        // local bf16 [m, width] or null
  // Seed mode starts a new step: it overwrites every rank's input buffer, so it first waits
  // until all ranks have signalled the end of their previous step (tp_signal_done):
  // done >= world * (*done_uses); the last CTA then advances done_uses.
  const int* done;         // local int32 counter
  int* done_uses;
  const void* weight;      // bf16 [width]
  float eps;
  void* xbuf[8];           // bf16 [ceil(m/128)*128, width] on every rank
  int* ready[8];           // int32 [ceil(m/128)] on every rank
  int rows_per_cta;        // 0: chosen from the number of owned rows; 1 or 4
  int* status;
};
cudaError_t tp_reduce_norm(const TpReduceArgs& args, cudaStream_t stream);
// End of a step: adds 1 (release, system scope) to the `done` counter of every rank.
cudaError_t tp_signal_done(int* const done[8], int world, cudaStream_t stream);

// -------------------------------------------------------------------------- pointwise
// All tensors bf16 unless stated.  `addend` may be null (plain RMSNorm); with it,
// total_out = bf16(x + addend) is written and normalised.  rstd (fp32 [rows]) may be null.
cudaError_t rms_norm_fwd(const void* x, const void* addend, const void* w, void* total_out,
                         void* out, float* rstd, int64_t rows, int width, float eps,
                         cudaStream_t stream);
// dw_partial is fp32 [rms_norm_bwd_partials(rows), width]; the caller sums it over dim 0.
int rms_norm_bwd_partials(int64_t rows);
// extra (bf16 [rows, width], may be null) is added to dx in FP32 before its one rounding.
cudaError_t rms_norm_bwd(const void* grad, const void* x, const void* w, const float* rstd,
                         void* dx, float* dw_partial, int64_t rows, int width,
                         cudaStream_t stream, const void* extra = nullptr);
// x [rows, heads, 128] with row_stride elements between rows (heads * 128 when dense; larger
// when x is a column block of a wider matrix); out is dense; cos/sin [rows, 128]; rstd fp32
// [rows, heads] (may be null in fwd).
cudaError_t head_norm_rope_fwd(const void* x, const void* w, const void* cosv, const void* sinv,
                               void* out, float* rstd, int64_t rows, int heads, int64_t row_stride,
                               float eps, cudaStream_t stream);
int head_norm_rope_bwd_partials(int64_t rows, int heads);  // rows of the fp32 [.,128] partial
cudaError_t head_norm_rope_bwd(const void* grad, const void* x, const void* w, const void* cosv,
                               const void* sinv, const float* rstd, void* dx, float* dw_partial,
                               int64_t rows, int heads, int64_t x_row_stride, int64_t dx_row_stride,
                               cudaStream_t stream);  // strides in elements per token row
cudaError_t silu_mul_fwd(const void* gate, const void* up, void* out, int64_t elements,
                         cudaStream_t stream);
// out[r, c] = bf16(silu(both[r, c])) * both[r, width + c] for both = [rows, 2 * width].
cudaError_t silu_mul_pair(const void* both, void* out, int64_t rows, int width, cudaStream_t stream);
// dboth = [dgate | dup] for grad [rows, width] and both = [gate | up] ([rows, 2 * width]).
// act (bf16 [rows, width], may be null) also receives the forward value silu(gate) * up.
cudaError_t silu_mul_pair_bwd(const void* grad, const void* both, void* dboth, int64_t rows,
                              int width, cudaStream_t stream, void* act = nullptr);
cudaError_t silu_mul_bwd(const void* grad, const void* gate, const void* up, void* dgate,
                         void* dup, int64_t elements, cudaStream_t stream);
// mode 0: (1-s)*a + s*b; mode 1: a - s*b.  sigma fp32 [batch, sigma_frames]
// (sigma_frames is 1 or frames); a/b/out are [batch, channels, frames, hw], fp32 or bf16.
cudaError_t rf_combine(const void* a, const void* b, const float* sigma, void* out, int64_t batch,
                       int64_t channels, int frames, int hw, int sigma_frames, int mode,
                       int is_bf16, cudaStream_t stream);
// Distribution-matching target in FP64: per sample (row of `per` fp32 elements) spread =
// max(mean |estimate - teacher|, 1e-5), target = estimate - (fake - teacher) / spread.
// `partial` and `squares` hold dmd_target_blocks() doubles per sample; `squares` receives the
// per-block sums of float(step)^2.
int dmd_target_blocks();
cudaError_t dmd_target(const float* estimate, const float* fake, const float* teacher, double* partial,
                       double* target, double* squares, int64_t batch, int64_t per, cudaStream_t stream);

// -------------------------------------------------------------------------- attention
// Segment-list flash attention, head_dim 128, bf16.  q [B, NQ, Hq, 128], k/v [B, NK, Hkv, 128]
// and optional text k/v [B, text_len, Hkv, 128]; strides in elements.  out has the layout
// of q (contiguous), lse is fp32 [B, Hq, NQ].  q_tiles is int32 [num_q_tiles, 5]
// (q_row, rows, first_entry, entries, q_local); entries int32 [*, 3] (source, k_row, k_len)
// with source 0 = text, 1 = visual, 2 = visual with a causal mask against the chunk.
struct AttnArgs {
  const void* q; const void* k; const void* v;
  const void* text_k; const void* text_v;   // may be null
  void* out; float* lse;
  const int* q_tiles; const int* entries; const int* text_valid;
  int64_t nq, nk, text_len, batch;
  int64_t q_row_stride, q_batch_stride, kv_row_stride, kv_batch_stride;
  int64_t v_row_stride, v_batch_stride;  // 0: v has the strides of k (v may be a column slice)
  int64_t text_row_stride, text_batch_stride;
  int hq, hkv, num_q_tiles;
  float scale;
  int* status;
  // Forward only: with key_splits > 1 the tile list holds key_splits copies of the query
  // tiles (each with its own key entries); copy s writes out / lse rows s * nq + q of tensors
  // with key_splits * nq rows per sample, to be merged by attention_combine.
  int key_splits;
};
cudaError_t attention_fwd(const AttnArgs& args, cudaStream_t stream);
// out[b, q, h, :] = sum_s w_s partial[b, s*nq + q, h, :], w_s = exp(lse_s - logsumexp_s lse_s).
cudaError_t attention_combine(const void* partial, const float* lse, void* out, int64_t batch,
                              int64_t nq, int hq, int splits, cudaStream_t stream);

// Backward of attention_fwd.  `fwd` carries the forward tensors (out and lse filled in);
// grad_out/dq have the layout of out, dk/dv the dense layout [B, NK, Hkv, 128]; rows of
// dk/dv that no query can see must be zeroed by the caller; delta is fp32 scratch
// [B, Hq, NQ].  k_tiles int32 [num_k_tiles, 5] (k_row, rows, first_reader, readers, -1),
// q_lists int32 [*, 2] (q_row, q_len).  Text keys receive no gradient.
struct AttnBwdArgs {
  AttnArgs fwd;
  const void* grad_out;
  void* dq; void* dk; void* dv;
  // Row / batch strides of dv in elements (0: dense [B, NK, Hkv, 128]), so that dv can be
  // written into the v columns of a fused [rows, q | k | v] gradient matrix.
  int64_t dv_row_stride, dv_batch_stride;
  float* delta;
  const int* k_tiles; const int* q_lists;
  int num_k_tiles;
};
cudaError_t attention_bwd(const AttnBwdArgs& args, cudaStream_t stream);
// The same gradients in one pass over the scores (csrc/attention_bwd_fused.cu).  k_tiles int32
// [num_k_tiles, 5] (k_row, rows, first_block, blocks, source: 0 text, 1 visual) in the order in
// which the tiles take their turns, text tiles included; blocks int32 [*, 4] (q_block_row, lo, hi,
// turn) with q_block_row a multiple of 128; dq_acc fp32 [B, nq_pad, Hq, 128] and turns int32
// [1 + B * Hq * nq_pad / 128], both zeroed by the caller.  args.k_tiles / q_lists are unused,
// args.num_k_tiles counts the rows of k_tiles.
cudaError_t attention_bwd_fused(const AttnBwdArgs& args, const int* k_tiles, const int* blocks,
                                float* dq_acc, int* turns, int64_t nq_pad, cudaStream_t stream);

// Attention with forward-mode tangents (dense keys, optional prefix-valid text segment):
// out/tangent fp32 [B, NQ, Hq, 128], lse fp32 [B, Hq, NQ] or null.  q/tq share strides, and so
// do k/tk/v/tv.  Keys [0, text_len) are visible below text_valid[b] (null: all), later keys always.
struct AttnJvpArgs {
  const void* q; const void* k; const void* v;
  const void* tq; const void* tk; const void* tv;
  float* out; float* tangent; float* lse;
  const int* text_valid;
  int64_t nq, nk, text_len, batch;
  int64_t q_row_stride, q_batch_stride, kv_row_stride, kv_batch_stride;
  int hq, hkv;
  float scale;
  int* status;
};
cudaError_t attention_jvp(const AttnJvpArgs& args, cudaStream_t stream);

// ------------------------------------------------------------------ streaming cache
// dst[t] = rotate(src[t < sink ? t : t + shift]) for t < kept_tokens; rows are
// [token][heads][128] bf16; cos/sin fp32 [kept_tokens, 128] or null (plain move).
cudaError_t relocate_rows(const void* src, void* dst, const float* cosv, const float* sinv,
                          int64_t kept_tokens, int sink_tokens, int shift_tokens, int heads,
                          cudaStream_t stream);

// ------------------------------------------------------------------------- video VAE
// AdaLN modulation of bf16 rows (x, out [rows, width]; w [width]):
//   norm_modulate:  out = rms_norm(x) * w * (1 + scale) + shift
//   gated_residual: out = hidden + gate * y
// scale, shift and gate are column blocks of the modulation projection: element [row, c] sits
// at pointer + row * stride + c (stride a multiple of 8).
cudaError_t norm_modulate(const void* x, const void* w, const void* scale, const void* shift,
                          void* out, int64_t rows, int width, int64_t mod_stride, float eps,
                          cudaStream_t stream);
cudaError_t gated_residual(const void* hidden, const void* gate, const void* y, void* out,
                           int64_t rows, int width, int64_t gate_stride, cudaStream_t stream);

// Channel RMS norm of channels-last bf16 activations (x, out: [pixels, channels], gamma fp32
// [channels]): out = x / max(||x||, 1e-12) * sqrt(channels) * gamma, then SiLU when silu != 0.
cudaError_t channel_norm(const void* x, const float* gamma, void* out, int64_t pixels, int channels,
                         int silu, cudaStream_t stream);

// ------------------------------------------------------------------ convolution (codecs)
// Stride-1 convolution of a channels-last bf16 volume on the tensor cores, as an implicit
// GEMM: x [B, Tin, H, W, Cin], weight [Cout, kt * kh * kw, Cin] (taps in (t, h, w) order),
// out [B, Tout, H, W, Cout] with Tout = Tin - kt + 1.  Space is zero-padded by (pad_h, pad_w)
// on both sides (kh = 2 * pad_h + 1, kw = 2 * pad_w + 1); time is not padded: the caller
// prepends the frames (or zeros) a causal convolution looks back at.
//   out = act(conv(x, weight) + bias + residual)   (bias [Cout], residual like out; both optional;
//                                                   act = ReLU when relu != 0, else identity)
// Cin and Cout are multiples of 8.  fp16 != 0: every tensor is fp16 instead of bf16.
struct ConvArgs {
  const void* x;
  const void* weight;
  const void* bias;
  const void* residual;
  void* out;
  int batch, frames_in, height, width, cin, cout;
  int kt, kh, kw;
  int relu, fp16;
  // causal != 0: kt - 1 implicit frames precede x, so Tout = Tin.  The last `history_frames`
  // of them are the frames of `history` ([B, history_frames, H, W, Cin]); those before are zero.
  int causal;
  const void* history;
  int history_frames;
  int* status;
};
cudaError_t conv3d_bf16(const ConvArgs& args, int sm_count, cudaStream_t stream);

// Depthwise k x k convolution (k = 3, 5 or 7; stride 1, zero padding k / 2) of channels-last
// frames: x, out [frames, H, W, C], weight [k * k, C], bias [C] or null; C a multiple of 8;
// bf16, or fp16 when fp16 != 0.
struct DepthwiseArgs {
  const void* x;
  const void* weight;
  const void* bias;
  void* out;
  int frames, height, width, channels, kernel;
  int fp16;
};
cudaError_t depthwise_conv(const DepthwiseArgs& args, cudaStream_t stream);

// Geometry preprocessing, one pass each over planar tensors (plane = T * H * W):
//   colorize_depth: depth fp32 [B, plane] (metric; invalid <= 0 or non-finite) -> RGB fp32
//                   [B, 3, plane] along the 7-segment colour-cube walk, scale [B] or [1];
//   decode_normal:  uint8 [B, 3, plane] -> unit vectors fp32 [B, 3, plane] (0 when degenerate).
cudaError_t colorize_depth(const float* depth, const float* scale, float* out, int64_t batch,
                           int64_t plane, int scale_count, cudaStream_t stream);
cudaError_t decode_normal(const void* normal, float* out, int64_t batch, int64_t plane,
                          cudaStream_t stream);
// Frame stacks [images, H, W] fp32.  pool_frames: mean over factor x factor windows, non-finite
// inputs as zero.  blur_frames: separable blur with 2 * radius + 1 taps and replicated borders
// (scratch has the size of src).  warp_frames: [B, C, T, H, W], bilinear sampling of the
// scale / shift / shear / perspective map given by params [B * T, 8] = (sx, sy, tx, ty, hx, hy,
// px, py), border clamped; frames with copy[b * T + t] != 0 are copied.
cudaError_t pool_frames(const float* src, float* dst, int64_t images, int h, int w, int factor,
                        cudaStream_t stream);
cudaError_t blur_frames(const float* src, float* scratch, float* dst, const float* taps, int radius,
                        int64_t images, int h, int w, cudaStream_t stream);
cudaError_t warp_frames(const float* src, float* dst, const float* params, const uint8_t* copy, int64_t batch,
                        int channels, int frames, int h, int w, cudaStream_t stream);
// resize_frames: [images, H, W] -> [images, OH, OW]; area = 1 takes the mean over each output
// pixel's source bin (adaptive average pooling), area = 0 samples bilinearly with aligned pixel
// centres.  stretch_frames: [B, planes, H, W] -> [B, planes, TH, TW], the four quadrants around
// the centre resized bilinearly; top[b] / left[b] (0 <= top <= TH - H, 0 <= left <= TW - W) are
// the rows / columns the upper / left half gains.
cudaError_t resize_frames(const float* src, float* dst, int64_t images, int h, int w, int oh, int ow,
                          int area, cudaStream_t stream);
cudaError_t stretch_frames(const float* src, float* dst, const int* top, const int* left, int64_t batch,
                           int64_t planes, int h, int w, int th, int tw, cudaStream_t stream);

// ------------------------------------------------- all-to-all over peer memory (one node)
// out[s] = block `rank` of rank s's `send`, for all s.  `recv[r]` is rank r's receive buffer
// (2 * half_bytes, the same symmetric allocation on every rank), `arrive[r]` its arrival
// counter; `count` (exchanges completed) and `ticket` (zero between launches) are local.
struct ExchangeArgs {
  const void* send;       // [world, bytes_per_rank]
  void* out;              // [world, bytes_per_rank]
  void* recv[8];
  int* arrive[8];
  int* count;
  int* ticket;
  int64_t bytes_per_rank;  // a multiple of 16
  int64_t half_bytes;      // >= world * bytes_per_rank
  int rank, world;
  int* status;
};
cudaError_t exchange_all_to_all(const ExchangeArgs& args, int sm_count, cudaStream_t stream);

// ----------------------------------------------------------- sharded optimizer (ZeRO)
// Base pointers of the same flat buffer on every rank of the node (index = rank).
struct ZeroPeers {
  void* ptr[8];
  int world;
};
// units: int64 [num_units, 4] = (flat offset, state offset, count, hyper row).
int zero_reduce_parts(int num_units, int sm_count);  // length of the partial buffers
cudaError_t zero_reduce(const ZeroPeers& grads, const int64_t* units, int num_units,
                        float* gshard, float* partial_sumsq, int* partial_bad, float* sumsq_out,
                        float* bad_out, int sm_count, cudaStream_t stream);
// The same reduce over units [unit_begin, unit_end) with `parts` CTAs (partial buffers of that
// length); with `ready` the kernel first waits, at most limit_ns, until *ready has reached
// ready_target (every rank has announced the gradients of this bucket).  write_back_rank >= 0:
// the bf16 average also replaces rank write_back_rank's own gradient of the range.
cudaError_t zero_reduce_range(const ZeroPeers& grads, const int64_t* units, int unit_begin,
                              int unit_end, float* gshard, float* partial_sumsq, int* partial_bad,
                              int parts, const int* ready, int ready_target, int* status,
                              uint64_t limit_ns, int write_back_rank, cudaStream_t stream);
// Adds one to int32 slot `slot` of the counter table of every rank (system-scope release).
cudaError_t zero_signal(const ZeroPeers& counters, int slot, cudaStream_t stream);
// Waits (bounded) until *counter has reached target.
cudaError_t zero_wait(const int* counter, int target, int* status, uint64_t limit_ns,
                      cudaStream_t stream);
// Folds the partials in index order and, with more than one rank, exchanges the two numbers
// through the ranks' tables (int32 [8][4]) and sums them in rank order.
cudaError_t zero_stats(const float* partial_sumsq, const int* partial_bad, int parts,
                       const ZeroPeers& tables, int rank, int epoch, float* sumsq_out,
                       float* bad_out, int* status, uint64_t limit_ns, cudaStream_t stream);
// hyper: fp32 [rows, 8] = lr, beta1, beta2, eps, weight_decay, 1-beta1^t, sqrt(1-beta2^t),
// adam_w flag.  grad_scale / skip_flag: device scalars (may be null).
// gshard may be null in both calls: zero_reduce then only produces the statistics and
// zero_adam averages the peers' gradients itself.
cudaError_t zero_adam(const ZeroPeers& params, const ZeroPeers& grads, const int64_t* units,
                      int num_units, const float* gshard, float* master, float* exp_avg, float* exp_avg_sq,
                      const float* hyper, const float* grad_scale, const float* skip_flag,
                      int sm_count, cudaStream_t stream);

// M-RoPE tables: positions fp32 [tokens, 3], inverse fp32 [64], axis int32 [64] -> cos / sin
// [tokens, 128] (bf16 or fp32), slot j and j + 64 alike.
cudaError_t rope_tables(const float* positions, const float* inverse, const int* axis, void* cosine, void* sine,
                        int64_t tokens, bool bf16_out, cudaStream_t stream);
// [B, C, T, H, W] <-> [B, T, (H/p)(W/p), p*p*C] with the cast between fp32 and bf16 in the same pass.
cudaError_t patch_layout(const void* src, void* dst, int64_t batch, int64_t channels, int64_t frames,
                         int64_t height, int64_t width, int patch, bool to_patches, bool src_bf16,
                         bool dst_bf16, cudaStream_t stream);

// Maximum of n <= 32 unsigned values over the GPUs that share the multicast mapping `multicast` of
// the symmetric buffer `local` (>= 65 words, zeroed before the first call); state is one int of
// this GPU's own memory (calls made).  One launch: csrc/multimem.cu.
cudaError_t multimem_max(void* local, void* multicast, int* state, const uint32_t* in, uint32_t* out, int n,
                         int world, int rank, int* status, uint64_t limit_ns, cudaStream_t stream);
// All-gather / broadcast of a payload through multicast stores (csrc/multimem.cu): this GPU's
// `bytes_mine` bytes (may be 0) go to `offset` of the shared payload of `bytes_total` bytes, and
// the whole payload is copied to `out` once every GPU's part has landed.  Sizes, offset and both
// pointers are multiples of 16; the symmetric buffer of `buffer_bytes` bytes holds a counter and
// two halves of multimem_share_capacity(buffer_bytes) bytes; state is int32[2] in local memory,
// zero before the first call.  Every GPU must make the same sequence of calls (same totals).
int64_t multimem_share_capacity(int64_t buffer_bytes);
cudaError_t multimem_share(void* local, void* multicast, int64_t buffer_bytes, int* state, const void* src,
                           int64_t bytes_mine, int64_t offset, void* out, int64_t bytes_total, int world,
                           int sm_count, int* status, uint64_t limit_ns, cudaStream_t stream);

// y [m, n] = x [m, k] W[n, k]^T + b for a few FP32 rows (m <= 64 is the intended range), W and b in
// bf16 or fp32; and its gradients dx [m, k], dw [n, k], db [n] in FP32 (any of the three may be null).
cudaError_t rows_linear_fwd(const float* x, const void* w, const void* bias, float* y, int m, int n, int k,
                            bool bf16_weights, cudaStream_t stream);
// k a multiple of 8.  dx is summed from per-slice partial sums: dx_partial holds
// rows_linear_slices(n) * m * k floats.
int rows_linear_slices(int n);
cudaError_t rows_linear_bwd(const float* dy, const float* x, const void* w, float* dx, float* dx_partial,
                            float* dw, float* db, int m, int n, int k, bool bf16_weights, cudaStream_t stream);

// Diagnostic: every SM issues `iterations` x 8 tcgen05.mma (M 128, K 16, `columns` wide) back to
// back; cycles[0] receives the cycles block 0 needed, or -1 when its bounded wait gave up.
cudaError_t mma_issue_rate(int columns, bool a_from_tmem, int iterations, int sm_count, long long* cycles,
                           int* status, cudaStream_t stream);

}  // namespace agb
