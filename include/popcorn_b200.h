/*
 * popcorn_b200.h — C ABI of libpopcorn_b200.so
 *
 * A single CUDA (sm_100a) backend for the memory-bound transformer-layer ops of
 * tilde-research/popcorn: RMSNorm, residual-add + RMSNorm, rotary embedding,
 * SwiGLU forward, and MoE routing / permute / unpermute.
 *
 * Conventions shared by every entry point
 *   - all pointers are DEVICE pointers on the current device unless a comment
 *     says "host"; the library never allocates, frees, synchronises or throws;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); work is enqueued on it and the call returns at once;
 *   - leading dimensions / strides are in ELEMENTS of the tensor's dtype, the
 *     innermost dimension is always contiguous;
 *   - the return value is a b200_status; b200_last_error() gives a
 *     human-readable reason for the calling thread's last non-zero status;
 *   - zero-sized problems (rows == 0, tokens == 0 ...) return B200_OK and
 *     launch nothing.
 *
 * The reference has no C interface for these ops: its one first-party CUDA
 * kernel is bound with pybind11 + ATen (src/popcorn/impls/swiglu.cu:132-135,
 * loaded by src/popcorn/impls/_cuda.py:17-23).  Each function below names the
 * reference Python callable whose arithmetic it reproduces.
 */
#ifndef POPCORN_B200_H_
#define POPCORN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

typedef enum b200_dtype {
  B200_F32 = 0,
  B200_F16 = 1,
  B200_BF16 = 2
} b200_dtype;

typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_NULL_POINTER = 1,  /* a required pointer is NULL */
  B200_ERR_DTYPE = 2,         /* dtype enum not supported by this entry point */
  B200_ERR_SHAPE = 3,         /* negative size, stride smaller than extent, size over a stated limit */
  B200_ERR_ALIGNMENT = 4,     /* pointer not aligned to its element size */
  B200_ERR_LAUNCH = 5,        /* cudaGetLastError() after the launch was not cudaSuccess */
  B200_ERR_SCRATCH = 6,       /* scratch buffer too small or misaligned */
  B200_ERR_DEVICE = 7         /* current device is not compute capability 10.x */
} b200_status;

/* ABI version of the loaded library (== B200_ABI_VERSION it was built with). */
int b200_version(void);

/* Static name of a status code. Host pointer, never NULL. */
const char* b200_status_string(int status);

/* Detail text for the calling thread's most recent failure. Host pointer, never NULL. */
const char* b200_last_error(void);

/* Number of kernels this library has launched in the calling process (all threads). */
uint64_t b200_launch_count(void);

/*
 * Diagnostic: how many bounded waits on an asynchronous copy ran out on the
 * current device since the library was loaded (a kernel whose wait runs out
 * takes a slower path with ordinary loads; results stay correct).  Expected
 * value: 0.  Unlike every other entry point this one synchronises the device.
 */
uint64_t b200_wait_timeouts(void);

/*
 * y = round_T(x * rsqrt(mean(x^2) + eps)) * weight (+ bias)
 *
 * Replaces rms_norm(x, weight, bias=None, eps=1e-6), src/popcorn/kernels/rms_norm.py:16-30,
 * with rms() from src/popcorn/kernels/_utils.py:14-16.  For 16-bit dtypes the
 * normalised value is rounded to T before the weight multiply and the product
 * is rounded again (and once more after the bias add), as the reference's
 * tensor-by-tensor evaluation does.  The row sum of squares is accumulated in
 * fp32.  x, y: [rows, cols]; weight, bias: [cols] of the same dtype; bias may
 * be NULL; y may alias x.
 */
int b200_rms_norm(const void* x, const void* weight, const void* bias, void* y,
                  int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                  int dtype, double eps, void* stream);

/*
 * s = round_T(x + residual);  y = round_T(round_T(s * rsqrt(mean(s^2) + eps)) * round_T(weight + offset))
 *
 * Replaces add_rms_norm(x, residual, weight, eps=1e-6, offset=0.0),
 * src/popcorn/kernels/add_rms_norm.py:8-23.  Both outputs are written:
 * y (normalised) and s (the new residual stream).  s may alias x or residual,
 * y may alias the other one.
 */
int b200_add_rms_norm(const void* x, const void* residual, const void* weight,
                      void* y, void* s,
                      int64_t rows, int64_t cols,
                      int64_t ldx, int64_t ldr, int64_t ldy, int64_t lds,
                      int dtype, double eps, double offset, void* stream);

/*
 * Backward of b200_rms_norm and b200_add_rms_norm: what autograd derives from the references
 * (src/popcorn/kernels/_utils.py:14-16, rms_norm.py:29-30, add_rms_norm.py:22-23), with
 * n = round_T(x * r), r = rsqrt(mean(x^2) + eps):
 *   grad_weight = round_T(sum_rows round_T(g * n)),  grad_bias = round_T(sum_rows g)  (if grad_bias != NULL)
 *   gn = round_T(g * w);  grad_x = round_T(gn * r - x * r^3 * mean_cols(gn * x))      (fp32 inside)
 * For add_rms_norm w is round_T(weight + offset), `s` is the residual stream the forward pass returned,
 * grad_s (may be NULL) is the gradient arriving on it, and grad_x = round_T(round_T(...) + grad_s) is
 * the gradient of both x and residual.  Sums over rows are accumulated in fp32.
 * scratch: b200_rms_norm_backward_scratch_bytes(rows, cols, grad_bias != NULL) bytes, 16-byte aligned.
 */
int b200_rms_norm_backward_scratch_bytes(int64_t rows, int64_t cols, int with_bias, size_t* bytes);
int b200_rms_norm_backward(const void* grad_y, const void* x, const void* weight, void* grad_x, void* grad_weight,
                           void* grad_bias, int64_t rows, int64_t cols, int64_t ldg, int64_t ldx, int64_t lddx,
                           int dtype, double eps, void* scratch, size_t scratch_bytes, void* stream);
int b200_add_rms_norm_backward(const void* grad_y, const void* grad_s, const void* s, const void* weight, void* grad_x,
                               void* grad_weight, int64_t rows, int64_t cols, int64_t ldgy, int64_t ldgs, int64_t lds,
                               int64_t lddx, int dtype, double eps, double offset, void* scratch, size_t scratch_bytes,
                               void* stream);

/*
 * Rotary position embedding over x[batch, seq, heads, head_dim]:
 *   interleaved == 0 (GPT-NeoX halves): (x[j], x[half + j]) rotated by angle (seq, j)
 *   interleaved != 0 (GPT-J pairs):     (x[2j], x[2j + 1])
 *   y1 = x1*cos - x2*sin, y2 = x1*sin + x2*cos, every product and sum rounded to
 *   fp32 separately (no fused multiply-add), one rounding to T at the end;
 *   channels >= 2*half are copied through.
 *
 * Replaces rotary_embedding(x, cos, sin, interleaved=False),
 * src/popcorn/kernels/rotary_embedding.py:12-40.  cos, sin: [seq, half]
 * contiguous, dtype cs_dtype (fp32 or the same 16-bit type as x).  out may
 * equal x (in place); otherwise the two must not overlap.  Strides are those of
 * the batch, seq and heads dimensions, so q and k may be views into one fused
 * qkv buffer.
 */
int b200_rope(const void* x, const void* cos, const void* sin, void* out,
              int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, int64_t half,
              int64_t x_stride_b, int64_t x_stride_s, int64_t x_stride_h,
              int64_t o_stride_b, int64_t o_stride_s, int64_t o_stride_h,
              int dtype, int cs_dtype, int interleaved, void* stream);

/*
 * The same rotation applied to q[batch, seq, q_heads, head_dim] and
 * k[batch, seq, k_heads, head_dim] in ONE launch, in place, so that the
 * cos/sin row of a position is fetched once for both.  Equivalent to two
 * b200_rope calls with out == x (the reference calls rotary_embedding once per
 * tensor, src/popcorn/kernels/rotary_embedding.py:12-40).
 */
int b200_rope_qk(void* q, void* k, const void* cos, const void* sin,
                 int64_t batch, int64_t seq, int64_t q_heads, int64_t k_heads,
                 int64_t head_dim, int64_t half,
                 int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                 int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
                 int dtype, int cs_dtype, int interleaved, void* stream);

/*
 * Paired Llama-style rotary embedding of queries and keys, out of place:
 *   y = round_T(round_T(x * cos) + round_T(rot(x) * sin)),  rot(x) = (-x[half:], x[:half]),  x in {q, k}
 * with every product and the sum rounded to T, as the reference's tensor arithmetic does.
 *
 * Replaces rope(q, k, cos, sin), src/popcorn/kernels/rope.py:24-36.  Layout (batch, heads, seq,
 * head_dim) with batch/head/seq strides and a contiguous head_dim; cos, sin: [cos_batch, seq,
 * head_dim] contiguous in the dtype of q, cos_batch 1 or batch.  The full tables are used (the second
 * half is not assumed to repeat the first).  q_out / k_out must not overlap q / k.
 */
int b200_rope_paired(const void* q, const void* k, const void* cos, const void* sin, void* q_out, void* k_out,
                     int64_t batch, int64_t q_heads, int64_t k_heads, int64_t seq, int64_t head_dim, int64_t cos_batch,
                     int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                     int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                     int64_t qo_stride_b, int64_t qo_stride_h, int64_t qo_stride_s,
                     int64_t ko_stride_b, int64_t ko_stride_h, int64_t ko_stride_s,
                     int dtype, void* stream);

/*
 * Per-head RMS normalisation of queries and keys followed by the paired rotary embedding, one launch:
 *   n = round_T(round_T(x * r) * w),  r = 1 / sqrt(mean(x^2 over head_dim) + eps) in fp32,  w = q_weight or k_weight
 *   y = round_T(round_T(n * cos) + round_T(rot(n) * sin))
 *
 * Replaces qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps=1e-6), the fused op the reference
 * builds in examples/03_write_a_kernel.ipynb (cell 3: reference; cells 7, 11: its Triton forward),
 * = rope(rms_norm(q, q_weight), rms_norm(k, k_weight), cos, sin) of src/popcorn/kernels/rope.py:24-36
 * and src/popcorn/kernels/_utils.py:14-16.  Layout and tables as in b200_rope_paired; q_weight, k_weight:
 * [head_dim] contiguous in the dtype of q.
 */
int b200_qk_norm_rope(const void* q, const void* k, const void* q_weight, const void* k_weight,
                      const void* cos, const void* sin, void* q_out, void* k_out,
                      int64_t batch, int64_t q_heads, int64_t k_heads, int64_t seq, int64_t head_dim, int64_t cos_batch,
                      int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                      int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                      int64_t qo_stride_b, int64_t qo_stride_h, int64_t qo_stride_s,
                      int64_t ko_stride_b, int64_t ko_stride_h, int64_t ko_stride_s,
                      double eps, int dtype, void* stream);

/*
 * Backward of b200_qk_norm_rope: gradients of q, k (contiguous [batch, heads, seq, head_dim]) and of the two
 * weights ([head_dim]) from the gradients of the two outputs (contiguous, same shapes as q and k).  The row
 * statistics are recomputed from q and k.  What autograd derives from the fused op's reference
 * (examples/03_write_a_kernel.ipynb cell 3); the notebook's hand-written Triton backward is its cells 8-11.
 * scratch: b200_qk_norm_rope_backward_scratch_bytes(batch, seq, head_dim, dtype) bytes of device memory,
 * 16-byte aligned, written by the call (per-CTA partial column sums of the weight gradients).
 */
int b200_qk_norm_rope_backward_scratch_bytes(int64_t batch, int64_t seq, int64_t head_dim, int dtype, size_t* bytes);
int b200_qk_norm_rope_backward(const void* grad_q_out, const void* grad_k_out, const void* q, const void* k,
                               const void* q_weight, const void* k_weight, const void* cos, const void* sin,
                               void* grad_q, void* grad_k, void* grad_q_weight, void* grad_k_weight,
                               int64_t batch, int64_t q_heads, int64_t k_heads, int64_t seq, int64_t head_dim, int64_t cos_batch,
                               int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                               int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                               double eps, int dtype, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Llama 4 rotary embedding of queries and keys: channels are (real, imaginary) pairs multiplied by
 * unit complex numbers given as (cos, sin) pairs,
 *   y_re = round_T(round_T(re * f_re) - round_T(im * f_im)),  y_im = round_T(round_T(re * f_im) + round_T(im * f_re))
 *
 * Replaces llama4_rope(q, k, freqs), src/popcorn/kernels/llama4_rope.py:14-39.  Layout (batch, seq,
 * heads, head_dim) with batch/seq/head strides and a contiguous head_dim; freqs: [seq, head_dim/2, 2]
 * contiguous in the dtype of q.  q_out == q and k_out == k are allowed.
 */
int b200_llama4_rope(const void* q, const void* k, const void* freqs, void* q_out, void* k_out,
                     int64_t batch, int64_t seq, int64_t q_heads, int64_t k_heads, int64_t head_dim,
                     int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                     int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
                     int64_t qo_stride_b, int64_t qo_stride_s, int64_t qo_stride_h,
                     int64_t ko_stride_b, int64_t ko_stride_s, int64_t ko_stride_h,
                     int dtype, void* stream);

/*
 * out = round_T(round_T(silu(a)) * b),  silu(a) = a / (1 + exp(-a)) in fp32
 *
 * Replaces swiglu(a, b) = F.silu(a) * b, src/popcorn/kernels/swiglu.py:9-18
 * (the incumbent CUDA kernel is src/popcorn/impls/swiglu.cu:25-41, 77-101).
 * a, b, out: [rows, cols] with independent leading dimensions, so the gate and
 * up halves of one [rows, 2*cols] buffer are passed without a copy.
 */
int b200_swiglu(const void* a, const void* b, void* out,
                int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo,
                int dtype, void* stream);

/*
 * out = round_T(round_T(gelu_tanh(a)) * b),  gelu_tanh(a) = 0.5*a*(1 + tanh(sqrt(2/pi)*(a + 0.044715*a^3)))
 * evaluated in fp32 as a / (1 + exp(-2u)), which is the same function.
 *
 * Replaces geglu(a, b) = F.gelu(a, approximate="tanh") * b, src/popcorn/kernels/geglu.py:8-17.
 * Same layout rules as b200_swiglu.
 */
int b200_geglu(const void* a, const void* b, void* out,
               int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo,
               int dtype, void* stream);

/*
 * y = round_T( round_T(round_T(round_T(x*r) * weight) [+ bias]) * round_T(act(gate)) ),
 * r = rsqrt(mean(x^2) + eps), act = silu (sigmoid_gate == 0) or sigmoid.
 *
 * Replaces rms_norm_gated(x, g, weight, bias=None, activation="swish", eps=1e-6),
 * src/popcorn/kernels/rms_norm_gated.py:12-29.  bias may be NULL.
 */
int b200_rms_norm_gated(const void* x, const void* gate, const void* weight, const void* bias, void* y,
                        int64_t rows, int64_t cols, int64_t ldx, int64_t ldg, int64_t ldy,
                        int dtype, int sigmoid_gate, double eps, void* stream);

/*
 * y = x * rsqrt(sum(x^2) + eps) with every intermediate (x^2, the sum, + eps, rsqrt) rounded to T, as the
 * reference's all-in-T expression does.  Replaces l2_norm(x, eps=1e-6), src/popcorn/kernels/l2_norm.py:8-14.
 */
int b200_l2_norm(const void* x, void* y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                 int dtype, double eps, void* stream);

/*
 * y = round_T((x*rstd - mean*rstd) * weight + bias), fp32 mean and biased variance over the row,
 * rstd = 1/sqrt(var + eps).  Replaces layer_norm(x, weight, bias=None, eps=1e-6) = F.layer_norm(...),
 * src/popcorn/kernels/layer_norm.py:8-20.  bias may be NULL.
 */
int b200_layer_norm(const void* x, const void* weight, const void* bias, void* y,
                    int64_t rows, int64_t cols, int64_t ldx, int64_t ldy,
                    int dtype, double eps, void* stream);

/*
 * Backward of b200_l2_norm: grad_x = g s - x s^3 <g, x> per row, s = 1/sqrt(sum x^2 + eps), in fp32 with one
 * rounding.  What autograd derives from the reference x * rsqrt(x.pow(2).sum(-1, keepdim=True) + eps),
 * src/popcorn/kernels/l2_norm.py:14.
 */
int b200_l2_norm_backward(const void* grad_y, const void* x, void* grad_x, int64_t rows, int64_t cols,
                          int64_t ldg, int64_t ldx, int64_t lddx, int dtype, double eps, void* stream);

/*
 * Backward of b200_layer_norm: grad_x = rstd (gw - mean(gw) - xhat mean(gw xhat)) with gw = g w, grad_weight =
 * sum over rows of g xhat, grad_bias (may be NULL) = sum over rows of g.  What autograd derives from
 * F.layer_norm, src/popcorn/kernels/layer_norm.py:20.  scratch: b200_layer_norm_backward_scratch_bytes(rows, cols)
 * bytes of device memory, 16-byte aligned, written by the call.
 */
int b200_layer_norm_backward_scratch_bytes(int64_t rows, int64_t cols, size_t* bytes);
int b200_layer_norm_backward(const void* grad_y, const void* x, const void* weight, void* grad_x, void* grad_weight,
                             void* grad_bias, int64_t rows, int64_t cols, int64_t ldg, int64_t ldx, int64_t lddx,
                             int dtype, double eps, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Backward of b200_swiglu: grad_a = round_T(round_T(g*b) * dsilu(a)), grad_b = round_T(g * round_T(silu(a))),
 * dsilu(a) = s * (1 + a * (1 - s)), s = sigmoid(a), in fp32.
 *
 * Replaces what autograd derives from the reference F.silu(a) * b, src/popcorn/kernels/swiglu.py:18
 * (the incumbent backward kernel is src/popcorn/impls/swiglu.cu:43-66).  All five matrices are
 * [rows, cols] with their own leading dimensions; grad_a and grad_b may be the two halves of one buffer.
 */
int b200_swiglu_backward(const void* grad_out, const void* a, const void* b, void* grad_a, void* grad_b,
                         int64_t rows, int64_t cols, int64_t ldg, int64_t lda, int64_t ldb,
                         int64_t ldda, int64_t lddb, int dtype, void* stream);

/*
 * Backward of b200_geglu, same shapes and roundings as b200_swiglu_backward with the tanh-approximate GELU in
 * place of silu: grad_a = round_T(round_T(g*b) * gelu'(a)), grad_b = round_T(g * round_T(gelu(a))).
 *
 * Replaces what autograd derives from the reference F.gelu(a, approximate="tanh") * b,
 * src/popcorn/kernels/geglu.py:17.
 */
int b200_geglu_backward(const void* grad_out, const void* a, const void* b, void* grad_a, void* grad_b,
                        int64_t rows, int64_t cols, int64_t ldg, int64_t lda, int64_t ldb,
                        int64_t ldda, int64_t lddb, int dtype, void* stream);

/*
 * Backward of out = sigmoid(a) * b, same shapes as b200_swiglu_backward:
 * grad_b = round_T(g * s), grad_a = round_T((round_T(g*b) * (1 - s)) * s) with s = round_T(sigmoid(a)), the
 * sequence of PyTorch's sigmoid backward on the saved 16-bit gate.
 *
 * Replaces what autograd derives from the sigmoid branch of the gated RMS norm, out * torch.sigmoid(g),
 * src/popcorn/kernels/rms_norm_gated.py:29 (a = g, b = the normalised, scaled row).
 */
int b200_sigmoid_gate_backward(const void* grad_out, const void* a, const void* b, void* grad_a, void* grad_b,
                               int64_t rows, int64_t cols, int64_t ldg, int64_t lda, int64_t ldb,
                               int64_t ldda, int64_t lddb, int dtype, void* stream);

/*
 * MoE routing: probs = softmax(fp32(logits)) over experts; the top_k largest
 * (descending, ties to the lower expert index); weights = picked / sum(picked).
 *
 * Replaces the routing lines of momoe, src/popcorn/kernels/momoe.py:47-49
 * (same arithmetic in src/popcorn/impls/momoe_tl.py:1277-1279).
 * logits: [tokens, experts] (ld_logits elements per row); indices: int32
 * [tokens, top_k]; weights: fp32 [tokens, top_k].  Limits: experts <= 1024,
 * top_k <= min(experts, 32).
 */
int b200_moe_route(const void* logits, int32_t* indices, float* weights,
                   int64_t tokens, int64_t experts, int64_t top_k, int64_t ld_logits,
                   int logits_dtype, void* stream);

/*
 * Bytes of device scratch b200_moe_index needs for this problem size
 * (written to *bytes, a host pointer).
 */
int b200_moe_index_scratch_bytes(int64_t tokens, int64_t top_k, int64_t experts, size_t* bytes);

/*
 * Expert histogram, exclusive scan and the stable permutation index.
 *   counts[e]   = number of (token, slot) pairs routed to expert e
 *   offsets[e]  = sum of counts[0..e), offsets[experts] = tokens*top_k
 *   perm_token[p] = token id of the pair at sorted position p; pairs are sorted
 *                 by (expert, token), i.e. a stable sort of the flattened
 *                 indices by expert
 *   pos[t, k]   = sorted position of pair (t, k)  (inverse map)
 * perm_token may be NULL for callers that only need pos (the permute and
 * unpermute kernels do); it is one scattered 4-byte store per pair.
 *
 * Replaces find_used_experts + scatter_cols_kernel,
 * src/popcorn/impls/momoe_tl.py:1071-1161 (counts :1135, prefix :1094-1101,
 * col_idx :1104-1112).  The reference does not materialise `pos`.
 * indices must lie in [0, experts) (the output of b200_moe_route does); a pair
 * with an out-of-range expert is left out of counts, perm_token and pos.  Limits:
 * experts <= 1024, tokens*top_k < 2^31.  `scratch` needs
 * b200_moe_index_scratch_bytes() bytes, 16-byte aligned; its contents are
 * overwritten, it need not be cleared, and two calls that may run at the same
 * time (different streams) must not share it.
 *
 * Up to 256 experts this is ONE cooperative kernel launch (one CTA per SM; the
 * CTAs meet once, through flags in `scratch`, with a wait bounded at two
 * seconds: if it ever ran out, offsets[experts] would read -1); above that, or
 * with B200_INDEX_CHAIN=1 in the environment, three dependent launches
 * (histogram, scan, scatter).  The results are the same either way.
 */
int b200_moe_index(const int32_t* indices, int64_t tokens, int64_t top_k, int64_t experts,
                   int32_t* counts, int32_t* offsets, int32_t* perm_token, int32_t* pos,
                   void* scratch, size_t scratch_bytes, void* stream);

/*
 * b200_moe_route followed by b200_moe_index on its indices as one call: same
 * arguments, same results, same scratch as b200_moe_index.  Every momoe forward
 * runs the two back to back (momoe.py:47-49, then find_used_experts,
 * momoe_tl.py:1071-1161).  Two kernel launches up to 256 experts.  (Routing inside
 * the index kernel was built and measured: 33-35 us for 65536 tokens x top-8 over
 * 64 experts against 15 + 15 us for the two launches, because the routing is
 * bound by the integer pipe and loses occupancy inside the cooperative kernel.)
 */
int b200_moe_route_index(const void* logits, int32_t* indices, float* weights,
                         int64_t tokens, int64_t experts, int64_t top_k, int64_t ld_logits, int logits_dtype,
                         int32_t* counts, int32_t* offsets, int32_t* perm_token, int32_t* pos,
                         void* scratch, size_t scratch_bytes, void* stream);

/*
 * b200_moe_index for callers that cannot hand over a workspace.  (This entry point
 * has no counterpart in the reference; it exists for hosts of this library, not
 * to mirror a popcorn function.)
 *
 * Who needs it: a serving process that plans all of its device memory at start-up
 * and forbids cudaMalloc afterwards (an allocation synchronises the device and can
 * fail once memory is fragmented), or a plugin host that gives the library neither
 * an allocator nor a scratch pointer.  Such a caller still owns the inputs and the
 * four outputs; only the intermediate per-block histogram, which b200_moe_index
 * takes as `scratch`, lives inside the library here, in a fixed 1 MiB device array
 * (plus 2.5 KiB for the generation word and flags of the one-launch kernel) that
 * every GPU loading the library holds until the process exits.
 *
 * Limit: ceil(tokens*top_k / 2048) * experts * 4 bytes must fit in that array
 * (b200_moe_index_static_max_bytes reports its size); e.g. 64 experts allow up to
 * 8,388,608 (token, slot) pairs.  Larger problems return B200_ERR_SCRATCH and
 * should use b200_moe_index.  Results are identical to b200_moe_index.
 *
 * The first call on each device looks up the array's device address (with that
 * device current) and remembers it; make that first call before any stream
 * capture begins.  No call allocates or frees device memory.  All calls on a
 * device share the one array, which keeps whatever the last call left in it (the
 * kernels overwrite every entry they later read, so no clearing is needed); two
 * calls whose kernels overlap on the GPU, e.g. on different streams, race on it.
 */
int b200_moe_index_static(const int32_t* indices, int64_t tokens, int64_t top_k, int64_t experts,
                          int32_t* counts, int32_t* offsets, int32_t* perm_token, int32_t* pos,
                          void* stream);

/* Size in bytes of the built-in scratch array of b200_moe_index_static (written to *bytes, a host pointer). */
int b200_moe_index_static_max_bytes(size_t* bytes);

/*
 * Permute (scatter form): rows[pos[t, k], :] = x[t, :] for every slot k.
 * Each token row is read once and written top_k times.
 *
 * Replaces the row gather of src/popcorn/impls/momoe_tl.py:156-158 (fused into
 * lin1_kernel) and making_nice_scatter_kernel :408-476.
 */
int b200_moe_permute(const void* x, const int32_t* pos, void* rows,
                     int64_t tokens, int64_t top_k, int64_t hidden,
                     int64_t ldx, int64_t ldrows, int dtype, void* stream);

/*
 * Gather form: out[p, :] = x[src_row[p], :] for p in [0, n_rows).
 * Used on the receiving side of the expert-parallel exchange and wherever only
 * perm_token is at hand.  Same reference lines as b200_moe_permute.
 */
int b200_moe_gather(const void* x, const int32_t* src_row, void* out,
                    int64_t n_rows, int64_t hidden, int64_t ldx, int64_t ldo,
                    int dtype, void* stream);

/*
 * Weighted unpermute-combine:
 *   y[t, :] = round_T( sum_k weights[t, k] * fp32(rows[pos[t, k], :]) )
 * accumulated in fp32 in ascending pos order (= ascending expert index), each
 * product and each sum rounded separately, one rounding to T at the end.
 *
 * Replaces the gate-weighted sum of src/popcorn/kernels/momoe.py:52-53
 * (einsum "bsed,bse->bsd" in fp32, then one cast); the Triton path does it in
 * lin2_kernel, src/popcorn/impls/momoe_tl.py:295-304 and :398.
 */
int b200_moe_unpermute(const void* rows, const float* weights, const int32_t* pos, void* y,
                       int64_t tokens, int64_t top_k, int64_t hidden,
                       int64_t ldrows, int64_t ldy, int dtype, void* stream);

/*
 * Expert-parallel forms.  The reference has no distributed code (its momoe op is
 * single-GPU, src/popcorn/kernels/momoe.py:34-53); these are the permute and
 * unpermute steps of src/popcorn/impls/momoe_tl.py:156-158 / :295-304 with the
 * rows living in SEVERAL buffers: entry r of `bufs` (a HOST array of n_bufs <= 16
 * device pointers) is rank r's exchange buffer, mapped into the calling process
 * (CUDA peer / symmetric memory).  Rows cross NVLink inside the kernel, as
 * ordinary 128-bit stores (permute) or loads (unpermute); the caller orders the
 * ranks around the call (all writes landed before anyone reads; all reads done
 * before anyone overwrites).
 */

/*
 * Grouped expert GEMM over the expert-major row buffer that b200_moe_permute writes (tensor cores:
 * tcgen05.mma with fp32 accumulators in tensor memory, operands staged by TMA):
 *   weight2 == NULL:  out[p, :] = rows[p, :] @ weight[e(p)]
 *   weight2 != NULL:  out[p, :] = silu(rows[p, :] @ weight[e(p)]) * (rows[p, :] @ weight2[e(p)])
 * with e(p) the expert whose segment offsets[e] <= p < offsets[e + 1] contains row p; products are exact,
 * sums are fp32, the result is rounded to the operand type once (the SwiGLU product is formed in fp32).
 *
 * Replaces the expert MLP steps of momoe: the registered reference's einsums over a dense
 * [batch, seq, experts, .] tensor (src/popcorn/kernels/momoe.py:50-52) and the incumbent's lin1_kernel
 * (gate and up projection + SwiGLU, src/popcorn/impls/momoe_tl.py:90-212) and lin2_kernel (down
 * projection, :225-330).  The first form with the down weights is lin2, the second form with
 * (gate_weight, up_weight) is lin1.  rows: [total_rows, k] with row stride ld_rows; weight, weight2:
 * [experts, k, n] contiguous, the reference's layout; offsets: [experts + 1] int32 on the device, ascending,
 * offsets[experts] <= total_rows; out: [total_rows, n] with row stride ld_out (rows outside every segment
 * are left untouched; segments are clamped to total_rows).  dtype: B200_BF16 or B200_F16.  k, n, ld_rows,
 * ld_out must be multiples of 8; all buffers 16-byte aligned; experts <= 1024.  Each CTA takes a whole SM (about
 * 219 KB of shared memory and all 512 tensor-memory columns), so other kernels that use tensor memory should not
 * be run concurrently with this one on the same device.  B200_GEMM_PAIR=0 in the environment selects single CTAs
 * (cta_group::1) instead of cluster pairs.
 */
int b200_moe_grouped_gemm(const void* rows, const void* weight, const void* weight2, const int32_t* offsets, void* out,
                          int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows, int64_t ld_out,
                          int dtype, void* stream);

/*
 * b200_moe_grouped_gemm with the row gather fused into the operand load, the way the reference's lin1_kernel
 * addresses its A rows through idx_ptr_Msum (src/popcorn/impls/momoe_tl.py:156-158): row p of the A operand is
 * x[perm[p], :], fetched straight from the token-order activations x [tokens, k] (row stride ldx) by four-row
 * gathered bulk-tensor copies, so no expert-major copy of the rows (b200_moe_permute) has to exist.  perm: int32
 * [total_rows], the `perm_token` output of b200_moe_index (every entry below offsets[experts] must be a valid token
 * id); out: [total_rows, n] expert-major as for b200_moe_grouped_gemm, bit-identical to it on permuted rows.
 */
int b200_moe_grouped_gemm_gathered(const void* x, const int32_t* perm, const void* weight, const void* weight2, const int32_t* offsets,
                                   void* out, int64_t tokens, int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ldx,
                                   int64_t ld_out, int dtype, void* stream);

/*
 * Both projections of the expert MLP's first step without the activation, for training calls that keep the
 * pre-activations: out[p, 0:n] = rows[p, :] @ gate_weight[e(p)], out[p, n:2n] = rows[p, :] @ up_weight[e(p)].
 * One pass over rows like the fused form of b200_moe_grouped_gemm; out: [total_rows, 2n] with row stride
 * ld_out >= 2n.  Everything else as for b200_moe_grouped_gemm.
 */
int b200_moe_grouped_gemm_gate_up(const void* rows, const void* gate_weight, const void* up_weight, const int32_t* offsets,
                                  void* out, int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows,
                                  int64_t ld_out, int dtype, void* stream);

/*
 * Gradient of b200_moe_grouped_gemm with respect to its rows (what autograd derives from the reference's einsums,
 * src/popcorn/kernels/momoe.py:50-52, restricted to the routed pairs; the incumbent's counterparts are
 * swiglu_backward_kernel and lin1_backward_kernel, src/popcorn/impls/momoe_tl.py:567-700, 835-950):
 *   grad_rows[p, :] = grad_out[p, :] @ weight[e(p)]^T  (+ grad_out2[p, :] @ weight2[e(p)]^T)
 * The weights are read in place along their rows (no transposed copy); the optional second pair sums the gate
 * and up branches into one result in the same accumulator.  grad_out, grad_out2: [total_rows, n], row stride
 * ld_grad (both); weight, weight2: [experts, k, n]; grad_rows: [total_rows, k], row stride ld_out.  grad_out2
 * and weight2 are both NULL or both given.  Limits as for b200_moe_grouped_gemm.
 */
int b200_moe_grouped_gemm_dgrad(const void* grad_out, const void* weight, const void* grad_out2, const void* weight2,
                                const int32_t* offsets, void* grad_rows, int64_t total_rows, int64_t k, int64_t n,
                                int64_t experts, int64_t ld_grad, int64_t ld_out, int dtype, void* stream);

/*
 * Gradient with respect to the weights: grad_weight[e] = rows[segment e]^T @ grad_out[segment e] (the incumbent's
 * weights_update_kernel, src/popcorn/impls/momoe_tl.py:484-550), an [k, n] matrix per expert contracted over the expert's rows (fp32 accumulation, one rounding); experts without
 * rows get zeros.  rows: [total_rows, k], row stride ld_rows; grad_out: [total_rows, n], row stride ld_grad;
 * grad_weight: [experts, k, n] contiguous, every element is written.  Both operands are read in place: the
 * tensor maps address them by (row, line within the K slice), so the last slice of a segment is padded with
 * zeros instead of the next expert's rows.  experts * k < 2^31.
 */
int b200_moe_grouped_gemm_wgrad(const void* rows, const void* grad_out, const int32_t* offsets, void* grad_weight,
                                int64_t total_rows, int64_t k, int64_t n, int64_t experts, int64_t ld_rows, int64_t ld_grad,
                                int dtype, void* stream);

/*
 * Expert-parallel exchange without the host in the loop (no counterpart in the reference, which is single-GPU:
 * src/popcorn/kernels/momoe.py:34-53).  Every rank owns a "meta" buffer of b200_moe_ep_meta_bytes() bytes, zeroed
 * once, 128-byte aligned and mapped by all ranks (symmetric memory); meta[r] is rank r's buffer as mapped into this
 * process.  Epochs must grow by one per step and start above zero.
 *
 * b200_moe_ep_exchange publishes this rank's per-expert `counts` (the output of b200_moe_index) into every rank's
 * meta buffer, waits for every rank's counts and derives this rank's addressing on the device:
 *   dst_base[experts]                 row in the buffer of the expert's owner at which THIS rank's rows for that
 *                                     expert start (expert-major, source ranks in rank order inside an expert): the
 *                                     dst_base input of b200_moe_ep_destinations
 *   expert_offsets[experts/world + 1] segment starts of this rank's own experts in its own buffer
 *   info[4]                           rows this rank receives, rows it sends to other ranks, largest receive, world
 * b200_moe_ep_barrier (channel 1 .. 3) announces that this rank has reached `epoch` on `channel` and waits until
 * every rank has: after a kernel that stored rows into peer memory, and before a kernel that loads them.
 *
 * Waits are bounded by budget_ns.  A wait that runs out, or a rank that would receive more than capacity_rows rows,
 * makes no kernel trap or hang: status[0] (int32, device memory, zeroed by the caller) gets 1 (count exchange timed
 * out), 2 (rendezvous timed out) or 3 (over capacity), status[1] the peer or the row count, and after a failed
 * exchange every dst_base entry is negative, so that the row kernels skip every pair.  Ranks must be separate GPUs:
 * two ranks launched on one GPU would wait for each other without a guarantee of running at the same time.
 */
int b200_moe_ep_meta_bytes(size_t* bytes);
int b200_moe_ep_exchange(const int32_t* counts, void* const* meta, int64_t world, int64_t rank, int64_t experts,
                         int64_t capacity_rows, int32_t epoch, int64_t budget_ns, int32_t* dst_base,
                         int32_t* expert_offsets, int32_t* info, int32_t* status, void* stream);
int b200_moe_ep_barrier(void* const* meta, int64_t world, int64_t rank, int64_t channel, int32_t epoch, int64_t budget_ns,
                        int32_t* status, void* stream);

/*
 * For each (token, slot) pair: dst_rank = indices / experts_per_rank and
 * dst_row = dst_base[expert] + (pos - local_offsets[expert]), the pair's row in the
 * owning rank's buffer.  dst_base[e] is the row at which this rank's block for
 * expert e starts in that buffer (from the all-gathered counts); local_offsets is
 * the `offsets` output of b200_moe_index on this rank.  All arrays int32;
 * dst_rank, dst_row: [tokens, top_k].
 */
int b200_moe_ep_destinations(const int32_t* indices, const int32_t* pos, const int32_t* local_offsets,
                             const int32_t* dst_base, int64_t tokens, int64_t top_k, int64_t experts,
                             int64_t experts_per_rank, int32_t* dst_rank, int32_t* dst_row, void* stream);

/* bufs[dst_buf[t, k]][dst_row[t, k], :] = x[t, :]; a negative dst_row skips the slot. */
int b200_moe_permute_multi(const void* x, const int32_t* dst_buf, const int32_t* dst_row,
                           void* const* bufs, int64_t n_bufs,
                           int64_t tokens, int64_t top_k, int64_t hidden,
                           int64_t ldx, int64_t ldrows, int dtype, void* stream);

/*
 * Backward of b200_moe_unpermute: grad_rows[pos[t,k]] = round_T(weights[t,k] * grad_y[t]) and
 * grad_weights[t,k] = <grad_y[t], rows[pos[t,k]]> (fp32).  What autograd derives from the reference's combine
 * einsum, src/popcorn/kernels/momoe.py:52-53.  Rows no (token, slot) points to are left untouched; negative
 * positions get a zero weight gradient.  The backward of b200_moe_permute is b200_moe_unpermute itself with unit
 * weights (every token row collects the gradients of its top_k copies).
 */
int b200_moe_unpermute_backward(const void* grad_y, const void* rows, const float* weights, const int32_t* pos,
                                void* grad_rows, float* grad_weights, int64_t tokens, int64_t top_k, int64_t hidden,
                                int64_t ld_grad_y, int64_t ldrows, int64_t ld_grad_rows, int dtype, void* stream);

/*
 * y[t, :] = round_T( sum_k weights[t, k] * fp32(bufs[src_buf[t, k]][src_row[t, k], :]) ), accumulated in
 * ascending (buffer, row) order, which is ascending expert index when buffers hold contiguous expert
 * blocks in rank order.  Same arithmetic as b200_moe_unpermute.
 */
int b200_moe_unpermute_multi(void* const* bufs, int64_t n_bufs, const int32_t* src_buf, const int32_t* src_row,
                             const float* weights, void* y,
                             int64_t tokens, int64_t top_k, int64_t hidden,
                             int64_t ldrows, int64_t ldy, int dtype, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* POPCORN_B200_H_ */
