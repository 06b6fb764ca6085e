/*
 * sparsecoder.h — C ABI of libsparsecoder.so: sm_100a kernels for the TopK
 * sparse-coder (SAE / transcoder) training step.
 *
 * Conventions for every entry point:
 *   - returns an int status, SC_OK (0) on success; sc_last_error() holds a
 *     message for the most recent failure in this process;
 *   - never allocates, frees or synchronises: all pointers are device
 *     pointers to caller-owned memory (the single exception is the
 *     *_noalloc entry point, which owns a fixed static device array);
 *   - the caller passes the CUDA stream as an opaque pointer
 *     (cudaStream_t) and must have made the right device current;
 *   - matrices are row-major and contiguous: x[N,D], W[M,D], out[N,D],
 *     idx[N,k] (int64), acts[N,k];
 *   - "dtype" arguments take SC_F32 or SC_BF16.
 *
 * Each declaration cites the routine of EleutherAI/sparsify v1.3.0 whose
 * arithmetic it replaces (file:line inside that project).
 */
#ifndef SPARSECODER_H_
#define SPARSECODER_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
enum {
  SC_OK = 0,
  SC_ERR_INVALID = 1,     /* bad argument (shape, dtype, null pointer, alignment) */
  SC_ERR_UNSUPPORTED = 2, /* valid request this build has no kernel for */
  SC_ERR_WORKSPACE = 3,   /* workspace smaller than sc_*_workspace_bytes() */
  SC_ERR_CUDA = 4,        /* a CUDA runtime/driver call failed */
  SC_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up */
  SC_ERR_TOO_LARGE = 6    /* size beyond a fixed maximum of the entry point */
};

enum { SC_F32 = 0, SC_BF16 = 1 };

enum { SC_ACT_TOPK = 0, SC_ACT_GROUPMAX = 1 };

/* ---- diagnostics ------------------------------------------------------- */
int sc_version(void);

/* The persistent tensor-core kernels (sc_encode_topk, sc_encode_groupmax,
 * sc_gemm_bf16_nt) launch one CTA per SM with nearly all of its shared memory,
 * so no other kernel can start beside them. n > 0 makes them leave n SMs free
 * (0 <= n <= 64), e.g. for the kernels of a communication library that should
 * run concurrently. Process-wide; set it before sizing workspaces. */
int sc_set_reserved_sms(int n);
/* Form of the tensor-core encoder (sc_encode_topk, sc_encode_groupmax): one CTA per
 * 128-row tile, or pairs of CTAs on the two SMs of a TPC sharing a 256-row tile
 * (tcgen05 cta_group::2, each CTA loading its own operands with its own loads).
 * on < 0 (default): chosen per shape - pairs when the top-k lists leave the one-CTA
 * form fewer than four operand stages (k above about 40), else one CTA, which
 * measured faster under the B200's power cap; on = 0 / 1 forces one form.
 * Process-wide; set it before sizing workspaces. Results are identical. */
int sc_set_cta_pairs(int on);
/* Copies the last error message (NUL-terminated) into buf; returns its length. */
size_t sc_last_error(char* buf, size_t cap);
const char* sc_status_string(int status);

/* Self-test of the bounded device-side wait shared by the tensor-core kernels:
 * a one-thread kernel waits for limit_ns (at most 100 ms) on a barrier that
 * nothing arrives on, gives up, stores its wait code (199) in *status_word and
 * returns. The context stays usable; a host that reads a non-zero status word
 * after any entry point that takes one must treat the outputs of that call as
 * invalid (SC_ERR_TIMEOUT). No counterpart in the reference (it has no device
 * code of its own). */
int sc_selftest_wait_timeout(int32_t* status_word, int64_t limit_ns, void* stream);

/* ---- encoder forward ---------------------------------------------------
 * sparsify/fused_encoder.py:19-50 (FusedEncoder.forward):
 *   preacts = relu(x @ W^T + b); top-k (or groupmax) per row.
 */

/* x' = x - b_dec (b_dec may be NULL), cast to out_dtype.
 * sparsify/sparse_coder.py:191-192 (the subtraction in SparseCoder.encode). */
int sc_prep_input(const void* x, int x_dtype, const float* b_dec, int64_t N,
                  int64_t D, void* out, int out_dtype, void* stream);

/* Dense pre-activations relu(x W^T + b) written to pre[N,M] (pre_dtype).
 * Any shape; fp32 FMA kernel (x, W given in x_dtype / w_dtype).
 * sparsify/fused_encoder.py:29. */
int sc_preacts_dense(const void* x, int x_dtype, const void* W, int w_dtype,
                     const float* bias, int64_t N, int64_t D, int64_t M,
                     void* pre, int pre_dtype, void* stream);

/* Per-row top-k over a dense [N,M] fp32 matrix, optionally restricted to the
 * columns where col_mask[m] != 0 (others count as -inf). Unsorted output.
 * If fewer than k columns are eligible the call fails with SC_ERR_INVALID.
 * sparsify/fused_encoder.py:33 (torch.topk, sorted=False) and
 * sparsify/sparse_coder.py:240-243 (AuxK: where(dead_mask, pre_acts, -inf).topk). */
int sc_topk_rows(const float* pre, int64_t N, int64_t M, int k,
                 const uint8_t* col_mask, float* top_vals, int64_t* top_idx,
                 void* stream);

/* The same selection written back densely: out_bf16[n,m] = bf16(pre[n,m]) for the
 * row's k largest entries (among the columns with col_mask != 0 when given) and 0
 * elsewhere. The AuxK reconstruction of sparsify/sparse_coder.py:240-247 then is
 * one dense GEMM over the dead latents' columns. */
int sc_topk_mask_rows(const float* pre, int64_t N, int64_t M, int k,
                      const uint8_t* col_mask, void* out_bf16, void* stream);

/* groupmax: max and argmax inside each of k contiguous groups of M/k columns.
 * sparsify/fused_encoder.py:34-43. */
int sc_groupmax_rows(const float* pre, int64_t N, int64_t M, int k,
                     float* top_vals, int64_t* top_idx, void* stream);

/* Fused tcgen05 path: bf16 x[N,D] and W[M,D], fp32 bias, fp32 TMEM
 * accumulation; bias + ReLU + running per-row top-k in the epilogue so the
 * N x M matrix never reaches HBM; then a merge picks the final k per row.
 * Requirements: D % 8 == 0 (16-byte rows), k <= 128, M >= k.
 * ws must hold sc_encode_topk_workspace_bytes(N, D, M, k) bytes, 256-aligned.
 * status_word (device int32, may be NULL; the caller zeroes it) receives a
 * non-zero code if a bounded wait inside the kernel gave up; a word that is
 * already non-zero is left alone, so one word can collect over many calls and
 * be read once where the host synchronises anyway.
 * sparsify/fused_encoder.py:29-33. */
size_t sc_encode_topk_workspace_bytes(int64_t N, int64_t D, int64_t M, int k);
int sc_encode_topk(const void* x_bf16, const void* W_bf16, const float* bias,
                   int64_t N, int64_t D, int64_t M, int k, float* top_vals,
                   int64_t* top_idx, void* ws, size_t ws_bytes,
                   int32_t* status_word, void* stream);

/* The same kernel with the groupmax activation of sparsify/fused_encoder.py:34-43:
 * the M latents form k groups of M/k consecutive latents; per row and group the
 * largest post-ReLU pre-activation and its latent index (ties: lowest index),
 * written in group order to top_vals / top_idx [N,k]. bf16 operands, D % 8 == 0;
 * group size 32, 64, 128 or a multiple of 256 (SC_ERR_UNSUPPORTED otherwise: use
 * sc_preacts_dense + sc_groupmax_rows). No workspace. status_word as above. */
int sc_encode_groupmax(const void* x_bf16, const void* W_bf16, const float* bias,
                       int64_t N, int64_t D, int64_t M, int k, float* top_vals,
                       int64_t* top_idx, int32_t* status_word, void* stream);

/* ---- sparse decode (embedding bag) --------------------------------------
 * out[n,:] = (bias ? bias : 0) + sum_j acts[n,j] * W[idx[n,j],:]
 * sparsify/xformers.py:9-53 (embedding_bag_k), sparsify/utils.py:81-90,
 * sparsify/sparse_coder.py:198-202 (decode, with bias = b_dec) and
 * sparsify/fused_encoder.py:58-64 (grad-x of the encoder, bias = NULL).
 * out is fp32. */
int sc_embedding_bag_fwd(const int64_t* idx, const float* acts, const void* W,
                         int w_dtype, const float* bias, int64_t N, int64_t D,
                         int64_t M, int k, float* out, void* stream);

/* grad_acts[n,j] = dot(grad_out[n,:], W[idx[n,j],:]); grad_out fp32 or bf16.
 * sparsify/xformers.py:125-131 (per_sample_weights_grad). */
int sc_embedding_bag_bwd_acts(const int64_t* idx, const void* grad_out,
                              int g_dtype, const void* W, int w_dtype, int64_t N,
                              int64_t D, int64_t M, int k, float* grad_acts,
                              void* stream);

/* Decode fused with the residual of the FVU loss: out = bias + sum_j acts W[idx],
 * e = y - out, *sse = sum e^2 (device fp32 scalar, fixed summation order). Each
 * of out (fp32), e_f32, e_bf16 is written when non-NULL. y is fp32 or bf16.
 * D % 4 == 0. ws: sc_decode_residual_workspace_bytes(N) bytes.
 * sparsify/sparse_coder.py:198-202,225,253 in one pass. */
size_t sc_decode_residual_workspace_bytes(int64_t N);
int sc_decode_residual(const int64_t* idx, const float* acts, const void* W,
                       int w_dtype, const float* bias, const void* y,
                       int y_dtype, int64_t N, int64_t D, int64_t M, int k,
                       float* out, float* e_f32, void* e_bf16, float* sse,
                       void* ws, size_t ws_bytes, void* stream);

/* sc_decode_residual that also returns dots[N,k] = dot(e[n,:], W[idx[n,j],:]) from the
 * same pass over the gathered rows (each row of W is read once): with grad_out = s * e
 * this is grad_acts / s of sc_embedding_bag_bwd_acts, so the backward of the decode
 * needs no second gather. The dot uses e as stored: rounded to bf16 when e_bf16 is the
 * only residual written. Ids outside [0, M) contribute nothing and get dot 0.
 * W must be bf16, k <= 32, D % 4 == 0; SC_ERR_UNSUPPORTED
 * otherwise (use the two separate calls).
 * sparsify/sparse_coder.py:198-202,225,253 and sparsify/xformers.py:125-131. */
int sc_decode_residual_dots(const int64_t* idx, const float* acts, const void* W,
                            int w_dtype, const float* bias, const void* y,
                            int y_dtype, int64_t N, int64_t D, int64_t M, int k,
                            float* out, float* e_f32, void* e_bf16, float* sse,
                            float* dots, void* ws, size_t ws_bytes, void* stream);

/* Latent-major CSR of the [N,k] index matrix: row_ptr[M+1], entries[N*k]
 * (flat position n*k+j, ascending inside each latent, whatever its length).
 * ws: sc_csr_workspace_bytes(M) bytes.
 * sparsify/xformers.py:56-85,146-163 (count, cumsum, reverse mapping). */
size_t sc_csr_workspace_bytes(int64_t M);
int sc_csr_build(const int64_t* idx, int64_t N, int k, int64_t M,
                 int32_t* row_ptr, int32_t* entries, void* ws, size_t ws_bytes,
                 void* stream);

/* sc_csr_build for callers that cannot hand over scratch memory. It has no
 * counterpart in the reference. Some hosts of this library may not allocate on
 * the device at the point where they need the CSR: code running inside another
 * framework's memory plan or a fixed arena, or inside a region where
 * cudaMalloc and cudaFree are off limits because they synchronise the device.
 * This variant takes inputs and outputs only; its two counter arrays live in
 * a static device array inside the library (2 MiB, held by every GPU that
 * loads the library until the process exits), which caps it at
 * M <= 262144 latents: a larger M returns SC_ERR_TOO_LARGE. It calls no
 * cudaMalloc, cudaFree or allocating routine. The first call on each device
 * resolves the array's device address (cudaGetSymbolAddress) and should
 * therefore come before any stream capture on that device. All calls share the
 * one array: calls that may overlap on the GPU (different streams, or the same
 * device from several threads) race and must be serialised by the caller.
 * The array is the one of the device that is current at the call, so `stream`
 * must belong to that device. */
int sc_csr_build_noalloc(const int64_t* idx, int64_t N, int k, int64_t M,
                         int32_t* row_ptr, int32_t* entries, void* stream);

/* Per-latent row accumulate over latents [lat_begin, lat_end):
 *   gradA[m,:] = sum_e coefA[e] * vecA[e / k, :]   gbiasA[m] = sum_e coefA[e]
 *   gradB[m,:] = sum_e coefB[e] * vecB[e / k, :]   gbiasB[m] = sum_e coefB[e]
 * e runs over the CSR entries of latent m; rows with no entries are zeroed.
 * The B operands are optional as a group (gradB == NULL), gbiasA / gbiasB are
 * optional individually. vecA/vecB are [N,D] in their dtypes; coefA/coefB are
 * fp32 [N*k]; gradients are fp32. D must be a multiple of 4.
 * Decoder use (coef = acts, vec = grad_out): sparsify/xformers.py:88-136.
 * Encoder use (coef = grad_acts, vec = x', bias): sparsify/fused_encoder.py:66-84. */
int sc_rows_accumulate(const int32_t* row_ptr, const int32_t* entries, int k,
                       const float* coefA, const void* vecA, int vecA_dtype,
                       float* gradA, float* gbiasA, const float* coefB,
                       const void* vecB, int vecB_dtype, float* gradB,
                       float* gbiasB, int64_t M, int64_t D, int64_t lat_begin,
                       int64_t lat_end, void* stream);

/* out[m] = sum of coef[e] over the CSR entries of latent m (the bias gradient
 * of sparsify/fused_encoder.py:79-84 on its own). */
int sc_csr_segment_sum(const int32_t* row_ptr, const int32_t* entries,
                       const float* coef, int64_t M, float* out, void* stream);

/* ---- losses -------------------------------------------------------------
 * sparsify/sparse_coder.py:225-228,253-254:
 *   total_variance = sum((y - mean_0(y))^2);  e = y - out;  l2 = sum(e^2).
 * sc_total_variance writes *tv (device fp32); y is fp32 or bf16; ws holds
 * sc_loss_workspace_bytes(D) bytes. */
size_t sc_loss_workspace_bytes(int64_t D);
int sc_total_variance(const void* y, int y_dtype, int64_t N, int64_t D,
                      float* tv, void* ws, size_t ws_bytes, void* stream);
/* sse[0] = sum((a - b)^2) over n elements (device fp32 scalar);
 * if diff != NULL also writes diff = a - b. */
int sc_sq_err(const float* a, const float* b, int64_t n, float* diff,
              float* sse, void* ws, size_t ws_bytes, void* stream);

/* out[d] = sum_r w[r] * Y[r,d] (w == NULL: plain column sums), fp32 result,
 * fixed summation order. Used for the b_dec gradient: column sums of the
 * residual, and W_enc^T grad_b_enc, which equals the column sum of the
 * encoder's input gradient (sparsify/fused_encoder.py:58-64 followed by the
 * `x - b_dec` of sparsify/sparse_coder.py:191-192) without gathering it.
 * ws: sc_loss_workspace_bytes(D) bytes. */
int sc_weighted_colsum(const void* Y, int y_dtype, const float* w, int64_t R,
                       int64_t D, float* out, void* ws, size_t ws_bytes,
                       void* stream);

/* ---- weight update ------------------------------------------------------
 * sparsify/sparse_coder.py:273-279: W[m,:] /= (||W[m,:]||_2 + eps), in place;
 * optionally refreshes a bf16 shadow copy in the same pass. */
int sc_normalize_rows(float* W, int64_t M, int64_t D, float eps,
                      void* shadow_bf16, void* stream);

/* torch.optim.Adam (betas, eps, no weight decay, no amsgrad) on rows of a
 * [M,D] matrix; when project != 0 the gradient row first loses its component
 * parallel to the parameter row (sparsify/sparse_coder.py:281-295, in place on
 * g, as the reference does). step is the 1-based step count. bc = bias
 * corrections computed on the host. Optionally refreshes a bf16 shadow.
 * sparsify/trainer.py:99-116,513-519. A vector is a [1,D] matrix. */
int sc_adam_rows(float* p, float* g, float* m, float* v, int64_t M, int64_t D,
                 float lr, float beta1, float beta2, float eps, int64_t step,
                 int project, void* shadow_bf16, void* stream);

/* Host-side Adam hyper-parameters of one parameter (torch.optim.Adam names);
 * step is the 1-based step count. */
typedef struct sc_adam_hparams {
  float lr, beta1, beta2, eps;
  int64_t step;
} sc_adam_hparams;

/* Sparse weight gradients and the optimiser step in one pass over the latents:
 * per latent m the CSR segment is walked as in sc_rows_accumulate
 * (A = decoder: coefA * vecA rows, B = encoder: coefB * vecB rows) and the two
 * gradient rows, held in registers, go straight into
 *   B: Adam on pB[m,:] (sparsify/trainer.py:517-519), bf16 shadow refresh;
 *   A: optional projection (sparsify/sparse_coder.py:281-295), Adam, optional
 *      row normalisation W /= ||W|| + norm_eps (sparse_coder.py:273-279, which
 *      the reference applies before the next forward), bf16 shadow refresh.
 * The dense [M,D] gradients are never materialised. D % 4 == 0, D <= 8192.
 * hpA / hpB are host pointers. shadow pointers may be NULL. extraA (fp32
 * [n,D]) with extra_rank (int32 [M]: row of extraA for latent m, or -1) adds
 * dense gradient rows to the decoder gradient - the AuxK term of
 * sparsify/sparse_coder.py:231-249, which touches dead latents only; both NULL
 * when unused. parts selects the
 * matrices a launch updates: 1 = decoder (A) only, 2 = encoder (B) only, 3 =
 * both (the decoder half can then run on a second stream under the next
 * forward's encoder GEMM, which does not read W_dec). max_ctas > 0 caps the
 * grid (persistent CTAs striding over the latents) so that such a background
 * launch leaves room on every SM for the kernel it overlaps; 0 = one CTA per
 * latent. */
int sc_rows_adam(const int32_t* row_ptr, const int32_t* entries, int k,
                 const float* coefA, const void* vecA, int vecA_dtype,
                 const float* coefB, const void* vecB, int vecB_dtype,
                 int64_t M, int64_t D, float* pA, float* mA, float* vA,
                 void* shadowA_bf16, int projectA, int normalizeA,
                 float norm_eps, const sc_adam_hparams* hpA, float* pB,
                 float* mB, float* vB, void* shadowB_bf16,
                 const sc_adam_hparams* hpB, const float* extraA,
                 const int32_t* extra_rank, int parts, int max_ctas,
                 void* stream);

/* ---- dense bf16 GEMM on tcgen05 ---------------------------------------------
 * out[m,n] = act(alpha * sum_k A[m,k] B[n,k] + beta * Cin[m,n] + bias[n]),
 * A [M,K] and B [N,K] row-major bf16, fp32 accumulation in tensor memory, out
 * (and the optional Cin) fp32 or bf16 [M,N], bias fp32 [N] or NULL, relu 0/1.
 * K % 8 == 0. Replaces the library matmuls of the path:
 * sparsify/muon.py:32-36 (A = X X^T, B = bA + cAA, X = aX + BX),
 * sparsify/sparse_coder.py:221-222 (skip connection) and
 * sparsify/fused_encoder.py:29 when the dense pre-activations are wanted.
 * symmetric != 0 (needs A == B, M == N, no bias): the result is symmetric, so
 * tiles wholly below the diagonal are not computed and are filled from their
 * mirror images (X X^T and bA + cAA of Newton-Schulz: about half the work).
 * out_t, when not NULL, receives the transposed result [N,M] as well (same
 * dtype as out), so that an iteration can keep a matrix in both orientations
 * without a transpose pass.
 * status_word as in sc_encode_topk (may be NULL). */
int sc_gemm_bf16_nt(const void* A_bf16, const void* B_bf16, int64_t M, int64_t N,
                    int64_t K, float alpha, float beta, const void* Cin,
                    int cin_dtype, const float* bias, int relu, void* out,
                    int out_dtype, int symmetric, void* out_t,
                    int32_t* status_word, void* stream);

/* out[c,r] = in[r,c] for a bf16 matrix (puts the right operand of X = aX + BX
 * into K-major form, sparsify/muon.py:36). */
int sc_transpose_bf16(const void* in, int64_t R, int64_t C, void* out, void* stream);

/* ---- Muon's elementwise passes (sparsify/muon.py:115-181) -------------------
 * sc_muon_momentum: buf = lerp(buf, g, 1-beta); u = nesterov ? lerp(g, buf, beta)
 * : buf (muon.py:150-156); out_bf16 = bf16(u) (muon.py:22) and *sumsq = sum of
 * out^2 (for muon.py:29's norm), one pass. ws: sc_muon_workspace_bytes() bytes. */
size_t sc_muon_workspace_bytes(void);
int sc_muon_momentum(const float* g, float* buf, int64_t n, float beta, int nesterov,
                     void* out_bf16, float* sumsq, void* ws, size_t ws_bytes, void* stream);

/* X / (||X||_F + 1e-7) on a bf16 [R,C] matrix with torch's bf16 roundings
 * (muon.py:29), written in the same orientation (out_scaled, may be NULL) and /
 * or transposed (out_t [C,R], may be NULL; muon.py:25-27). sumsq = sum of
 * squares of X on the device, NULL for a plain copy / transpose. */
int sc_scale_transpose_bf16(const void* in, int64_t R, int64_t C, const float* sumsq,
                            void* out_scaled, void* out_t, void* stream);

/* p = p * decay - alpha * upd (bf16): decoupled weight decay (muon.py:120-123)
 * and the update (muon.py:139-141,176-178) in one pass; optional bf16 copy. */
int sc_muon_apply(float* p, const void* upd_bf16, int64_t n, float decay, float alpha,
                  void* shadow_bf16, void* stream);

/* sparsify/sparse_coder.py:281-295 on its own: g[m,:] -= (g[m,:] . w[m,:]) w[m,:]
 * in place, for optimisers that do not fold the projection into their update. */
int sc_project_rows(float* g, const float* w, int64_t M, int64_t D, void* stream);

/* optimizer="signum" of the reference Trainer (sparsify/trainer.py:146-161):
 * SignSGD (sparsify/sign_sgd.py:18-26, p -= lr * sign(g)) inside the
 * third-party schedulefree.ScheduleFreeWrapper(momentum=0.95), one fused pass.
 * p holds y (training mode), z the wrapped optimiser's iterate, ckp1 the
 * averaging weight of this step (weight / weight_sum, computed on the host):
 *   x = y + (1 - 1/momentum)(z - y);  z -= lr * sign(g);
 *   x += ckp1 (z - x);                y = x + (1 - momentum)(z - x).
 * Optionally refreshes a bf16 shadow of p. */
int sc_signum_schedulefree(float* p, float* z, const float* g, int64_t n, float lr,
                           float momentum, float ckp1, void* shadow_bf16, void* stream);

/* fp32 -> bf16 copy (shadow refresh). */
int sc_cast_bf16(const float* src, void* dst_bf16, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPARSECODER_H_ */
