/*
 * autograd_b200 - C ABI of the B200 (sm_100a) backend for autograd's fused layer kernels.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on the
 * context's CUDA stream and returns a status code (0 = AG_OK).  Nothing here allocates
 * device memory except ag_alloc/ag_ctx_create: kernels run inside buffers the caller owns
 * (the runtime's arena), and every workspace is passed in explicitly, with its size given
 * by the matching *_scratch_bytes() query.  No call aborts the process and no kernel
 * traps: device-side problems (an id outside the table, a bounded wait that expired)
 * set bits in a status word that ag_status() returns.
 *
 * "Replaces" lines cite the interface of the reference project (tuzbing/autograd) that an
 * entry point stands in for, as file:line of that project.
 *
 * Conventions: row-major contiguous tensors; N = token rows, C = hidden size, V = vocab
 * rows, I = MLP intermediate size, D = head dim.  `dtype` is AG_F32 or AG_BF16 (bf16 is
 * stored as 16-bit words with round-to-nearest-even, arithmetic is always fp32).
 * Gradient outputs accumulate unless stated otherwise, as the reference's non-Metal
 * execution path requires (runtime.py:844-854, backend.py:86, :414, :477-487, :538).
 */
#ifndef AUTOGRAD_B200_H
#define AUTOGRAD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ag_ctx ag_ctx;

enum {
  AG_OK = 0,
  AG_ERR_INVALID = 1,     /* bad argument (null pointer, misalignment, unsupported shape) */
  AG_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed; see ag_last_error        */
  AG_ERR_SCRATCH = 3,     /* workspace smaller than *_scratch_bytes() asks for           */
  AG_ERR_DEVICE = 4       /* device status word non-zero (ag_status)                     */
};

enum { AG_F32 = 0, AG_BF16 = 1 };

/* bits of the device status word */
enum {
  AG_STATUS_BAD_INDEX = 1,      /* gather / scatter-add / CE target outside its table     */
  AG_STATUS_WAIT_EXPIRED = 2,   /* a bounded mbarrier wait gave up (results are invalid)  */
  AG_STATUS_STAGE_FALLBACK = 4  /* bulk-copy staging timed out, plain loads used instead  */
};

/* ---- context, memory, copies ---------------------------------------------------------
 * Replaces: metal_ext.mm:770-796 (MetalContext: alloc/free/begin_pass/end_pass/fill_scalar/
 * copy_from_host/copy_to_host/synchronize) and storage.py:72-90 (MetalAllocator).        */

/* `stream` is a cudaStream_t to adopt (e.g. the host framework's current stream) or NULL
 * to create a private non-blocking stream. */
int ag_ctx_create(int device, void* stream, ag_ctx** out);
int ag_ctx_destroy(ag_ctx* ctx);
int ag_set_stream(ag_ctx* ctx, void* stream);
/* Message of the last failing call on this context (or of ag_ctx_create when ctx is NULL). */
const char* ag_last_error(const ag_ctx* ctx);
int ag_device_info(ag_ctx* ctx, int* sm_count, int64_t* l2_bytes, int64_t* total_bytes,
                   int* cc_major, int* cc_minor);
int ag_alloc(ag_ctx* ctx, size_t bytes, void** out);
int ag_free(ag_ctx* ctx, void* ptr);
int ag_copy_h2d(ag_ctx* ctx, void* dst, const void* src, size_t bytes);   /* stream-ordered  */
int ag_copy_d2h(ag_ctx* ctx, void* dst, const void* src, size_t bytes);   /* returns after the copy */
int ag_synchronize(ag_ctx* ctx);
/* Synchronises, returns the device status word in *flags and clears it. */
int ag_status(ag_ctx* ctx, int* flags);
/* Number of this library's kernels launched through ctx since creation. */
int64_t ag_launch_count(const ag_ctx* ctx);
/* Replaces: metal_ext.mm:215-286 (begin_pass_profiled/end_pass_profiled): CUDA-event
 * bracket on the context stream; end returns the elapsed milliseconds after syncing. */
int ag_pass_begin_profiled(ag_ctx* ctx);
int ag_pass_end_profiled(ag_ctx* ctx, float* ms);
/* Per-dispatch timing (replaces the per-dispatch proxies of debug/timing_ops_v2.py:479-543):
 * a pool of CUDA events owned by the context.  ag_event_record enqueues event `index` on the
 * context stream (the pool grows on demand); ag_event_elapsed waits for both events and
 * returns the milliseconds between them. */
int ag_event_record(ag_ctx* ctx, int index);
int ag_event_elapsed(ag_ctx* ctx, int start_index, int end_index, float* ms);
/* Per-launch timing of the tensor-core GEMM inside the fused linear+CE calls: while enabled,
 * every launch of that kernel is bracketed by events first_event_index + 2*i (before) and
 * + 2*i + 1 (after), i counting from 0 at the enabling call; ag_tc_timing_count returns i. */
int ag_tc_timing(ag_ctx* ctx, int enable, int first_event_index);
int ag_tc_timing_count(const ag_ctx* ctx);
/* Pinned host memory for staging inputs (cudaHostAlloc / cudaFreeHost). */
int ag_alloc_host(ag_ctx* ctx, size_t bytes, void** out);
int ag_free_host(ag_ctx* ctx, void* ptr);

/* Replaces: backend.py:5069-5080 fill_storage / fill_storage2 (fill_scalar_kernel,
 * fill_scalar_kernel2 in metal_ops.metal:122-137). */
int ag_fill_f32(ag_ctx* ctx, float* dst, float value, int64_t n);
/* n items of `itemsize` (1, 2 or 4) bytes each set to the low bytes of `pattern`. */
int ag_fill_pattern(ag_ctx* ctx, void* dst, uint32_t pattern, int itemsize, int64_t n);

/* ---- a1 residual add ------------------------------------------------------------------
 * Replaces: backend.py:74-105 cpu_add_forward/cpu_add_backward (same-shape case);
 * metal_ops.metal:161-200 add_residual_forward/backward.                                 */
int ag_add_forward(ag_ctx* ctx, const float* x, const float* y, float* out, int64_t n);
/* xgrad += g; ygrad += g (either may be NULL). */
int ag_add_backward(ag_ctx* ctx, const float* g, float* xgrad, float* ygrad, int64_t n);

/* ---- a2/a3 (residual add +) LayerNorm ------------------------------------------------
 * Replaces: backend.py:416-433 cpu_layernorm_forward (+ :74-76 for the fused add),
 * backend.py:435-487 cpu_layernorm_backward.
 * forward: h = x + r (r NULL: h = x), y = (h-mean)*rstd*gamma+beta, two-pass variance.
 *   h, mean, rstd may be NULL (not written).
 * backward: recomputes mean/rstd from x (= the h fed to the norm);
 *   dx = (dres ? dres : 0) + rstd*(dy*g - mean(dy*g) - xhat*mean(dy*g*xhat));
 *   dres == dx accumulates in place.  dgamma += sum_rows(dy*xhat), dbeta += sum_rows(dy)
 *   through per-CTA partial sums in `partials` (no atomics, fixed order); either may be
 *   NULL.  partials needs ag_norm_partials_bytes(ctx, C) bytes. */
int ag_add_layernorm_forward(ag_ctx* ctx, const float* x, const float* r, const float* gamma,
                             const float* beta, float* h, float* y, float* mean, float* rstd,
                             int64_t N, int C, float eps);
size_t ag_norm_partials_bytes(ag_ctx* ctx, int C);
int ag_layernorm_backward(ag_ctx* ctx, const float* dy, const float* x, const float* gamma,
                          const float* dres, float* dx, float* dgamma, float* dbeta,
                          void* partials, size_t partials_bytes, int64_t N, int C, float eps);
/* No counterpart in the reference.  Same result as ag_layernorm_backward for callers that
 * have no way to provide the partial-sum workspace: a runtime whose arena was planned without
 * this backend's scratch slots, a plugin interface that passes only the op's tensors, or code
 * running where device allocation is not permitted.  The workspace is a fixed array of
 * AG_LN_NOALLOC_SCRATCH_BYTES inside the library image (held on every GPU that loads the
 * library until the process exits), so this call allocates and frees nothing.
 *   - C must not exceed AG_LN_NOALLOC_MAX_C; larger rows are rejected with AG_ERR_INVALID.
 *   - The first call on a device resolves the array's device address; make that call before
 *     any stream capture begins.
 *   - All calls share the one array.  Calls on the same stream are ordered and safe; calls
 *     whose kernels may overlap on the GPU race on it.  Its previous contents never matter.
 *   - dgamma/dbeta are summed over a grid that may be smaller than the one
 *     ag_layernorm_backward uses, so they agree with it to rounding, not bit for bit. */
#define AG_LN_NOALLOC_SCRATCH_BYTES (8u << 20)
#define AG_LN_NOALLOC_MAX_C 4096
int ag_layernorm_backward_noalloc(ag_ctx* ctx, const float* dy, const float* x, const float* gamma,
                                  const float* dres, float* dx, float* dgamma, float* dbeta,
                                  int64_t N, int C, float eps);

/* Test hook (no counterpart in the reference): the next LayerNorm / RMSNorm kernel launched through
 * ctx gives up its bounded wait for the staged gamma/beta vectors at once, so that the unwind path
 * runs: AG_STATUS_STAGE_FALLBACK is set, the copy in flight is given time to land, the vectors
 * are filled with plain loads and the results are still correct.  One-shot. */
int ag_debug_expire_staging(ag_ctx* ctx);

/* ---- a4 RMSNorm -----------------------------------------------------------------------
 * Replaces: the RMSNorm stage of backend.py:1097-1108 / :1228-1251 (also :741-749,
 * :862-886, :1737-1745, :1990-2011); metal_ops.metal:3412-3537, :8107-8240, :14542.
 * y = x * inv * gamma, inv = 1/sqrt(mean(x^2)+eps); gamma NULL: unweighted.
 * backward: dx = (dres ? dres : 0) + inv*(dz*g - xhat*mean(dz*g*xhat)), dgamma += sum dz*xhat.
 * x/y/dz/dres/dx have `dtype`; gamma, inv_rms, dgamma are fp32. */
int ag_rmsnorm_forward(ag_ctx* ctx, const void* x, const float* gamma, void* y, float* inv_rms,
                       int64_t N, int C, float eps, int dtype);
int ag_rmsnorm_backward(ag_ctx* ctx, const void* dz, const void* x, const float* gamma,
                        const void* dres, void* dx, float* dgamma, void* partials,
                        size_t partials_bytes, int64_t N, int C, float eps, int dtype);

/* ---- a5 GELU (tanh form) --------------------------------------------------------------
 * Replaces: backend.py:376-414 cpu_gelu_forward/backward; metal_ops.metal:3775-3806.
 * backward: dx = (dres ? dres : 0) + dy * gelu'(x). */
int ag_gelu_forward(ag_ctx* ctx, const float* x, float* y, int64_t n);
int ag_gelu_backward(ag_ctx* ctx, const float* x, const float* dy, const float* dres, float* dx,
                     int64_t n);

/* ---- a6 SwiGLU on packed [gate|up] rows of width 2*I -----------------------------------
 * Replaces: backend.py:1113-1126 (forward), :1202-1217 (backward, in place);
 * metal_ops.metal:3808-3900.  backward overwrites gu with [dgate|dup]. */
int ag_swiglu_forward(ag_ctx* ctx, const void* gu, void* hidden, int64_t N, int I, int dtype);
int ag_swiglu_backward(ag_ctx* ctx, void* gu, const void* dhidden, int64_t N, int I, int dtype);

/* ---- a7 RoPE (rotate-half) on q and k, in place ---------------------------------------
 * Replaces: backend.py:1382-1417 apply_rope_np / apply_rope_backward_np and the inline
 * copies at :1755-1782, :1937-1958; metal_ops.metal:7423 rope_qk_inplace, :11732.
 * q: (B,T,H,D), k: (B,T,HKV,D) (k may be NULL); cos/sin: (T, D/2) fp32; position = t.
 * q_token_stride / k_token_stride are the element distance between consecutive tokens
 * (H*D / HKV*D when dense; larger when q,k are slices of a packed qkv row).
 * sin_sign=+1: lo' = lo*c - hi*s, hi' = lo*s + hi*c; sin_sign=-1 is its transpose. */
int ag_rope_qk(ag_ctx* ctx, void* q, void* k, const float* cos_tab, const float* sin_tab,
               int B, int T, int H, int HKV, int D, int64_t q_token_stride,
               int64_t k_token_stride, int sin_sign, int dtype);

/* ---- a8/a9 embedding gather and deterministic scatter-add ------------------------------
 * Replaces: backend.py:525-538 cpu_gather_forward/backward; metal_ops.metal:390-420,
 * :12395.  ids are int32; an id outside [0,V) writes zeros / is skipped and raises
 * AG_STATUS_BAD_INDEX.  backward: dtable[ids[i]] += dout[i] with a fixed summation order
 * (ascending i inside fixed-size groups of a row's occurrences, groups combined in
 * order); needs ag_scatter_add_scratch_bytes() of workspace. */
int ag_gather_forward(ag_ctx* ctx, const int32_t* ids, const float* table, float* out,
                      int64_t n_ids, int C, int V);
size_t ag_scatter_add_scratch_bytes(int64_t n_ids, int C, int V);
int ag_gather_backward(ag_ctx* ctx, const int32_t* ids, const float* dout, float* dtable,
                       void* scratch, size_t scratch_bytes, int64_t n_ids, int C, int V);

/* ---- a10/a11 fused linear + cross-entropy ----------------------------------------------
 * Replaces: backend.py:628-714 cpu_fused_linear_ce_forward/backward;
 * backend.py:3155-3301 + metal_ops.metal:8808-9180 (Metal path).
 * logits = X (N,C) . W (V,C)^T are produced one vocab chunk at a time and never stored
 * whole.  A row takes part when 0 <= target < V. */
/* precision: exact fp32 FFMA; 3xTF32 tensor cores (fp32-grade, the default); bf16 tensor cores (2e-2);
 * bf16 (hi, lo) pairs, three MMAs at the bf16 rate (products to ~2^-17; measured like 3xTF32: loss to
 * 1e-5, gradients to 1e-4) */
enum { AG_CE_FP32 = 0, AG_CE_3XTF32 = 1, AG_CE_BF16 = 2, AG_CE_BF16X3 = 3 };
enum { AG_CE_MEAN_ALL_ROWS = 0, AG_CE_MEAN_VALID = 1 };              /* reduction        */
enum { AG_CE_IGNORE_MASKED = 0, AG_CE_IGNORE_COMPAT_UNMASKED = 1 };  /* ignored-row grads */
typedef struct ag_flce_desc {
  int64_t N;
  int32_t C;
  int32_t V;
  int32_t vocab_chunk;   /* columns of logits alive at once (e.g. 4096)                    */
  int32_t precision;
  int32_t reduction;
  int32_t ignore_mode;
} ag_flce_desc;
size_t ag_flce_scratch_bytes(const ag_flce_desc* d);
/* loss: 1 float (device).  lse: N floats (device), log-sum-exp per row, consumed by
 * backward.  row_scale (N floats) may be NULL; with it loss = sum(row_loss*row_scale) and
 * dlogits rows are scaled by dloss*row_scale (backend.py:786-797, :850-853). */
int ag_flce_forward(ag_ctx* ctx, const ag_flce_desc* d, const float* X, const float* W,
                    const int32_t* targets, const float* row_scale, float* loss, float* lse,
                    void* scratch, size_t scratch_bytes);
/* dloss: device pointer to the upstream gradient of the loss (1 float).
 * dX (N,C) and dW (V,C) accumulate; either may be NULL. */
int ag_flce_backward(ag_ctx* ctx, const ag_flce_desc* d, const float* X, const float* W,
                     const int32_t* targets, const float* row_scale, const float* dloss,
                     const float* lse, float* dX, float* dW, void* scratch, size_t scratch_bytes);

/* ---- f2 linear projection with bias + residual epilogue --------------------------------------
 * Replaces: backend.py:2040-2058 cpu_fused_linear_add_forward and :2147-2259
 * cpu_fused_linear_add_backward (the branch whose `act` is materialised); Metal path
 * backend.py bind of FusedLinearAddOp.  out[N,C] = act[N,K] . w[K,C] + b[C] + x[N,C]; b and x may be
 * NULL; out may alias x (runtime.py:397-417 aliases them).  The GEMMs run on tcgen05 tensor cores,
 * precision AG_CE_3XTF32 (fp32-grade) or AG_CE_BF16; K and C must be multiples of 4 (8 for bf16).
 * backward accumulates: dx += dout, dact += dout . w^T, dw += act^T . dout, db += colsum(dout);
 * any of the four may be NULL. */
size_t ag_linear_add_scratch_bytes(int64_t N, int K, int C, int precision);
int ag_linear_add_forward(ag_ctx* ctx, const float* x, const float* act, const float* w, const float* b,
                          float* out, int64_t N, int K, int C, int precision, void* scratch,
                          size_t scratch_bytes);
int ag_linear_add_backward(ag_ctx* ctx, const float* dout, const float* act, const float* w, float* dx,
                           float* dact, float* dw, float* db, int64_t N, int K, int C, int precision,
                           void* scratch, size_t scratch_bytes);

/* ---- f3 AdamW fp32 step ----------------------------------------------------------------
 * Replaces: backend.py:2013-2038 cpu_adamw_step; metal_ops.metal:10139-10227.
 * g is read as g*grad_scale. */
int ag_adamw_step(ag_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, double lr,
                  double lr_t, double b1, double b2, double eps, double weight_decay,
                  double grad_scale);

/* ---- f4 parameter gradients stored as bf16 ------------------------------------------------
 * The reference keeps the gradient of a parameter whose grad_dtype is "bf16" as bf16 bit
 * patterns (uint16, runtime.py:185-202) and halves gradient memory and exchange bytes that way.
 * Rounding everywhere: to nearest, ties to even, Inf kept, NaN kept NaN (utils.py:20-27).
 *
 * ag_f32_to_bf16 replaces the `fp32_to_bf16` kernel (metal_ops.metal:12010-12041; call sites
 * backend.py:3298, :4743): dst = bf16(src), or bf16(src + float(dst)) when accumulate != 0 - how
 * a gradient computed in fp32 scratch is added into bf16 storage.  ag_bf16_to_f32 widens (exact).
 * ag_gather_backward_bf16 replaces `gather_backward_bf16_kernel` (metal_ops.metal:12395-12446,
 * backend.py:2807-2812): per touched table row, the fp32 sum of its dout rows in ascending
 * position order starting from zero, then row = bf16(float(row) + sum); untouched rows are not
 * written.  Scratch as for ag_gather_backward.
 * ag_adamw_step_bf16grad replaces `adamw_step` with its bf16-gradient flag (backend.py:5125-5140):
 * g is widened to fp32, then the fp32 step. */
int ag_f32_to_bf16(ag_ctx* ctx, const float* src, uint16_t* dst, int64_t n, int accumulate);
int ag_bf16_to_f32(ag_ctx* ctx, const uint16_t* src, float* dst, int64_t n);
int ag_gather_backward_bf16(ag_ctx* ctx, const int32_t* ids, const float* dout, uint16_t* dtable,
                            void* scratch, size_t scratch_bytes, int64_t n_ids, int C, int V);
int ag_adamw_step_bf16grad(ag_ctx* ctx, float* p, const uint16_t* g, float* m, float* v, int64_t n,
                           double lr, double lr_t, double b1, double b2, double eps,
                           double weight_decay, double grad_scale);

#ifdef __cplusplus
}
#endif
#endif /* AUTOGRAD_B200_H */
