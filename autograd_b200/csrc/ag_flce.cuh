// Internal interface between the fused linear+CE driver (ag_flce.cu) and the tcgen05
// tensor-core panels (ag_flce_tc.cu).
#pragma once

#include "ag_common.cuh"

// True when the tensor-core path takes this problem (precision mode, shape, alignment).
bool ag_flce_tc_supported(const ag_flce_desc* d);
// Extra workspace (split / converted operands, dlogits panel, split-K partials) the tensor-core path needs.
size_t ag_flce_tc_scratch_bytes(const ag_flce_desc* d);
// Converts X and W into the operand format of d->precision inside tc_scratch.
int ag_flce_tc_prepare(ag_ctx* ctx, const ag_flce_desc* d, const float* X, const float* W, void* tc_scratch);
// Forward of one panel without materialising it: logits tiles stay in TMEM, the GEMM epilogue
// reduces them to per-tile (max, sum exp) and picks the target logit; the partials are folded
// into run_max / run_sum (full-length arrays, indexed from r0 inside).
int ag_flce_tc_forward_panel(ag_ctx* ctx, const ag_flce_desc* d, void* tc_scratch, int64_t r0, int rows, int v0,
                             int vc, const int32_t* targets, float* run_max, float* run_sum, float* tgt_logit,
                             bool first_panel);
// Backward of one panel: the logits are recomputed, the GEMM epilogue turns them into dlogits in
// operand form, then dX[r0:r0+rows] += dl . W[v0:v0+vc] and dW[v0:v0+vc] += dl^T . X[r0:r0+rows]
// (either output may be null).  targets / lse / row_scale are the full-length arrays.
int ag_flce_tc_grads(ag_ctx* ctx, const ag_flce_desc* d, void* tc_scratch, int64_t r0, int rows, int v0, int vc,
                     const int32_t* targets, const float* lse, const float* row_scale, const float* dloss,
                     const float* denom, float* dX, float* dW);

// Token rows handled per pass over the vocabulary panels (the rows of the logits / dlogits panel held in
// scratch).  148 SMs x 128-row tiles = 74 CTA pairs x 256-row tiles: every GEMM of a full row tile then
// has a whole number of rounds over the SMs in the row direction (the dX panel, 1280 columns = 5 column
// tiles, takes exactly 5 rounds; with 16384 rows its 320 tiles took 5 rounds for 4.3 rounds of work).
constexpr int64_t AG_FLCE_ROWS_TILE = 148 * 128;

// Operand modes of the tensor-core GEMM: tf32 (hi, lo) pairs (3 MMAs per k-step, fp32-grade), bf16
// values (1 MMA), bf16 (hi, lo) pairs (3 MMAs at the bf16 rate).
enum AgTcMode { AG_TC_TF32X3 = 0, AG_TC_BF16 = 1, AG_TC_BF16X3 = 2 };

// ---- the tensor-core GEMM as a building block (used by the linear + bias + residual op) --------
struct AgTcOperand {
  const void* hi;   // tf32 "hi" parts, or the bf16 values
  const void* lo;   // tf32 "lo" parts (null / unused in bf16 mode)
  int64_t ld;       // elements between consecutive rows of the array as stored
  int mn_major;     // 0: stored [MN][K] (K contiguous); 1: stored [K][MN] (MN contiguous)
};
// D[M,N] (+)= A . B^T with A logically [M][K] and B logically [N][K], each stored K-major or MN-major
// (+ bias[n]) (+ resid[m,n]); split-K with an ordered reduction when a
// workspace is given and the problem has few tiles.
int ag_tc_gemm(ag_ctx* ctx, int mode, const AgTcOperand& A, const AgTcOperand& B, float* D, int64_t ldd, int M, int N,
               int K, bool accumulate, const float* bias, const float* resid, int64_t ld_resid, float* splitk_ws,
               size_t splitk_ws_bytes);
// src[R][Cc] (row stride lds) -> operand form [R][Cc] (row stride ldo): (hi, lo) tf32 pairs or bf16 in `hi`.
int ag_tc_split(ag_ctx* ctx, int mode, const float* src, int64_t lds, void* hi, void* lo, int64_t ldo, int64_t R,
                int Cc);
