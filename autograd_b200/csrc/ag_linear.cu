// Linear projection with fused bias + residual epilogue: out = act . W + b + x.
//
// This is the node that closes every attention / MLP branch of the reference models and feeds the
// next norm (backend.py:2040-2058 forward, :2249-2259 backward).  The GEMMs run on the tcgen05
// kernel of ag_flce_tc.cu in 3xTF32 (fp32-grade) or bf16; bias and residual are added in its
// epilogue while the accumulator is read out of TMEM, so the projection output is written once and
// `out` may alias `x` (the reference aliases them when x dies here, runtime.py:397-417).
//   forward : out[N,C]  = act[N,K] . W[K,C] + b[C] + x[N,C]     (W read MN-major)
//   backward: dx   += dout
//             dact += dout . W^T                                 (both K-major as stored)
//             dW   += act^T . dout          (both MN-major; split-K with ordered reduction)
//             db   += column sums of dout   (two passes, fixed order, no atomics)
// act, W and dout are only converted to the operand format (tf32 hi/lo pairs or bf16); the GEMM
// reads them in whichever orientation each product needs, so no transposed copy is made.
#include "ag_flce.cuh"

namespace {

inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

struct LinPlan {
  size_t es;
  size_t act, act_lo, w, w_lo;                              // operands of forward and backward
  size_t dout, dout_lo, splitk, splitk_bytes, colsum;       // backward only
  size_t total_fwd, total_bwd;
};

constexpr int COLSUM_ROWS = 256;  // partial rows of the bias-gradient reduction

LinPlan lin_plan(int64_t N, int K, int C, int precision) {
  LinPlan p;
  const bool bf16 = precision == AG_CE_BF16;
  p.es = bf16 ? 2 : 4;
  size_t off = 0;
  auto take = [&](size_t elems) { size_t o = off; off += up256(elems * p.es); return o; };
  p.act = take((size_t)N * K);
  p.act_lo = bf16 ? p.act : take((size_t)N * K);
  p.w = take((size_t)K * C);
  p.w_lo = bf16 ? p.w : take((size_t)K * C);
  p.total_fwd = off;
  p.dout = take((size_t)N * C);
  p.dout_lo = bf16 ? p.dout : take((size_t)N * C);
  p.splitk = off;
  p.splitk_bytes = up256((size_t)16 * K * C * sizeof(float));
  off += p.splitk_bytes;
  p.colsum = off;
  off += up256((size_t)COLSUM_ROWS * C * sizeof(float));
  p.total_bwd = off;
  return p;
}

// partial[rchunk][c] = sum of g over the rows of chunk rchunk (rows in ascending order)
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const float* __restrict__ g, int64_t N, int C, float* __restrict__ partial) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  const int64_t per = (N + gridDim.y - 1) / gridDim.y;
  const int64_t r0 = (int64_t)blockIdx.y * per;
  const int64_t r1 = r0 + per < N ? r0 + per : N;
  float acc = 0.0f;
  int64_t r = r0;
  for (; r + 8 <= r1; r += 8) {  // eight rows in flight, added in row order
    float a[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) a[u] = __ldcs(g + (r + u) * C + c);
#pragma unroll
    for (int u = 0; u < 8; ++u) acc += a[u];
  }
  for (; r < r1; ++r) acc += g[r * C + c];
  partial[(int64_t)blockIdx.y * C + c] = acc;
}

__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, int P, int C, float* __restrict__ out) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  float acc = out[c];
  int p = 0;
  for (; p + 8 <= P; p += 8) {
    float a[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) a[u] = partial[(int64_t)(p + u) * C + c];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc += a[u];
  }
  for (; p < P; ++p) acc += partial[(int64_t)p * C + c];
  out[c] = acc;
}

int check_shape(ag_ctx* ctx, int64_t N, int K, int C, int precision) {
  AG_REQUIRE(ctx, N > 0 && K > 0 && C > 0 && N < (1ll << 31), "linear_add: bad shape N=%lld K=%d C=%d", (long long)N, K, C);
  AG_REQUIRE(ctx, precision == AG_CE_3XTF32 || precision == AG_CE_BF16,
             "linear_add: precision must be AG_CE_3XTF32 or AG_CE_BF16 (tensor-core op)");
  const int q = precision == AG_CE_BF16 ? 8 : 4;
  AG_REQUIRE(ctx, K % q == 0 && C % q == 0, "linear_add: K and C must be multiples of %d for the TMA operand rows", q);
  return AG_OK;
}

}  // namespace

extern "C" size_t ag_linear_add_scratch_bytes(int64_t N, int K, int C, int precision) {
  if (N <= 0 || K <= 0 || C <= 0) return 0;
  const LinPlan p = lin_plan(N, K, C, precision);
  return p.total_fwd > p.total_bwd ? p.total_fwd : p.total_bwd;
}

extern "C" int ag_linear_add_forward(ag_ctx* ctx, const float* x, const float* act, const float* w, const float* b,
                                     float* out, int64_t N, int K, int C, int precision, void* scratch,
                                     size_t scratch_bytes) {
  if (!ctx) return AG_ERR_INVALID;
  int rc = check_shape(ctx, N, K, C, precision);
  if (rc) return rc;
  AG_REQUIRE(ctx, act && w && out, "ag_linear_add_forward: null pointer");
  const LinPlan p = lin_plan(N, K, C, precision);
  if (!scratch || scratch_bytes < p.total_fwd)
    AG_FAIL(ctx, AG_ERR_SCRATCH, "ag_linear_add_forward: scratch has %zu bytes, needs %zu", scratch_bytes, p.total_fwd);
  AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "ag_linear_add_forward: scratch not 256-byte aligned");
  unsigned char* s = static_cast<unsigned char*>(scratch);
  const bool bf16 = precision == AG_CE_BF16;
  if ((rc = ag_tc_split(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, act, K, s + p.act, s + p.act_lo, K, N, K))) return rc;
  if ((rc = ag_tc_split(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, w, C, s + p.w, s + p.w_lo, C, K, C))) return rc;
  // B[n = C][k = K] is W[K][C] as stored with the contraction index as row index: MN-major.
  // K is taken in pieces: an accumulation chain inside the tensor core is biased in proportion to its
  // length (its adds truncate), the pieces' results are added by the epilogue with round-to-nearest.
  // Measured against the fp32 reference (N 4096, C 1280, max |d| / (rms + |ref|)): chains of 2048 give
  // 2.5e-5 (K 1280) and 3.6e-5 (K 5120), chains of 512 9.6e-6 / 9.3e-6, chains of 256 5.5e-6 / 4.6e-6, at
  // 1.0 / 1.15 / 1.5 times the forward time.  The default limit of 384 holds the fp32-forward bound of
  // 1e-5; the pieces are of equal length (K 1280: four of 320).  The first piece carries bias and residual.
  const size_t es = bf16 ? 2 : 4;
  int k_chunk = K;
  if (!bf16) {
    const int pieces = (K + ctx->linear_k_chunk - 1) / ctx->linear_k_chunk;
    k_chunk = ((K + pieces - 1) / pieces + 31) / 32 * 32;
  }
  for (int k0 = 0; k0 < K; k0 += k_chunk) {
    const int kc = K - k0 < k_chunk ? K - k0 : k_chunk;
    AgTcOperand A{s + p.act + (size_t)k0 * es, s + p.act_lo + (size_t)k0 * es, K, 0};
    AgTcOperand B{s + p.w + (size_t)k0 * C * es, s + p.w_lo + (size_t)k0 * C * es, C, 1};
    const bool first = k0 == 0;
    if ((rc = ag_tc_gemm(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, A, B, out, C, (int)N, C, kc, !first, first ? b : nullptr,
                         first ? x : nullptr, C, nullptr, 0)))
      return rc;
  }
  return AG_OK;
}

extern "C" int ag_linear_add_backward(ag_ctx* ctx, const float* dout, const float* act, const float* w, float* dx,
                                      float* dact, float* dw, float* db, int64_t N, int K, int C, int precision,
                                      void* scratch, size_t scratch_bytes) {
  if (!ctx) return AG_ERR_INVALID;
  int rc = check_shape(ctx, N, K, C, precision);
  if (rc) return rc;
  AG_REQUIRE(ctx, dout, "ag_linear_add_backward: null dout");
  AG_REQUIRE(ctx, (!dact || w) && (!dw || act), "ag_linear_add_backward: dact needs w, dw needs act");
  const LinPlan p = lin_plan(N, K, C, precision);
  if (!scratch || scratch_bytes < p.total_bwd)
    AG_FAIL(ctx, AG_ERR_SCRATCH, "ag_linear_add_backward: scratch has %zu bytes, needs %zu", scratch_bytes, p.total_bwd);
  AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "ag_linear_add_backward: scratch not 256-byte aligned");
  unsigned char* s = static_cast<unsigned char*>(scratch);
  const bool bf16 = precision == AG_CE_BF16;
  if (dx) {
    rc = ag_add_backward(ctx, dout, dx, nullptr, N * (int64_t)C);
    if (rc) return rc;
  }
  if (db) {
    dim3 grid((C + 255) / 256, COLSUM_ROWS);
    float* partial = reinterpret_cast<float*>(s + p.colsum);
    colsum_partial_kernel<<<grid, 256, 0, ctx->stream>>>(dout, N, C, partial);
    AG_LAUNCHED(ctx, "colsum_partial_kernel");
    colsum_final_kernel<<<(C + 255) / 256, 256, 0, ctx->stream>>>(partial, COLSUM_ROWS, C, db);
    AG_LAUNCHED(ctx, "colsum_final_kernel");
  }
  if (!dact && !dw) return AG_OK;
  if ((rc = ag_tc_split(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, dout, C, s + p.dout, s + p.dout_lo, C, N, C))) return rc;
  if (dact) {
    // dact[N,K] += dout[N,C] . (W[K,C])^T : both K-major as stored
    if ((rc = ag_tc_split(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, w, C, s + p.w, s + p.w_lo, C, K, C))) return rc;
    // contraction over C in chunks of at most 2048 (bounded accumulation chains, see the forward)
    const size_t es_ = bf16 ? 2 : 4;
    const int c_chunk = bf16 ? C : 2048;
    for (int c0 = 0; c0 < C; c0 += c_chunk) {
      const int cc = C - c0 < c_chunk ? C - c0 : c_chunk;
      AgTcOperand A{s + p.dout + (size_t)c0 * es_, s + p.dout_lo + (size_t)c0 * es_, C, 0};
      AgTcOperand B{s + p.w + (size_t)c0 * es_, s + p.w_lo + (size_t)c0 * es_, C, 0};
      if ((rc = ag_tc_gemm(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, A, B, dact, K, (int)N, K, cc, true, nullptr, nullptr, 0,
                           nullptr, 0)))
        return rc;
    }
  }
  if (dw) {
    // dW[K,C] += act^T . dout : the contraction index (token row) is the row index of both as stored
    if ((rc = ag_tc_split(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, act, K, s + p.act, s + p.act_lo, K, N, K))) return rc;
    // Row tiles of at most 32768 tokens: with the 16 splits the workspace allows, an accumulation chain
    // inside the tensor core then covers at most 2048 rows (its truncating adds bias long chains); the
    // tiles' results are added into dW by the epilogue of the split-K reduction, round-to-nearest.
    const size_t es = bf16 ? 2 : 4;
    for (int64_t r0 = 0; r0 < N; r0 += 32768) {
      const int rows = (int)(N - r0 < 32768 ? N - r0 : 32768);
      AgTcOperand A{s + p.act + (size_t)r0 * K * es, s + p.act_lo + (size_t)r0 * K * es, K, 1};
      AgTcOperand B{s + p.dout + (size_t)r0 * C * es, s + p.dout_lo + (size_t)r0 * C * es, C, 1};
      if ((rc = ag_tc_gemm(ctx, bf16 ? AG_TC_BF16 : AG_TC_TF32X3, A, B, dw, C, K, C, rows, true, nullptr, nullptr, 0,
                           reinterpret_cast<float*>(s + p.splitk), p.splitk_bytes)))
        return rc;
    }
  }
  return AG_OK;
}
