// Linear projection with fused bias + residual epilogue: out = act . W + b + x.
//
// This is the node that closes every attention / MLP branch of the reference models and feeds the
// next norm (backend.py:2040-2058 forward, :2249-2259 backward).  The GEMMs run on the tcgen05
// kernel of ag_flce_tc.cu in 3xTF32 (fp32-grade) or bf16; bias and residual are added in its
// epilogue while the accumulator is read out of TMEM, so the projection output is written once and
// `out` may alias `x` (the reference aliases them when x dies here, runtime.py:397-417).
//   forward : out[N,C]  = act[N,K] . W[K,C] + b[C] + x[N,C]
//   backward: dx   += dout
//             dact += dout . W^T
//             dW   += act^T . dout          (split-K with ordered reduction)
//             db   += column sums of dout   (two passes, fixed order, no atomics)
#include "ag_flce.cuh"

namespace {

inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }
inline int64_t up8(int64_t x) { return (x + 7) & ~(int64_t)7; }

struct LinPlan {
  size_t es;
  int64_t ldn;  // row stride of the [*, N] transposed activations
  size_t act, act_lo, wT, wT_lo;                          // forward operands
  size_t dout, dout_lo, w, w_lo, actT, actT_lo, doutT, doutT_lo, splitk, splitk_bytes, colsum;  // backward
  size_t total_fwd, total_bwd;
};

constexpr int COLSUM_ROWS = 64;  // partial rows of the bias-gradient reduction

LinPlan lin_plan(int64_t N, int K, int C, int precision) {
  LinPlan p;
  const bool bf16 = precision == AG_CE_BF16;
  p.es = bf16 ? 2 : 4;
  p.ldn = up8(N);
  size_t off = 0;
  auto take = [&](size_t elems) { size_t o = off; off += up256(elems * p.es); return o; };
  p.act = take((size_t)N * K);
  p.act_lo = bf16 ? p.act : take((size_t)N * K);
  p.wT = take((size_t)C * up8(K));
  p.wT_lo = bf16 ? p.wT : take((size_t)C * up8(K));
  p.total_fwd = off;
  off = 0;
  p.dout = take((size_t)N * C);
  p.dout_lo = bf16 ? p.dout : take((size_t)N * C);
  p.w = take((size_t)K * C);
  p.w_lo = bf16 ? p.w : take((size_t)K * C);
  p.actT = take((size_t)K * p.ldn);
  p.actT_lo = bf16 ? p.actT : take((size_t)K * p.ldn);
  p.doutT = take((size_t)C * p.ldn);
  p.doutT_lo = bf16 ? p.doutT : take((size_t)C * p.ldn);
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
  for (; r + 4 <= r1; r += 4) {
    const float a0 = g[r * C + c], a1 = g[(r + 1) * C + c], a2 = g[(r + 2) * C + c], a3 = g[(r + 3) * C + c];
    acc += a0; acc += a1; acc += a2; acc += a3;
  }
  for (; r < r1; ++r) acc += g[r * C + c];
  partial[(int64_t)blockIdx.y * C + c] = acc;
}

__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, int P, int C, float* __restrict__ out) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  float acc = out[c];
  for (int p = 0; p < P; ++p) acc += partial[(int64_t)p * C + c];
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
  // act -> (hi, lo) [N][K];  W [K][C] -> W^T (hi, lo) [C][ldk]
  if ((rc = ag_tc_split(ctx, bf16, act, K, s + p.act, s + p.act_lo, K, nullptr, nullptr, 0, (int)N, K))) return rc;
  if ((rc = ag_tc_split(ctx, bf16, w, C, nullptr, nullptr, 0, s + p.wT, s + p.wT_lo, up8(K), K, C))) return rc;
  AgTcOperand A{s + p.act, s + p.act_lo, K};
  AgTcOperand B{s + p.wT, s + p.wT_lo, up8(K)};
  return ag_tc_gemm(ctx, bf16, A, B, out, C, (int)N, C, K, false, b, x, C, nullptr, 0);
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
  // dout -> (hi, lo) [N][C] for dact and, transposed [C][ldn], for dW
  if ((rc = ag_tc_split(ctx, bf16, dout, C, dact ? s + p.dout : nullptr, s + p.dout_lo, C, dw ? s + p.doutT : nullptr,
                        s + p.doutT_lo, p.ldn, (int)N, C)))
    return rc;
  if (dact) {
    // dact[N,K] += dout[N,C] . (W[K,C])^T : W is K-major as stored
    if ((rc = ag_tc_split(ctx, bf16, w, C, s + p.w, s + p.w_lo, C, nullptr, nullptr, 0, K, C))) return rc;
    AgTcOperand A{s + p.dout, s + p.dout_lo, C};
    AgTcOperand B{s + p.w, s + p.w_lo, C};
    if ((rc = ag_tc_gemm(ctx, bf16, A, B, dact, K, (int)N, K, C, true, nullptr, nullptr, 0, nullptr, 0))) return rc;
  }
  if (dw) {
    // dW[K,C] += act^T[K,N] . (dout^T[C,N])^T
    if ((rc = ag_tc_split(ctx, bf16, act, K, nullptr, nullptr, 0, s + p.actT, s + p.actT_lo, p.ldn, (int)N, K))) return rc;
    AgTcOperand A{s + p.actT, s + p.actT_lo, p.ldn};
    AgTcOperand B{s + p.doutT, s + p.doutT_lo, p.ldn};
    if ((rc = ag_tc_gemm(ctx, bf16, A, B, dw, C, K, C, (int)N, true, nullptr, nullptr, 0,
                         reinterpret_cast<float*>(s + p.splitk), p.splitk_bytes)))
      return rc;
  }
  return AG_OK;
}
