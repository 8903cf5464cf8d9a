// Fused linear + cross-entropy head, vocabulary-chunked: the (N,V) logits never exist
// as a whole, only one (rows x vocab_chunk) panel at a time inside the caller's scratch.
//
// forward : per panel  L = X . W[v0:v1]^T  ->  online (max, sum-exp) per row + target pick;
//           then lse = max + log(sum), row_loss = lse - logit[target] (0 for ignored rows),
//           loss = sum(row_loss)/denom (fixed-order tree sum, no atomics).
// backward: per panel  L recomputed, overwritten by dlogits = scale*(exp(L-lse) - onehot),
//           dX += dlogits . W[v0:v1],  dW[v0:v1] += dlogits^T . X.
//
// Every dX row tile and every dW vocab panel has exactly one writer CTA per output tile,
// so the accumulation order is fixed.  The GEMMs of this file are the exact-fp32 (FFMA)
// implementation used for AG_CE_FP32 and for shapes the tensor-core path does not take;
// ag_flce_tc.cu provides the tcgen05 panels for AG_CE_3XTF32 / AG_CE_BF16 / AG_CE_BF16X3.
#include <math.h>

#include "ag_common.cuh"
#include "ag_flce.cuh"

namespace {

// ---------------------------------------------------------------------------------------
// exact fp32 GEMM, generic strides:  Cmat[m,n] (+)= sum_k A(m,k) * B(k,n)
//   A(m,k) = A[m*sam + k*sak],  B(k,n) = B[k*sbk + n*sbn],  Cmat row-major with ldc.
// 64x64 output tile per CTA, 16-deep k slices, 4x4 outputs per thread; every load guarded,
// so any M, N, K is accepted.
// ---------------------------------------------------------------------------------------
constexpr int GT = 64, GK = 16, GTHREADS = 256;

__global__ void __launch_bounds__(GTHREADS)
sgemm_generic_kernel(const float* __restrict__ A, int64_t sam, int64_t sak, const float* __restrict__ B, int64_t sbk,
                     int64_t sbn, float* Cmat, int64_t ldc, int M, int N, int K, int accumulate) {
  __shared__ float As[GK][GT + 4];
  __shared__ float Bs[GK][GT + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // load mapping: choose the fastest-varying thread index along the unit-stride dimension
  const bool a_k_fast = sak == 1;
  const bool b_n_fast = sbn == 1;
  for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
    for (int it = 0; it < (GT * GK) / GTHREADS; ++it) {
      const int e = it * GTHREADS + threadIdx.x;
      int mm, kk;
      if (a_k_fast) { kk = e % GK; mm = e / GK; } else { mm = e % GT; kk = e / GT; }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? A[(int64_t)gm * sam + (int64_t)gk * sak] : 0.0f;
      int nn, kb;
      if (b_n_fast) { nn = e % GT; kb = e / GT; } else { kb = e % GK; nn = e / GK; }
      const int gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < N && gkb < K) ? B[(int64_t)gkb * sbk + (int64_t)gn * sbn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float* p = Cmat + (int64_t)gm * ldc + gn;
      *p = accumulate ? *p + acc[i][j] : acc[i][j];
    }
  }
}

int sgemm(ag_ctx* ctx, const float* A, int64_t sam, int64_t sak, const float* B, int64_t sbk, int64_t sbn, float* Cm,
          int64_t ldc, int M, int N, int K, bool accumulate) {
  dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  sgemm_generic_kernel<<<grid, GTHREADS, 0, ctx->stream>>>(A, sam, sak, B, sbk, sbn, Cm, ldc, M, N, K,
                                                           accumulate ? 1 : 0);
  AG_LAUNCHED(ctx, "sgemm_generic_kernel");
  return AG_OK;
}

// ---------------------------------------------------------------------------------------
// row kernels on a logits panel L[rows][ld] (columns [0,vc) valid), vocab offset v0
// ---------------------------------------------------------------------------------------
constexpr int CE_THREADS = 256;

__device__ __forceinline__ float block_reduce_max(float v, float* s_red) {
  v = ag_warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = s_red[0];
#pragma unroll
  for (int w = 1; w < CE_THREADS / 32; ++w) t = fmaxf(t, s_red[w]);
  return t;
}

__device__ __forceinline__ float block_reduce_sum(float v, float* s_red) {
  v = ag_warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int w = 0; w < CE_THREADS / 32; ++w) t += s_red[w];  // fixed order
  return t;
}

// Online softmax statistics: merges this panel into run_max/run_sum, picks the target logit.
__global__ void __launch_bounds__(CE_THREADS)
ce_panel_stats_kernel(const float* __restrict__ L, int64_t ld, int vc, int v0, const int32_t* __restrict__ targets,
                      float* __restrict__ run_max, float* __restrict__ run_sum, float* __restrict__ tgt_logit,
                      int first_panel) {
  __shared__ float s_red[CE_THREADS / 32];
  const int64_t row = blockIdx.x;
  const float* l = L + row * ld;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < vc; c += CE_THREADS) m = fmaxf(m, l[c]);
  m = block_reduce_max(m, s_red);
  float s = 0.0f;
  for (int c = threadIdx.x; c < vc; c += CE_THREADS) s += expf(l[c] - m);
  s = block_reduce_sum(s, s_red);
  if (threadIdx.x == 0) {
    if (first_panel) {
      run_max[row] = m;
      run_sum[row] = s;
    } else {
      const float pm = run_max[row], ps = run_sum[row];
      const float nm = fmaxf(pm, m);
      run_sum[row] = ps * expf(pm - nm) + s * expf(m - nm);
      run_max[row] = nm;
    }
    const int t = targets[row];
    if (t >= v0 && t < v0 + vc) tgt_logit[row] = l[t - v0];
  }
}

// lse, row_loss; then the loss itself by one CTA (fixed-order strided sums + tree).
__global__ void __launch_bounds__(1024)
ce_finalize_kernel(const float* __restrict__ run_max, const float* __restrict__ run_sum,
                   const float* __restrict__ tgt_logit, const int32_t* __restrict__ targets,
                   const float* __restrict__ row_scale, float* __restrict__ lse, float* __restrict__ loss, int64_t N,
                   int V, int reduction) {
  __shared__ float s_sum[1024];
  __shared__ int s_cnt[1024];
  float acc = 0.0f;
  int cnt = 0;
  for (int64_t r = threadIdx.x; r < N; r += 1024) {
    const float e = run_max[r] + logf(run_sum[r]);
    lse[r] = e;
    const int t = targets[r];
    if (t >= 0 && t < V) {
      float rl = e - tgt_logit[r];
      if (row_scale) rl *= row_scale[r];
      acc += rl;
      ++cnt;
    }
  }
  s_sum[threadIdx.x] = acc;
  s_cnt[threadIdx.x] = cnt;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) {
      s_sum[threadIdx.x] += s_sum[threadIdx.x + o];
      s_cnt[threadIdx.x] += s_cnt[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    float denom = 1.0f;
    if (!row_scale) denom = reduction == AG_CE_MEAN_ALL_ROWS ? (float)N : (float)(s_cnt[0] > 0 ? s_cnt[0] : 1);
    loss[0] = s_sum[0] / denom;
  }
}

// n_valid -> out[0] (as float denominator per the reduction mode)
__global__ void __launch_bounds__(1024)
ce_denominator_kernel(const int32_t* __restrict__ targets, int64_t N, int V, int reduction, float* __restrict__ out) {
  __shared__ int s_cnt[1024];
  int cnt = 0;
  for (int64_t r = threadIdx.x; r < N; r += 1024) {
    const int t = targets[r];
    cnt += (t >= 0 && t < V) ? 1 : 0;
  }
  s_cnt[threadIdx.x] = cnt;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) s_cnt[threadIdx.x] += s_cnt[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0)
    out[0] = reduction == AG_CE_MEAN_ALL_ROWS ? (float)N : (float)(s_cnt[0] > 0 ? s_cnt[0] : 1);
}

// L <- scale_row * (exp(L - lse) - onehot(target)), in place.
__global__ void __launch_bounds__(CE_THREADS)
ce_panel_dlogits_kernel(float* __restrict__ L, int64_t ld, int vc, int v0, const int32_t* __restrict__ targets,
                        const float* __restrict__ lse, const float* __restrict__ row_scale,
                        const float* __restrict__ dloss, const float* __restrict__ denom, int V, int ignore_mode) {
  const int64_t row = blockIdx.x;
  float* l = L + row * ld;
  const int t = targets[row];
  const bool valid = t >= 0 && t < V;
  const float scale = row_scale ? dloss[0] * row_scale[row] : dloss[0] / denom[0];
  if (!valid && ignore_mode == AG_CE_IGNORE_MASKED) {
    for (int c = threadIdx.x; c < vc; c += CE_THREADS) l[c] = 0.0f;
    return;
  }
  const float e = lse[row];
  const int tc = valid ? t - v0 : -1;
  for (int c = threadIdx.x; c < vc; c += CE_THREADS) {
    float p = expf(l[c] - e);
    if (c == tc) p -= 1.0f;
    l[c] = p * scale;
  }
}

struct FlcePlan {
  int64_t rows_per_tile;
  size_t off_panel, off_max, off_sum, off_tgt, off_denom, total;
};

inline size_t al256(size_t x) { return (x + 255) & ~(size_t)255; }

FlcePlan flce_plan(const ag_flce_desc* d) {
  FlcePlan p;
  p.rows_per_tile = d->N < AG_FLCE_ROWS_TILE ? d->N : AG_FLCE_ROWS_TILE;
  const int vc = d->vocab_chunk < d->V ? d->vocab_chunk : d->V;
  size_t off = 0;
  p.off_panel = off; off += al256((size_t)p.rows_per_tile * vc * 4);
  p.off_max = off; off += al256((size_t)d->N * 4);
  p.off_sum = off; off += al256((size_t)d->N * 4);
  p.off_tgt = off; off += al256((size_t)d->N * 4);
  p.off_denom = off; off += 256;
  p.total = off;
  return p;
}

int check_desc(ag_ctx* ctx, const ag_flce_desc* d) {
  AG_REQUIRE(ctx, d, "flce: null descriptor");
  AG_REQUIRE(ctx, d->N > 0 && d->C > 0 && d->V > 0 && d->vocab_chunk > 0, "flce: bad shape N=%lld C=%d V=%d chunk=%d",
             (long long)d->N, d->C, d->V, d->vocab_chunk);
  AG_REQUIRE(ctx, d->N < (1ll << 31), "flce: N too large");
  AG_REQUIRE(ctx, d->precision >= AG_CE_FP32 && d->precision <= AG_CE_BF16X3, "flce: unknown precision %d", d->precision);
  AG_REQUIRE(ctx, d->reduction == AG_CE_MEAN_ALL_ROWS || d->reduction == AG_CE_MEAN_VALID, "flce: unknown reduction %d",
             d->reduction);
  AG_REQUIRE(ctx, d->ignore_mode == AG_CE_IGNORE_MASKED || d->ignore_mode == AG_CE_IGNORE_COMPAT_UNMASKED,
             "flce: unknown ignore_mode %d", d->ignore_mode);
  return AG_OK;
}

}  // namespace

// =========================================================================================
extern "C" size_t ag_flce_scratch_bytes(const ag_flce_desc* d) {
  if (!d || d->N <= 0 || d->C <= 0 || d->V <= 0 || d->vocab_chunk <= 0) return 0;
  size_t base = flce_plan(d).total;
  if (d->precision != AG_CE_FP32 && ag_flce_tc_supported(d)) base += ag_flce_tc_scratch_bytes(d);
  return base;
}

extern "C" int ag_flce_forward(ag_ctx* ctx, const ag_flce_desc* d, const float* X, const float* W,
                               const int32_t* targets, const float* row_scale, float* loss, float* lse, void* scratch,
                               size_t scratch_bytes) {
  if (!ctx) return AG_ERR_INVALID;
  int rc = check_desc(ctx, d);
  if (rc) return rc;
  AG_REQUIRE(ctx, X && W && targets && loss && lse, "ag_flce_forward: null pointer");
  const size_t need = ag_flce_scratch_bytes(d);
  if (!scratch || scratch_bytes < need)
    AG_FAIL(ctx, AG_ERR_SCRATCH, "ag_flce_forward: scratch has %zu bytes, needs %zu", scratch_bytes, need);
  AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "ag_flce_forward: scratch not 256-byte aligned");
  const FlcePlan p = flce_plan(d);
  unsigned char* base = static_cast<unsigned char*>(scratch);
  float* panel = reinterpret_cast<float*>(base + p.off_panel);
  float* run_max = reinterpret_cast<float*>(base + p.off_max);
  float* run_sum = reinterpret_cast<float*>(base + p.off_sum);
  float* tgt = reinterpret_cast<float*>(base + p.off_tgt);
  const bool tc = d->precision != AG_CE_FP32 && ag_flce_tc_supported(d);
  void* tc_scratch = base + p.total;
  if (tc) {
    rc = ag_flce_tc_prepare(ctx, d, X, W, tc_scratch);
    if (rc) return rc;
  }
  AG_CUDA(ctx, cudaMemsetAsync(tgt, 0, (size_t)d->N * 4, ctx->stream));
  const int C = d->C, V = d->V;
  for (int64_t r0 = 0; r0 < d->N; r0 += p.rows_per_tile) {
    const int rows = (int)((d->N - r0) < p.rows_per_tile ? (d->N - r0) : p.rows_per_tile);
    for (int v0 = 0; v0 < V; v0 += d->vocab_chunk) {
      const int vc = (V - v0) < d->vocab_chunk ? (V - v0) : d->vocab_chunk;
      if (tc) {
        rc = ag_flce_tc_forward_panel(ctx, d, tc_scratch, r0, rows, v0, vc, targets, run_max, run_sum, tgt, v0 == 0);
        if (rc) return rc;
        continue;
      }
      rc = sgemm(ctx, X + r0 * C, C, 1, W + (int64_t)v0 * C, 1, C, panel, vc, rows, vc, C, false);
      if (rc) return rc;
      ce_panel_stats_kernel<<<rows, CE_THREADS, 0, ctx->stream>>>(panel, vc, vc, v0, targets + r0, run_max + r0,
                                                                  run_sum + r0, tgt + r0, v0 == 0);
      AG_LAUNCHED(ctx, "ce_panel_stats_kernel");
    }
  }
  ce_finalize_kernel<<<1, 1024, 0, ctx->stream>>>(run_max, run_sum, tgt, targets, row_scale, lse, loss, d->N, V,
                                                  d->reduction);
  AG_LAUNCHED(ctx, "ce_finalize_kernel");
  return AG_OK;
}

extern "C" int ag_flce_backward(ag_ctx* ctx, const ag_flce_desc* d, const float* X, const float* W,
                                const int32_t* targets, const float* row_scale, const float* dloss, const float* lse,
                                float* dX, float* dW, void* scratch, size_t scratch_bytes) {
  if (!ctx) return AG_ERR_INVALID;
  int rc = check_desc(ctx, d);
  if (rc) return rc;
  AG_REQUIRE(ctx, X && W && targets && dloss && lse, "ag_flce_backward: null pointer");
  if (!dX && !dW) return AG_OK;
  const size_t need = ag_flce_scratch_bytes(d);
  if (!scratch || scratch_bytes < need)
    AG_FAIL(ctx, AG_ERR_SCRATCH, "ag_flce_backward: scratch has %zu bytes, needs %zu", scratch_bytes, need);
  AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "ag_flce_backward: scratch not 256-byte aligned");
  const FlcePlan p = flce_plan(d);
  unsigned char* base = static_cast<unsigned char*>(scratch);
  float* panel = reinterpret_cast<float*>(base + p.off_panel);
  float* denom = reinterpret_cast<float*>(base + p.off_denom);
  const bool tc = d->precision != AG_CE_FP32 && ag_flce_tc_supported(d);
  void* tc_scratch = base + p.total;
  if (tc) {
    rc = ag_flce_tc_prepare(ctx, d, X, W, tc_scratch);
    if (rc) return rc;
  }
  ce_denominator_kernel<<<1, 1024, 0, ctx->stream>>>(targets, d->N, d->V, d->reduction, denom);
  AG_LAUNCHED(ctx, "ce_denominator_kernel");
  const int C = d->C, V = d->V;
  for (int64_t r0 = 0; r0 < d->N; r0 += p.rows_per_tile) {
    const int rows = (int)((d->N - r0) < p.rows_per_tile ? (d->N - r0) : p.rows_per_tile);
    for (int v0 = 0; v0 < V; v0 += d->vocab_chunk) {
      const int vc = (V - v0) < d->vocab_chunk ? (V - v0) : d->vocab_chunk;
      if (tc) {
        rc = ag_flce_tc_grads(ctx, d, tc_scratch, r0, rows, v0, vc, targets, lse, row_scale, dloss, denom, dX, dW);
        if (rc) return rc;
        continue;
      }
      rc = sgemm(ctx, X + r0 * C, C, 1, W + (int64_t)v0 * C, 1, C, panel, vc, rows, vc, C, false);
      if (rc) return rc;
      ce_panel_dlogits_kernel<<<rows, CE_THREADS, 0, ctx->stream>>>(panel, vc, vc, v0, targets + r0, lse + r0,
                                                                    row_scale ? row_scale + r0 : nullptr, dloss, denom,
                                                                    V, d->ignore_mode);
      AG_LAUNCHED(ctx, "ce_panel_dlogits_kernel");
      if (dX) {
        // dX[r0:r0+rows, :] += dl (rows x vc) . W[v0:v0+vc, :] (vc x C)
        rc = sgemm(ctx, panel, vc, 1, W + (int64_t)v0 * C, C, 1, dX + r0 * C, C, rows, C, vc, true);
        if (rc) return rc;
      }
      if (dW) {
        // dW[v0:v0+vc, :] += dl^T (vc x rows) . X[r0:r0+rows, :] (rows x C)
        rc = sgemm(ctx, panel, 1, vc, X + r0 * C, C, 1, dW + (int64_t)v0 * C, C, vc, C, rows, true);
        if (rc) return rc;
      }
    }
  }
  return AG_OK;
}
