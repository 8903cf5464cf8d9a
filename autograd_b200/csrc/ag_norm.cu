// (residual add +) LayerNorm and RMSNorm, forward and backward.
//
// Layout: one warp owns one row at a time and keeps the whole row in registers
// (KP 16-byte packets per lane, packet p of lane l covers columns (p*32+l)*NV ..+NV), so a
// row is read from HBM exactly once per kernel even though the statistics are two-pass
// (mean, then centred variance - the reference's formulation, backend.py:423-429).
// gamma/beta are staged once per CTA in shared memory by the bulk-copy (TMA) engine.
// Rows are distributed grid-stride over a persistent grid (a multiple of the SM count).
//
// Backward column sums (dgamma, dbeta) use no atomics: every lane accumulates its own
// columns over the rows its warp visits, the CTA folds its warps through shared memory in
// warp order and writes one partial row, and a second kernel adds the partial rows in
// index order into dgamma/dbeta.  The summation order is therefore fixed by (N, C, grid).
//
// Shapes that do not fit the register layout (C not a multiple of the packet width, or a
// row longer than 16 packets per lane) take a CTA-per-row kernel with scalar accesses.
#include "ag_common.cuh"

namespace {

constexpr int NORM_WARPS = 8;
constexpr int NORM_THREADS = NORM_WARPS * 32;

enum NormKind { kLayerNorm = 0, kRmsNorm = 1 };

// ---------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------
template <typename T, int KP, int KIND>
__global__ void __launch_bounds__(NORM_THREADS)
norm_forward_kernel(const T* x, const T* r, const float* __restrict__ gamma,
                    const float* __restrict__ beta, T* h, T* __restrict__ y, float* __restrict__ stat0,
                    float* __restrict__ stat1, int64_t N, int C, float eps, uint32_t stage_poll_limit, int* status,
                    int pdl_early) {
  ag_pdl_wait();
  // Early trigger only when the whole grid is resident at once: otherwise the next kernel's CTAs,
  // which only wait, would take SM slots from this grid's later waves.
  if (pdl_early) ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* s_gamma = reinterpret_cast<float*>(smem_raw);
  float* s_beta = s_gamma + C;
  __shared__ __align__(8) uint64_t s_bar;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const float inv_c = 1.0f / (float)C;
  // Narrow rows keep gamma/beta in registers (plain loads that overlap the first row's loads);
  // wide rows stage them once per CTA in shared memory through the bulk-copy engine.
  constexpr bool IN_REGS = KP <= 4;
  float rg[IN_REGS ? KP : 1][NV], rb[IN_REGS ? KP : 1][NV];
  if (IN_REGS) {
#pragma unroll
    for (int p = 0; p < (IN_REGS ? KP : 1); ++p) {
      const int col = (p * 32 + lane) * NV;
#pragma unroll
      for (int e = 0; e < NV; ++e) {
        rg[p][e] = (gamma && col < C) ? __ldg(gamma + col + e) : 1.0f;
        rb[p][e] = (KIND == kLayerNorm && col < C) ? __ldg(beta + col + e) : 0.0f;
      }
    }
  } else if (gamma) {
    ag_stage_vectors(s_gamma, gamma, s_beta, (KIND == kLayerNorm) ? beta : nullptr, C, &s_bar, status, stage_poll_limit);
  }

  for (int64_t row = (int64_t)blockIdx.x * NORM_WARPS + warp; row < N; row += (int64_t)gridDim.x * NORM_WARPS) {
    float v[KP][NV];
    const T* xr = x + row * C;
#pragma unroll
    for (int p = 0; p < KP; ++p) {
      const int col = (p * 32 + lane) * NV;
      if (col < C) {
        Pack<T>::load_stream(xr + col, v[p]);
      } else {
#pragma unroll
        for (int e = 0; e < NV; ++e) v[p][e] = 0.0f;
      }
    }
    if (r) {
      const T* rr = r + row * C;
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) {
          float t[NV];
          Pack<T>::load_stream(rr + col, t);
#pragma unroll
          for (int e = 0; e < NV; ++e) v[p][e] += t[e];
        }
      }
    }
    if (h) {
      T* hr = h + row * C;
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) Pack<T>::store(hr + col, v[p]);
      }
    }
    float mean = 0.0f, scale;
    if (KIND == kLayerNorm) {
      float s = 0.0f;
#pragma unroll
      for (int p = 0; p < KP; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) s += v[p][e];
      mean = ag_warp_sum(s) * inv_c;
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) {
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            v[p][e] -= mean;
            q += v[p][e] * v[p][e];
          }
        }
      }
      scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
    } else {
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) q += v[p][e] * v[p][e];
      scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
    }
    if (lane == 0) {
      if (KIND == kLayerNorm) {
        if (stat0) stat0[row] = mean;
        if (stat1) stat1[row] = scale;
      } else if (stat0) {
        stat0[row] = scale;
      }
    }
    T* yr = y + row * C;
#pragma unroll
    for (int p = 0; p < KP; ++p) {
      const int col = (p * 32 + lane) * NV;
      if (col < C) {
        float o[NV];
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          float t = v[p][e] * scale;
          if (IN_REGS) {
            if (gamma) t = t * rg[p][e];
            if (KIND == kLayerNorm) t = t + rb[p][e];
          } else {
            if (gamma) t = t * s_gamma[col + e];
            if (KIND == kLayerNorm) t = t + s_beta[col + e];
          }
          o[e] = t;
        }
        Pack<T>::store_stream(yr + col, o);
      }
    }
  }
}

// CTA-per-row fallback for arbitrary C (scalar, row re-read from L1/L2 between passes).
template <typename T, int KIND>
__global__ void __launch_bounds__(NORM_THREADS)
norm_forward_generic_kernel(const T* x, const T* r, const float* __restrict__ gamma,
                            const float* __restrict__ beta, T* h, T* __restrict__ y,
                            float* __restrict__ stat0, float* __restrict__ stat1, int64_t N, int C, float eps) {
  __shared__ float s_red[NORM_WARPS];
  __shared__ float s_bcast;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto block_sum = [&](float v) -> float {
    v = ag_warp_sum(v);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int w = 0; w < NORM_WARPS; ++w) t += s_red[w];
      s_bcast = t;
    }
    __syncthreads();
    return s_bcast;
  };
  const float inv_c = 1.0f / (float)C;
  for (int64_t row = blockIdx.x; row < N; row += gridDim.x) {
    const T* xr = x + row * C;
    const T* rr = r ? r + row * C : nullptr;
    auto val = [&](int c) -> float {
      float t = Pack<T>::load1(xr + c);
      if (rr) t += Pack<T>::load1(rr + c);
      return t;
    };
    float mean = 0.0f, scale;
    if (KIND == kLayerNorm) {
      float s = 0.0f;
      for (int c = threadIdx.x; c < C; c += NORM_THREADS) s += val(c);
      mean = block_sum(s) * inv_c;
      float q = 0.0f;
      for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
        float d = val(c) - mean;
        q += d * d;
      }
      scale = 1.0f / sqrtf(block_sum(q) * inv_c + eps);
    } else {
      float q = 0.0f;
      for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
        float d = val(c);
        q += d * d;
      }
      scale = 1.0f / sqrtf(block_sum(q) * inv_c + eps);
    }
    if (threadIdx.x == 0) {
      if (KIND == kLayerNorm) {
        if (stat0) stat0[row] = mean;
        if (stat1) stat1[row] = scale;
      } else if (stat0) {
        stat0[row] = scale;
      }
    }
    for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
      const float hv = val(c);
      float t = (hv - mean) * scale;
      if (gamma) t = t * gamma[c];
      if (KIND == kLayerNorm) t = t + beta[c];
      if (h) Pack<T>::store1(h + row * C + c, hv);
      Pack<T>::store1(y + row * C + c, t);
    }
  }
}

// ---------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------
// partials layout: [gridDim.x][2][C] floats (slot 0: dgamma, slot 1: dbeta; RMSNorm leaves
// slot 1 unwritten and unread).
// Shared memory: gamma (C floats) + per-warp column accumulators [warp][slot][C].  The column
// sums live in shared memory rather than registers so that the registers can hold x, dy AND the
// incoming residual gradient of a row at once: all three are requested from HBM up front, in
// one burst per row, instead of a second dependent load phase after the row reductions.
template <int KIND>
__host__ __device__ constexpr int norm_bwd_slots() { return KIND == kLayerNorm ? 2 : 1; }

template <typename T, int KP, int KIND>
__global__ void __launch_bounds__(NORM_THREADS)
norm_backward_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                     const T* dres, T* dx, float* __restrict__ partials, int want_dgamma, int want_dbeta, int64_t N,
                     int C, float eps, uint32_t stage_poll_limit, int* status, int pdl_early) {
  ag_pdl_wait();
  if (pdl_early) ag_pdl_trigger();  // see norm_forward_kernel
  constexpr int NV = Pack<T>::N;
  constexpr int SLOTS = norm_bwd_slots<KIND>();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* s_gamma = reinterpret_cast<float*>(smem_raw);  // C floats
  float* s_acc = s_gamma + C;                           // NORM_WARPS * SLOTS * C floats
  __shared__ __align__(8) uint64_t s_bar;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const float inv_c = 1.0f / (float)C;
  constexpr bool IN_REGS = KP <= 4;  // as in forward
  float rg[IN_REGS ? KP : 1][NV];
  if (IN_REGS) {
#pragma unroll
    for (int p = 0; p < (IN_REGS ? KP : 1); ++p) {
      const int col = (p * 32 + lane) * NV;
#pragma unroll
      for (int e = 0; e < NV; ++e) rg[p][e] = (gamma && col < C) ? __ldg(gamma + col + e) : 1.0f;
    }
  } else if (gamma) {
    ag_stage_vectors(s_gamma, gamma, nullptr, nullptr, C, &s_bar, status, stage_poll_limit);
  }
  float* my_g = s_acc + (size_t)warp * SLOTS * C;
  float* my_b = my_g + C;  // LayerNorm only
  // each lane zeroes exactly the columns it will accumulate into: no cross-lane hazard
#pragma unroll
  for (int p = 0; p < KP; ++p) {
    const int col = (p * 32 + lane) * NV;
    if (col < C) {
#pragma unroll
      for (int e = 0; e < NV; ++e) {
        my_g[col + e] = 0.0f;
        if (KIND == kLayerNorm) my_b[col + e] = 0.0f;
      }
    }
  }

  for (int64_t row = (int64_t)blockIdx.x * NORM_WARPS + warp; row < N; row += (int64_t)gridDim.x * NORM_WARPS) {
    float v[KP][NV], g[KP][NV], o[KP][NV];
    const T* xr = x + row * C;
    const T* gr = dy + row * C;
    const T* drr = (dres && dx) ? dres + row * C : nullptr;
    {
      // the rows this warp will visit next are requested into L2 now, so that their loads meet a
      // short latency: with one resident CTA per SM at wide rows there are few warps to hide HBM
      const int64_t nxt = row + (int64_t)gridDim.x * NORM_WARPS;
      if (lane == 0 && nxt < N) {
        const uint32_t rb = (uint32_t)C * (uint32_t)sizeof(T);
        ag_prefetch_l2_bulk(x + nxt * C, rb);
        ag_prefetch_l2_bulk(dy + nxt * C, rb);
        if (drr) ag_prefetch_l2_bulk(dres + nxt * C, rb);
      }
    }
#pragma unroll
    for (int p = 0; p < KP; ++p) {
      const int col = (p * 32 + lane) * NV;
      if (col < C) {
        Pack<T>::load_stream(xr + col, v[p]);
        Pack<T>::load_stream(gr + col, g[p]);
      } else {
#pragma unroll
        for (int e = 0; e < NV; ++e) v[p][e] = g[p][e] = 0.0f;
      }
    }
#pragma unroll
    for (int p = 0; p < KP; ++p) {
      const int col = (p * 32 + lane) * NV;
      if (drr && col < C) {
        Pack<T>::load(drr + col, o[p]);
      } else {
#pragma unroll
        for (int e = 0; e < NV; ++e) o[p][e] = 0.0f;
      }
    }
    // statistics, recomputed from the saved input exactly as in forward
    float scale;
    if (KIND == kLayerNorm) {
      float s = 0.0f;
#pragma unroll
      for (int p = 0; p < KP; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) s += v[p][e];
      const float mean = ag_warp_sum(s) * inv_c;
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) {
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            v[p][e] -= mean;
            q += v[p][e] * v[p][e];
          }
        }
      }
      scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
    } else {
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) q += v[p][e] * v[p][e];
      scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
    }
    // v <- xhat ; column sums ; g <- dy*gamma ; row sums
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int p = 0; p < KP; ++p) {
      const int col = (p * 32 + lane) * NV;
      if (col < C) {
#pragma unroll
        for (int e4 = 0; e4 < NV; e4 += 4) {
          float4 ag = *reinterpret_cast<float4*>(my_g + col + e4);
          float4 ab = make_float4(0.f, 0.f, 0.f, 0.f);
          if (KIND == kLayerNorm) ab = *reinterpret_cast<float4*>(my_b + col + e4);
          float* agp = reinterpret_cast<float*>(&ag);
          float* abp = reinterpret_cast<float*>(&ab);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = e4 + j;
            const float xh = v[p][e] * scale;
            v[p][e] = xh;
            agp[j] += g[p][e] * xh;
            if (KIND == kLayerNorm) abp[j] += g[p][e];
            const float dg = gamma ? g[p][e] * (IN_REGS ? rg[p][e] : s_gamma[col + e]) : g[p][e];
            g[p][e] = dg;
            s1 += dg;
            s2 += dg * xh;
          }
          *reinterpret_cast<float4*>(my_g + col + e4) = ag;
          if (KIND == kLayerNorm) *reinterpret_cast<float4*>(my_b + col + e4) = ab;
        }
      }
    }
    float m1 = 0.0f;
    if (KIND == kLayerNorm) m1 = (ag_warp_sum(s1) * inv_c) * scale;
    const float m2 = (ag_warp_sum(s2) * inv_c) * scale;
    if (dx == nullptr) continue;  // only the column sums were asked for
    T* dxr = dx + row * C;
#pragma unroll
    for (int p = 0; p < KP; ++p) {
      const int col = (p * 32 + lane) * NV;
      if (col < C) {
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          // backend.py:475-487: xg += dyg*rstd; xg -= m1; xg -= xhat*m2
          float t = o[p][e] + g[p][e] * scale;
          if (KIND == kLayerNorm) t = t - m1;
          o[p][e] = t - v[p][e] * m2;
        }
        Pack<T>::store(dxr + col, o[p]);
      }
    }
  }

  // fold the warps' column accumulators in warp order
  __syncthreads();
  for (int slot = 0; slot < SLOTS; ++slot) {
    const bool wanted = slot == 0 ? (want_dgamma != 0) : (want_dbeta != 0);
    if (!wanted) continue;  // uniform across the CTA
    float* out = partials + ((int64_t)blockIdx.x * 2 + slot) * C;
    for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < NORM_WARPS; ++w) t += s_acc[((size_t)w * SLOTS + slot) * C + c];
      out[c] = t;
    }
  }
}

// ---------------------------------------------------------------------------------------
// backward, two warps per row
// ---------------------------------------------------------------------------------------
// Same arithmetic as norm_backward_kernel, but a row is shared by a pair of warps: each lane holds
// half as many packets of x, dy and the residual gradient, so the kernel needs about 100 registers
// instead of 170 and two CTAs fit an SM - twice the warps, each with half the dependent work per row.
// The three row reductions go through the pair: warp sums, two words of shared memory, a named
// barrier of 64 threads, and both warps add the two halves in the same order.  With wide rows the
// one-warp kernel is bound by its per-row dependency chains once the SM clock drops under the power
// cap (0.73 of the copy rate inside the benchmark step against 0.91 alone); this one is for those rows.
constexpr int PAIR_TEAMS = NORM_WARPS / 2;

// Sum of `v` over the 64 lanes of a warp pair.  `slot` alternates between consecutive calls, so a
// warp that runs one reduction ahead never overwrites words its partner is still reading.
__device__ __forceinline__ float pair_sum(float v, float* s_red, int team, int half, int lane, int slot) {
  v = ag_warp_sum(v);
  float* w = s_red + (team * 2 + slot) * 2;
  if (lane == 0) w[half] = v;
  asm volatile("bar.sync %0, 64;" ::"r"(team + 1) : "memory");
  return w[0] + w[1];
}

template <typename T, int KP2, int KIND>
__global__ void __launch_bounds__(NORM_THREADS, 2)
norm_backward_pair_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                          const T* dres, T* dx, float* __restrict__ partials, int want_dgamma, int want_dbeta,
                          int64_t N, int C, float eps, uint32_t stage_poll_limit, int* status, int pdl_early) {
  ag_pdl_wait();
  if (pdl_early) ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  constexpr int SLOTS = norm_bwd_slots<KIND>();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* s_gamma = reinterpret_cast<float*>(smem_raw);  // C floats
  float* s_acc = s_gamma + C;                           // PAIR_TEAMS * SLOTS * C floats: column sums per team
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ float s_red[PAIR_TEAMS * 2 * 2];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int team = warp >> 1, half = warp & 1;
  const int tl = half * 32 + lane;  // lane of the pair, 0..63
  const float inv_c = 1.0f / (float)C;
  if (gamma) ag_stage_vectors(s_gamma, gamma, nullptr, nullptr, C, &s_bar, status, stage_poll_limit);
  float* my_g = s_acc + (size_t)team * SLOTS * C;
  float* my_b = my_g + C;  // LayerNorm only
  // each lane zeroes exactly the columns it will accumulate into: no cross-lane hazard
#pragma unroll
  for (int p = 0; p < KP2; ++p) {
    const int col = (p * 64 + tl) * NV;
    if (col < C) {
#pragma unroll
      for (int e = 0; e < NV; ++e) {
        my_g[col + e] = 0.0f;
        if (KIND == kLayerNorm) my_b[col + e] = 0.0f;
      }
    }
  }
  int red = 0;  // parity of the next pair reduction
  // bf16 storage: a row's packets are 4 registers per 8 elements, so the x and dy packets of the row
  // the pair visits NEXT are requested before the current row is computed and wait in registers;
  // the row's latency then overlaps the arithmetic of its predecessor.  (fp32 rows would need twice
  // the registers and lose the second CTA of an SM.)
  constexpr bool AHEAD = NV == 8;
  using Raw = typename Pack<T>::Raw;
  Raw nx[AHEAD ? KP2 : 1], ng[AHEAD ? KP2 : 1];
  const int64_t row_step = (int64_t)gridDim.x * PAIR_TEAMS;
  const int64_t row0 = (int64_t)blockIdx.x * PAIR_TEAMS + team;
  if constexpr (AHEAD) {
    if (row0 < N) {
#pragma unroll
      for (int p = 0; p < KP2; ++p) {
        const int col = (p * 64 + tl) * NV;
        if (col < C) {
          nx[p] = Pack<T>::load_raw_stream(x + row0 * C + col);
          ng[p] = Pack<T>::load_raw_stream(dy + row0 * C + col);
        }
      }
    }
  }
  for (int64_t row = row0; row < N; row += row_step) {
    float v[KP2][NV], g[KP2][NV], o[KP2][NV];
    const T* xr = x + row * C;
    const T* gr = dy + row * C;
    const T* drr = (dres && dx) ? dres + row * C : nullptr;
    // (no L2 prefetch of the pair's next row here: with 16 warps per SM it only added requests - 112.4 -> 107.6 us
    // at 32768 x 1280, 39.9 -> 37.8 us at 8192 x 1536 without it; the one-warp kernel above keeps it)
    if constexpr (AHEAD) {
#pragma unroll
      for (int p = 0; p < KP2; ++p) {
        const int col = (p * 64 + tl) * NV;
        if (col < C) {
          Pack<T>::unpack_raw(nx[p], v[p]);
          Pack<T>::unpack_raw(ng[p], g[p]);
        } else {
#pragma unroll
          for (int e = 0; e < NV; ++e) v[p][e] = g[p][e] = 0.0f;
        }
      }
      const int64_t nxt = row + row_step;
      if (nxt < N) {
#pragma unroll
        for (int p = 0; p < KP2; ++p) {
          const int col = (p * 64 + tl) * NV;
          if (col < C) {
            nx[p] = Pack<T>::load_raw_stream(x + nxt * C + col);
            ng[p] = Pack<T>::load_raw_stream(dy + nxt * C + col);
          }
        }
      }
    } else {
#pragma unroll
      for (int p = 0; p < KP2; ++p) {
        const int col = (p * 64 + tl) * NV;
        if (col < C) {
          Pack<T>::load_stream(xr + col, v[p]);
          Pack<T>::load_stream(gr + col, g[p]);
        } else {
#pragma unroll
          for (int e = 0; e < NV; ++e) v[p][e] = g[p][e] = 0.0f;
        }
      }
    }
#pragma unroll
    for (int p = 0; p < KP2; ++p) {
      const int col = (p * 64 + tl) * NV;
      if (drr && col < C) {
        Pack<T>::load(drr + col, o[p]);
      } else {
#pragma unroll
        for (int e = 0; e < NV; ++e) o[p][e] = 0.0f;
      }
    }
    // statistics, recomputed from the saved input exactly as in forward
    float scale;
    if (KIND == kLayerNorm) {
      float s = 0.0f;
#pragma unroll
      for (int p = 0; p < KP2; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) s += v[p][e];
      const float mean = pair_sum(s, s_red, team, half, lane, red) * inv_c;
      red ^= 1;
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP2; ++p) {
        const int col = (p * 64 + tl) * NV;
        if (col < C) {
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            v[p][e] -= mean;
            q += v[p][e] * v[p][e];
          }
        }
      }
      scale = 1.0f / sqrtf(pair_sum(q, s_red, team, half, lane, red) * inv_c + eps);
      red ^= 1;
    } else {
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP2; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) q += v[p][e] * v[p][e];
      scale = 1.0f / sqrtf(pair_sum(q, s_red, team, half, lane, red) * inv_c + eps);
      red ^= 1;
    }
    // v <- xhat ; column sums ; g <- dy*gamma ; row sums
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int p = 0; p < KP2; ++p) {
      const int col = (p * 64 + tl) * NV;
      if (col < C) {
#pragma unroll
        for (int e4 = 0; e4 < NV; e4 += 4) {
          float4 ag = *reinterpret_cast<float4*>(my_g + col + e4);
          float4 ab = make_float4(0.f, 0.f, 0.f, 0.f);
          if (KIND == kLayerNorm) ab = *reinterpret_cast<float4*>(my_b + col + e4);
          float4 gg = make_float4(1.f, 1.f, 1.f, 1.f);
          if (gamma) gg = *reinterpret_cast<const float4*>(s_gamma + col + e4);
          float* agp = reinterpret_cast<float*>(&ag);
          float* abp = reinterpret_cast<float*>(&ab);
          const float* gp = reinterpret_cast<const float*>(&gg);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e = e4 + j;
            const float xh = v[p][e] * scale;
            v[p][e] = xh;
            agp[j] += g[p][e] * xh;
            if (KIND == kLayerNorm) abp[j] += g[p][e];
            const float dg = gamma ? g[p][e] * gp[j] : g[p][e];
            g[p][e] = dg;
            s1 += dg;
            s2 += dg * xh;
          }
          *reinterpret_cast<float4*>(my_g + col + e4) = ag;
          if (KIND == kLayerNorm) *reinterpret_cast<float4*>(my_b + col + e4) = ab;
        }
      }
    }
    float m1 = 0.0f;
    if (KIND == kLayerNorm) {
      m1 = (pair_sum(s1, s_red, team, half, lane, red) * inv_c) * scale;
      red ^= 1;
    }
    const float m2 = (pair_sum(s2, s_red, team, half, lane, red) * inv_c) * scale;
    red ^= 1;
    if (dx == nullptr) continue;  // only the column sums were asked for
    T* dxr = dx + row * C;
#pragma unroll
    for (int p = 0; p < KP2; ++p) {
      const int col = (p * 64 + tl) * NV;
      if (col < C) {
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          // backend.py:475-487: xg += dyg*rstd; xg -= m1; xg -= xhat*m2
          float t = o[p][e] + g[p][e] * scale;
          if (KIND == kLayerNorm) t = t - m1;
          o[p][e] = t - v[p][e] * m2;
        }
        Pack<T>::store(dxr + col, o[p]);
      }
    }
  }

  // fold the teams' column sums in team order
  __syncthreads();
  for (int slot = 0; slot < SLOTS; ++slot) {
    const bool wanted = slot == 0 ? (want_dgamma != 0) : (want_dbeta != 0);
    if (!wanted) continue;  // uniform across the CTA
    float* out = partials + ((int64_t)blockIdx.x * 2 + slot) * C;
    for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < PAIR_TEAMS; ++w) t += s_acc[((size_t)w * SLOTS + slot) * C + c];
      out[c] = t;
    }
  }
}

// ---------------------------------------------------------------------------------------
// forward, two warps per row
// ---------------------------------------------------------------------------------------
// norm_forward_kernel with a row shared by a pair of warps (see norm_backward_pair_kernel): half the
// registers per lane, so more CTAs per SM and half the dependent work per row and warp.
template <typename T, int KP2, int KIND>
__global__ void __launch_bounds__(NORM_THREADS)
norm_forward_pair_kernel(const T* x, const T* r, const float* __restrict__ gamma, const float* __restrict__ beta, T* h,
                         T* __restrict__ y, float* __restrict__ stat0, float* __restrict__ stat1, int64_t N, int C,
                         float eps, uint32_t stage_poll_limit, int* status, int pdl_early) {
  ag_pdl_wait();
  if (pdl_early) ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* s_gamma = reinterpret_cast<float*>(smem_raw);
  float* s_beta = s_gamma + C;
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ float s_red[PAIR_TEAMS * 2 * 2];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int team = warp >> 1, half = warp & 1;
  const int tl = half * 32 + lane;
  const float inv_c = 1.0f / (float)C;
  if (gamma)
    ag_stage_vectors(s_gamma, gamma, s_beta, (KIND == kLayerNorm) ? beta : nullptr, C, &s_bar, status, stage_poll_limit);
  int red = 0;
  for (int64_t row = (int64_t)blockIdx.x * PAIR_TEAMS + team; row < N; row += (int64_t)gridDim.x * PAIR_TEAMS) {
    float v[KP2][NV];
    const T* xr = x + row * C;
#pragma unroll
    for (int p = 0; p < KP2; ++p) {
      const int col = (p * 64 + tl) * NV;
      if (col < C) {
        Pack<T>::load_stream(xr + col, v[p]);
      } else {
#pragma unroll
        for (int e = 0; e < NV; ++e) v[p][e] = 0.0f;
      }
    }
    if (r) {
      const T* rr = r + row * C;
#pragma unroll
      for (int p = 0; p < KP2; ++p) {
        const int col = (p * 64 + tl) * NV;
        if (col < C) {
          float t[NV];
          Pack<T>::load_stream(rr + col, t);
#pragma unroll
          for (int e = 0; e < NV; ++e) v[p][e] += t[e];
        }
      }
    }
    if (h) {
      T* hr = h + row * C;
#pragma unroll
      for (int p = 0; p < KP2; ++p) {
        const int col = (p * 64 + tl) * NV;
        if (col < C) Pack<T>::store(hr + col, v[p]);
      }
    }
    float mean = 0.0f, scale;
    if (KIND == kLayerNorm) {
      float s = 0.0f;
#pragma unroll
      for (int p = 0; p < KP2; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) s += v[p][e];
      mean = pair_sum(s, s_red, team, half, lane, red) * inv_c;
      red ^= 1;
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP2; ++p) {
        const int col = (p * 64 + tl) * NV;
        if (col < C) {
#pragma unroll
          for (int e = 0; e < NV; ++e) {
            v[p][e] -= mean;
            q += v[p][e] * v[p][e];
          }
        }
      }
      scale = 1.0f / sqrtf(pair_sum(q, s_red, team, half, lane, red) * inv_c + eps);
      red ^= 1;
    } else {
      float q = 0.0f;
#pragma unroll
      for (int p = 0; p < KP2; ++p)
#pragma unroll
        for (int e = 0; e < NV; ++e) q += v[p][e] * v[p][e];
      scale = 1.0f / sqrtf(pair_sum(q, s_red, team, half, lane, red) * inv_c + eps);
      red ^= 1;
    }
    if (tl == 0) {
      if (KIND == kLayerNorm) {
        if (stat0) stat0[row] = mean;
        if (stat1) stat1[row] = scale;
      } else if (stat0) {
        stat0[row] = scale;
      }
    }
    T* yr = y + row * C;
#pragma unroll
    for (int p = 0; p < KP2; ++p) {
      const int col = (p * 64 + tl) * NV;
      if (col < C) {
        float o[NV];
#pragma unroll
        for (int e4 = 0; e4 < NV; e4 += 4) {
          float4 gg = make_float4(1.f, 1.f, 1.f, 1.f), bb = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gamma) gg = *reinterpret_cast<const float4*>(s_gamma + col + e4);
          if (KIND == kLayerNorm) bb = *reinterpret_cast<const float4*>(s_beta + col + e4);
          const float* gp = reinterpret_cast<const float*>(&gg);
          const float* bp = reinterpret_cast<const float*>(&bb);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float t = v[p][e4 + k] * scale;
            if (gamma) t = t * gp[k];
            if (KIND == kLayerNorm) t = t + bp[k];
            o[e4 + k] = t;
          }
        }
        Pack<T>::store_stream(yr + col, o);
      }
    }
  }
}

// CTA-per-row fallback: per-thread column accumulators for columns c = tid + k*THREADS are
// kept in shared memory rows (one per CTA), rows visited grid-stride.
template <typename T, int KIND>
__global__ void __launch_bounds__(NORM_THREADS)
norm_backward_generic_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                             const T* dres, T* dx, float* __restrict__ partials, int want_dgamma, int want_dbeta,
                             int64_t N, int C, float eps) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* s_g = reinterpret_cast<float*>(smem_raw);  // C floats: dgamma accumulators
  float* s_b = s_g + C;                             // C floats: dbeta accumulators
  __shared__ float s_red[NORM_WARPS];
  __shared__ float s_bcast;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  auto block_sum = [&](float v) -> float {
    v = ag_warp_sum(v);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int w = 0; w < NORM_WARPS; ++w) t += s_red[w];
      s_bcast = t;
    }
    __syncthreads();
    return s_bcast;
  };
  for (int c = threadIdx.x; c < C; c += NORM_THREADS) s_g[c] = s_b[c] = 0.0f;
  const float inv_c = 1.0f / (float)C;
  for (int64_t row = blockIdx.x; row < N; row += gridDim.x) {
    const T* xr = x + row * C;
    const T* gr = dy + row * C;
    float mean = 0.0f, scale;
    if (KIND == kLayerNorm) {
      float s = 0.0f;
      for (int c = threadIdx.x; c < C; c += NORM_THREADS) s += Pack<T>::load1(xr + c);
      mean = block_sum(s) * inv_c;
      float q = 0.0f;
      for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
        float d = Pack<T>::load1(xr + c) - mean;
        q += d * d;
      }
      scale = 1.0f / sqrtf(block_sum(q) * inv_c + eps);
    } else {
      float q = 0.0f;
      for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
        float d = Pack<T>::load1(xr + c);
        q += d * d;
      }
      scale = 1.0f / sqrtf(block_sum(q) * inv_c + eps);
    }
    float s1 = 0.0f, s2 = 0.0f;
    for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
      const float xh = (Pack<T>::load1(xr + c) - mean) * scale;
      const float g = Pack<T>::load1(gr + c);
      s_g[c] += g * xh;  // column c is always visited by the same thread
      if (KIND == kLayerNorm) s_b[c] += g;
      const float dg = gamma ? g * gamma[c] : g;
      s1 += dg;
      s2 += dg * xh;
    }
    float m1 = 0.0f;
    if (KIND == kLayerNorm) m1 = (block_sum(s1) * inv_c) * scale;
    const float m2 = (block_sum(s2) * inv_c) * scale;
    for (int c = threadIdx.x; dx != nullptr && c < C; c += NORM_THREADS) {
      const float xh = (Pack<T>::load1(xr + c) - mean) * scale;
      const float g = Pack<T>::load1(gr + c);
      const float dg = gamma ? g * gamma[c] : g;
      float t = (dres ? Pack<T>::load1(dres + row * C + c) : 0.0f) + dg * scale;
      if (KIND == kLayerNorm) t = t - m1;
      Pack<T>::store1(dx + row * C + c, t - xh * m2);
    }
  }
  for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
    if (want_dgamma) partials[((int64_t)blockIdx.x * 2 + 0) * C + c] = s_g[c];
    if (KIND == kLayerNorm && want_dbeta) partials[((int64_t)blockIdx.x * 2 + 1) * C + c] = s_b[c];
  }
}

// Second pass: dgamma[c] += sum_p partials[p][0][c], dbeta[c] += sum_p partials[p][1][c].
// Block = 32 columns x 32 partial-row groups; group y adds rows y, y+32, ... in order, the
// 32 group sums are then added in group order.  Fixed order, no atomics.
__global__ void __launch_bounds__(1024)
norm_partials_reduce_kernel(const float* __restrict__ partials, int P, int C, float* dgamma, float* dbeta) {
  ag_pdl_wait();
  ag_pdl_trigger();
  __shared__ float s[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int slot = blockIdx.y;
  float* out = slot == 0 ? dgamma : dbeta;
  if (!out) return;  // uniform per block
  float t = 0.0f;
  float prev = 0.0f;
  if (c < C) {
    // the accumulator's old value travels with the partial rows instead of after them
    if (threadIdx.y == 0) prev = out[c];
    // sixteen loads in flight per thread (one round for up to 512 partial rows), added in row order;
    // rows past the end contribute +0, which leaves the sum's bits as they are
    for (int p = threadIdx.y; p < P; p += 16 * 32) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int q = p + j * 32;
        v[j] = q < P ? partials[((int64_t)q * 2 + slot) * C + c] : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) t += v[j];
    }
  }
  s[threadIdx.y][threadIdx.x] = t;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    float tot = 0.0f;
#pragma unroll
    for (int y = 0; y < 32; ++y) tot += s[y][threadIdx.x];
    out[c] = prev + tot;
  }
}

// ---------------------------------------------------------------------------------------
// Row ring: rows travel HBM -> shared memory through the bulk-copy (TMA) engine
// ---------------------------------------------------------------------------------------
// The kernels above hold a row in registers from the moment its loads are issued, so the bytes a
// warp has in flight and the bytes it computes on compete for the same registers, and with wide
// rows only one CTA fits an SM.  Here the rows in flight live in shared memory instead: one
// producer lane per CTA issues a 1-D bulk copy per operand row into a ring of R slots
// (mbarrier complete_tx), the consumer warps (eight, fewer for wide rows) take the rows in turn,
// two slots each, and a slot goes back to the producer (a second mbarrier) as soon as its row has
// been read.  Registers then hold only
// the row being computed and the dgamma/dbeta column sums.  Every CTA owns whole rows: CTA b
// takes rows b, b + grid, b + 2*grid, ...; local row j sits in slot j % R.
//
// Every wait is bounded.  When one runs out the CTA sets AG_STATUS_WAIT_EXPIRED, all roles leave
// their loops, the producer gives the copies it has issued a last bounded wait to land, and the
// kernel returns.
constexpr int RING_MAX_CONSUMERS = 8;                        // consumer warps per CTA (fewer for wide rows)
constexpr int RING_MAX_THREADS = (RING_MAX_CONSUMERS + 1) * 32;  // + the producer warp
constexpr int RING_MAX_SLOTS = 16;                           // two slots per consumer warp
constexpr uint32_t RING_POLL_LIMIT = 1u << 18;  // polls with back-off: tens of milliseconds
constexpr int RING_MAX_PER_LANE = 48;  // row elements per lane (C <= 1536)

struct __align__(16) RingHeader {
  uint64_t full[RING_MAX_SLOTS];   // producer -> consumer: the slot's bytes have landed
  uint64_t empty[RING_MAX_SLOTS];  // consumer -> producer: the slot's row has been read
  uint64_t stage_bar;              // gamma/beta staging
  int abort;                       // a wait expired somewhere in this CTA
  int issued;                      // rows the producer has issued so far
};
constexpr size_t kRingHeaderBytes = (sizeof(RingHeader) + 127) / 128 * 128;

struct RingPlan {
  int slots;            // R = 2 * consumers
  int consumers;        // consumer warps; the CTA has one more warp, the producer
  uint32_t row_bytes;   // bytes of one operand row
  uint32_t slot_bytes;  // operand rows per slot * row_bytes
  size_t vec_bytes;     // staged fp32 vectors (gamma, beta)
  size_t ring_bytes;    // ring, also reused for the final fold of the column sums
  size_t smem;          // total dynamic shared memory
};

// Two slots per consumer warp: while a warp computes on one row its next row is in flight.  A slot
// is always consumed by the same warp (slot s belongs to warp s % consumers), see ring_wait_full.
// Narrow rows: 8 consumer warps, 16 slots, small enough that several CTAs share an SM.  Wide rows:
// one CTA per SM and as many consumer warps (at most 8) as 200 KB of slots allow.
inline RingPlan ring_plan(int C, size_t elem_bytes, int rows_per_slot, int n_vectors, int fold_slots) {
  RingPlan p;
  p.row_bytes = (uint32_t)((size_t)C * elem_bytes);
  p.slot_bytes = p.row_bytes * (uint32_t)rows_per_slot;
  p.vec_bytes = ((size_t)n_vectors * C * sizeof(float) + 127) / 128 * 128;
  int cw = RING_MAX_CONSUMERS;
  if (p.slot_bytes >= 8192) {
    const size_t fit = ((size_t)200 * 1024) / ((size_t)2 * p.slot_bytes);
    if (fit < (size_t)cw) cw = (int)fit;
  }
  if (cw < 3) cw = 0;  // too wide for this scheme: the caller falls back
  const int r = 2 * cw;
  p.consumers = cw;
  const size_t fold_bytes = (size_t)cw * fold_slots * C * sizeof(float);
  p.slots = r;
  p.ring_bytes = (size_t)r * p.slot_bytes;
  if (p.ring_bytes < fold_bytes) p.ring_bytes = fold_bytes;
  p.ring_bytes = (p.ring_bytes + 127) / 128 * 128;
  p.smem = kRingHeaderBytes + p.vec_bytes + p.ring_bytes;
  return p;
}

__device__ __forceinline__ void ring_init(RingHeader* hd, int R) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < R; ++s) {
      ag_mbar_init(&hd->full[s], 1);
      ag_mbar_init(&hd->empty[s], 1);
    }
    hd->abort = 0;
    hd->issued = 0;
    ag_fence_mbar_init();
  }
  __syncthreads();
}

// Producer lane: issues the operand rows of local rows j_begin .. j_end-1 in order.  Rows of the
// first round (j < R) find their slot empty; later ones wait for the consumer of row j - R.
__device__ __forceinline__ void ring_produce(RingHeader* hd, unsigned char* ring, int R, uint32_t slot_bytes,
                                             uint32_t row_bytes, const unsigned char* src0, const unsigned char* src1,
                                             const unsigned char* src2, int64_t first_row, int64_t row_stride,
                                             uint32_t j_begin, uint32_t j_end, int* status) {
  volatile int* abort_flag = &hd->abort;
  volatile int* issued = &hd->issued;
  const uint32_t nsrc = 1u + (src1 ? 1u : 0u) + (src2 ? 1u : 0u);
  uint32_t slot = j_begin % (uint32_t)R;
  uint32_t round = j_begin / (uint32_t)R;
  for (uint32_t j = j_begin; j < j_end; ++j) {
    if (round > 0 && !ag_mbar_wait_bounded(&hd->empty[slot], (round - 1) & 1u, RING_POLL_LIMIT)) {
      atomicOr(status, AG_STATUS_WAIT_EXPIRED);
      *abort_flag = 1;
      break;
    }
    if (*abort_flag) break;
    const int64_t off = (first_row + (int64_t)j * row_stride) * (int64_t)row_bytes;
    unsigned char* dst = ring + (size_t)slot * slot_bytes;
    ag_mbar_expect_tx(&hd->full[slot], row_bytes * nsrc);
    ag_bulk_g2s(dst, src0 + off, row_bytes, &hd->full[slot]);
    if (src1) ag_bulk_g2s(dst + row_bytes, src1 + off, row_bytes, &hd->full[slot]);
    if (src2) ag_bulk_g2s(dst + (src1 ? 2u : 1u) * row_bytes, src2 + off, row_bytes, &hd->full[slot]);
    *issued = (int)(j + 1);
    if (++slot == (uint32_t)R) {
      slot = 0;
      ++round;
    }
  }
}

// Consumer side of a slot: every lane polls, the warp takes one decision.
// A parity wait can only tell the current phase of a barrier from the one just before it, so a slot
// must always be consumed by the same warp, which then meets its phases strictly in order: the ring
// has two slots per consumer warp and rows go to the warps round-robin.
__device__ __forceinline__ bool ring_wait_full(RingHeader* hd, uint32_t slot, uint32_t round) {
  const bool ok = ag_mbar_wait_bounded(&hd->full[slot], round & 1u, RING_POLL_LIMIT);
  return __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
}

// After an abort: the latest copy issued into each slot is given a bounded wait, so that no copy
// is still writing this CTA's shared memory when it exits.  Producer lane only.
__device__ __forceinline__ void ring_drain(RingHeader* hd, int R, int* status) {
  const uint32_t issued = (uint32_t) * (volatile int*)&hd->issued;
  const uint32_t first = issued > (uint32_t)R ? issued - (uint32_t)R : 0u;
  for (uint32_t j = first; j < issued; ++j) {
    const uint32_t slot = j % (uint32_t)R;
    const uint32_t par = (j / (uint32_t)R) & 1u;
    if (!ag_mbar_wait_bounded(&hd->full[slot], par, RING_POLL_LIMIT)) atomicOr(status, AG_STATUS_WAIT_EXPIRED);
  }
}

// ---- forward --------------------------------------------------------------------------
template <typename T, int KP, int KIND>
__global__ void __launch_bounds__(RING_MAX_THREADS, 1)
norm_forward_ring_kernel(const T* x, const T* r, const float* __restrict__ gamma, const float* __restrict__ beta, T* h,
                         T* __restrict__ y, float* __restrict__ stat0, float* __restrict__ stat1, int64_t N, int C,
                         float eps, int R, int CW, uint32_t slot_bytes, uint32_t stage_poll_limit, int* status, int pdl_early) {
  ag_pdl_wait();
  if (pdl_early) ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  RingHeader* hd = reinterpret_cast<RingHeader*>(smem_raw);
  float* s_gamma = reinterpret_cast<float*>(smem_raw + kRingHeaderBytes);
  float* s_beta = s_gamma + C;
  const size_t vec_bytes = ((size_t)(KIND == kLayerNorm ? 2 : 1) * C * sizeof(float) + 127) / 128 * 128;
  unsigned char* ring = smem_raw + kRingHeaderBytes + vec_bytes;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t row_bytes = (uint32_t)C * (uint32_t)sizeof(T);
  const float inv_c = 1.0f / (float)C;

  ring_init(hd, R);
  const int64_t first_row = blockIdx.x;
  const uint32_t n_local = first_row < N ? (uint32_t)((N - first_row + gridDim.x - 1) / gridDim.x) : 0u;
  const uint32_t n_first = n_local < (uint32_t)R ? n_local : (uint32_t)R;
  const unsigned char* gx = reinterpret_cast<const unsigned char*>(x);
  const unsigned char* gr = reinterpret_cast<const unsigned char*>(r);
  // the first rows are requested before gamma/beta are staged, so both transfers overlap
  if (warp == CW) {
    if (lane == 0)
      ring_produce(hd, ring, R, slot_bytes, row_bytes, gx, gr, nullptr, first_row, gridDim.x, 0u, n_first, status);
    __syncwarp();
  }
  if (gamma)
    ag_stage_vectors(s_gamma, gamma, s_beta, (KIND == kLayerNorm) ? beta : nullptr, C, &hd->stage_bar, status,
                     stage_poll_limit);
  volatile int* abort_flag = &hd->abort;

  if (warp == CW) {
    if (lane == 0)
      ring_produce(hd, ring, R, slot_bytes, row_bytes, gx, gr, nullptr, first_row, gridDim.x, n_first, n_local, status);
    __syncwarp();
  } else {
    for (uint32_t j = (uint32_t)warp; j < n_local; j += (uint32_t)CW) {
      if (__any_sync(0xffffffffu, *abort_flag)) break;
      const uint32_t slot = j % (uint32_t)R;
      if (!ring_wait_full(hd, slot, j / (uint32_t)R)) {
        if (lane == 0) atomicOr(status, AG_STATUS_WAIT_EXPIRED);
        *abort_flag = 1;
        break;
      }
      const T* sx = reinterpret_cast<const T*>(ring + (size_t)slot * slot_bytes);
      const T* sr = sx + C;
      float v[KP][NV];
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) {
          Pack<T>::load(sx + col, v[p]);
          if (r) {
            float t[NV];
            Pack<T>::load(sr + col, t);
#pragma unroll
            for (int e = 0; e < NV; ++e) v[p][e] += t[e];
          }
        } else {
#pragma unroll
          for (int e = 0; e < NV; ++e) v[p][e] = 0.0f;
        }
      }
      // the row is in registers: the slot can take the next row already
      __syncwarp();
      if (lane == 0) ag_mbar_arrive(&hd->empty[slot]);
      const int64_t row = first_row + j * (int64_t)gridDim.x;
      if (h) {
        T* hr = h + row * C;
#pragma unroll
        for (int p = 0; p < KP; ++p) {
          const int col = (p * 32 + lane) * NV;
          if (col < C) Pack<T>::store(hr + col, v[p]);
        }
      }
      float mean = 0.0f, scale;
      if (KIND == kLayerNorm) {
        float s = 0.0f;
#pragma unroll
        for (int p = 0; p < KP; ++p)
#pragma unroll
          for (int e = 0; e < NV; ++e) s += v[p][e];
        mean = ag_warp_sum(s) * inv_c;
        float q = 0.0f;
#pragma unroll
        for (int p = 0; p < KP; ++p) {
          const int col = (p * 32 + lane) * NV;
          if (col < C) {
#pragma unroll
            for (int e = 0; e < NV; ++e) {
              v[p][e] -= mean;
              q += v[p][e] * v[p][e];
            }
          }
        }
        scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
      } else {
        float q = 0.0f;
#pragma unroll
        for (int p = 0; p < KP; ++p)
#pragma unroll
          for (int e = 0; e < NV; ++e) q += v[p][e] * v[p][e];
        scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
      }
      if (lane == 0) {
        if (KIND == kLayerNorm) {
          if (stat0) stat0[row] = mean;
          if (stat1) stat1[row] = scale;
        } else if (stat0) {
          stat0[row] = scale;
        }
      }
      T* yr = y + row * C;
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) {
          float o[NV];
#pragma unroll
          for (int e4 = 0; e4 < NV; e4 += 4) {
            float4 gg = make_float4(1.f, 1.f, 1.f, 1.f), bb = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gamma) gg = *reinterpret_cast<const float4*>(s_gamma + col + e4);
            if (KIND == kLayerNorm) bb = *reinterpret_cast<const float4*>(s_beta + col + e4);
            const float* gp = reinterpret_cast<const float*>(&gg);
            const float* bp = reinterpret_cast<const float*>(&bb);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              float t = v[p][e4 + k] * scale;
              if (gamma) t = t * gp[k];
              if (KIND == kLayerNorm) t = t + bp[k];
              o[e4 + k] = t;
            }
          }
          Pack<T>::store_stream(yr + col, o);
        }
      }
    }
  }
  __syncthreads();
  if (*abort_flag && warp == CW && lane == 0) ring_drain(hd, R, status);
}

// ---- backward -------------------------------------------------------------------------
// Slot: [x row | dy row | dres row (when a residual gradient is added)].  The column sums live in
// registers (C/32 values per lane and sum), x-hat of the current row too; dy is read from the slot
// twice (column/row sums, then dx) rather than kept.
template <typename T, int KP, int KIND>
__global__ void __launch_bounds__(RING_MAX_THREADS, 1)
norm_backward_ring_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                          const T* dres, T* dx, float* __restrict__ partials, int want_dgamma, int want_dbeta,
                          int64_t N, int C, float eps, int R, int CW, uint32_t slot_bytes,
                          uint32_t stage_poll_limit, int* status, int pdl_early) {
  ag_pdl_wait();
  if (pdl_early) ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  constexpr int SLOTS = norm_bwd_slots<KIND>();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  RingHeader* hd = reinterpret_cast<RingHeader*>(smem_raw);
  float* s_gamma = reinterpret_cast<float*>(smem_raw + kRingHeaderBytes);
  const size_t vec_bytes = ((size_t)C * sizeof(float) + 127) / 128 * 128;
  unsigned char* ring = smem_raw + kRingHeaderBytes + vec_bytes;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t row_bytes = (uint32_t)C * (uint32_t)sizeof(T);
  const float inv_c = 1.0f / (float)C;
  const bool with_res = dres != nullptr && dx != nullptr;

  ring_init(hd, R);
  const int64_t first_row = blockIdx.x;
  const uint32_t n_local = first_row < N ? (uint32_t)((N - first_row + gridDim.x - 1) / gridDim.x) : 0u;
  const uint32_t n_first = n_local < (uint32_t)R ? n_local : (uint32_t)R;
  const unsigned char* gx = reinterpret_cast<const unsigned char*>(x);
  const unsigned char* gdy = reinterpret_cast<const unsigned char*>(dy);
  const unsigned char* gres = with_res ? reinterpret_cast<const unsigned char*>(dres) : nullptr;
  if (warp == CW) {
    if (lane == 0)
      ring_produce(hd, ring, R, slot_bytes, row_bytes, gx, gdy, gres, first_row, gridDim.x, 0u, n_first, status);
    __syncwarp();
  }
  if (gamma) ag_stage_vectors(s_gamma, gamma, nullptr, nullptr, C, &hd->stage_bar, status, stage_poll_limit);
  volatile int* abort_flag = &hd->abort;

  float acc_g[KP][NV], acc_b[KIND == kLayerNorm ? KP : 1][NV];
#pragma unroll
  for (int p = 0; p < KP; ++p)
#pragma unroll
    for (int e = 0; e < NV; ++e) {
      acc_g[p][e] = 0.0f;
      if constexpr (KIND == kLayerNorm) acc_b[p][e] = 0.0f;
    }

  if (warp == CW) {
    if (lane == 0)
      ring_produce(hd, ring, R, slot_bytes, row_bytes, gx, gdy, gres, first_row, gridDim.x, n_first, n_local, status);
    __syncwarp();
  } else {
    for (uint32_t j = (uint32_t)warp; j < n_local; j += (uint32_t)CW) {
      if (__any_sync(0xffffffffu, *abort_flag)) break;
      const uint32_t slot = j % (uint32_t)R;
      if (!ring_wait_full(hd, slot, j / (uint32_t)R)) {
        if (lane == 0) atomicOr(status, AG_STATUS_WAIT_EXPIRED);
        *abort_flag = 1;
        break;
      }
      const T* sx = reinterpret_cast<const T*>(ring + (size_t)slot * slot_bytes);
      const T* sdy = sx + C;
      const T* sres = sdy + C;
      float v[KP][NV];
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) {
          Pack<T>::load(sx + col, v[p]);
        } else {
#pragma unroll
          for (int e = 0; e < NV; ++e) v[p][e] = 0.0f;
        }
      }
      // statistics, recomputed from the saved input exactly as in forward
      float scale;
      if (KIND == kLayerNorm) {
        float s = 0.0f;
#pragma unroll
        for (int p = 0; p < KP; ++p)
#pragma unroll
          for (int e = 0; e < NV; ++e) s += v[p][e];
        const float mean = ag_warp_sum(s) * inv_c;
        float q = 0.0f;
#pragma unroll
        for (int p = 0; p < KP; ++p) {
          const int col = (p * 32 + lane) * NV;
          if (col < C) {
#pragma unroll
            for (int e = 0; e < NV; ++e) {
              v[p][e] -= mean;
              q += v[p][e] * v[p][e];
            }
          }
        }
        scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
      } else {
        float q = 0.0f;
#pragma unroll
        for (int p = 0; p < KP; ++p)
#pragma unroll
          for (int e = 0; e < NV; ++e) q += v[p][e] * v[p][e];
        scale = 1.0f / sqrtf(ag_warp_sum(q) * inv_c + eps);
      }
      // v <- xhat ; column sums ; row sums of dy*gamma and dy*gamma*xhat
      float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
      for (int p = 0; p < KP; ++p) {
        const int col = (p * 32 + lane) * NV;
        if (col < C) {
          float g[NV];
          Pack<T>::load(sdy + col, g);
#pragma unroll
          for (int e4 = 0; e4 < NV; e4 += 4) {
            float4 gg = make_float4(1.f, 1.f, 1.f, 1.f);
            if (gamma) gg = *reinterpret_cast<const float4*>(s_gamma + col + e4);
            const float* gp = reinterpret_cast<const float*>(&gg);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int e = e4 + k;
              const float xh = v[p][e] * scale;
              v[p][e] = xh;
              acc_g[p][e] += g[e] * xh;
              if constexpr (KIND == kLayerNorm) acc_b[p][e] += g[e];
              const float dg = gamma ? g[e] * gp[k] : g[e];
              s1 += dg;
              s2 += dg * xh;
            }
          }
        }
      }
      float m1 = 0.0f;
      if (KIND == kLayerNorm) m1 = (ag_warp_sum(s1) * inv_c) * scale;
      const float m2 = (ag_warp_sum(s2) * inv_c) * scale;
      if (dx != nullptr) {
        T* dxr = dx + (first_row + j * (int64_t)gridDim.x) * C;
#pragma unroll
        for (int p = 0; p < KP; ++p) {
          const int col = (p * 32 + lane) * NV;
          if (col < C) {
            float g[NV], o[NV];
            Pack<T>::load(sdy + col, g);
            if (with_res) {
              Pack<T>::load(sres + col, o);
            } else {
#pragma unroll
              for (int e = 0; e < NV; ++e) o[e] = 0.0f;
            }
#pragma unroll
            for (int e4 = 0; e4 < NV; e4 += 4) {
              float4 gg = make_float4(1.f, 1.f, 1.f, 1.f);
              if (gamma) gg = *reinterpret_cast<const float4*>(s_gamma + col + e4);
              const float* gp = reinterpret_cast<const float*>(&gg);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int e = e4 + k;
                // backend.py:475-487: xg += dyg*rstd; xg -= m1; xg -= xhat*m2
                const float dg = gamma ? g[e] * gp[k] : g[e];
                float t = o[e] + dg * scale;
                if (KIND == kLayerNorm) t = t - m1;
                o[e] = t - v[p][e] * m2;
              }
            }
            Pack<T>::store(dxr + col, o);
          }
        }
      }
      __syncwarp();
      if (lane == 0) ag_mbar_arrive(&hd->empty[slot]);
    }
  }

  // every role is out of its loop; after an abort the copies still in flight are waited for before
  // the ring is reused for the fold
  __syncthreads();
  if (*abort_flag) {
    if (warp == CW && lane == 0) ring_drain(hd, R, status);
    __syncthreads();
  }
  // fold the warps' column sums in warp order: [warp][slot][C] floats in the ring's memory
  float* s_fold = reinterpret_cast<float*>(ring);
  if (warp < CW) {
    float* my_g = s_fold + (size_t)warp * SLOTS * C;
    float* my_b = my_g + C;
#pragma unroll
    for (int p = 0; p < KP; ++p) {
      const int col = (p * 32 + lane) * NV;
      if (col < C) {
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          my_g[col + e] = acc_g[p][e];
          if constexpr (KIND == kLayerNorm) my_b[col + e] = acc_b[p][e];
        }
      }
    }
  }
  __syncthreads();
  for (int slot = 0; slot < SLOTS; ++slot) {
    const bool wanted = slot == 0 ? (want_dgamma != 0) : (want_dbeta != 0);
    if (!wanted) continue;  // uniform across the CTA
    float* out = partials + ((int64_t)blockIdx.x * 2 + slot) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float t = 0.0f;
      for (int w = 0; w < CW; ++w) t += s_fold[((size_t)w * SLOTS + slot) * C + c];
      out[c] = t;
    }
  }
}

// ---------------------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------------------
// One-shot test hook: the next norm kernel that stages gamma/beta gives up its staging wait at once.
inline uint32_t take_stage_poll_limit(ag_ctx* ctx) {
  const uint32_t limit = ctx->debug_stage_expire ? 0u : (1u << 20);
  ctx->debug_stage_expire = 0;
  return limit;
}

// Two warps per row (see norm_backward_pair_kernel).  ctx->norm_pair: 0 never, 1 whenever the shape fits,
// 2 (default): fp32 rows of at least 1024 columns in backward, where the one-warp kernel needs 140-175
// registers (inside the benchmark step, 32768 x 1280: 0.85 of the copy rate against 0.70-0.75; 8192 x 1536
// alone: 0.75 against 0.70), and fp32 rows of at least 1536 columns in forward (8192 x 1536: 0.85 against
// 0.80; at 1280 columns the one-warp forward is as fast or faster, 0.92 against 0.90 alone).
// bf16 storage, backward: the pair kernel with a row ahead in registers (8192 x 1536: 0.52 against 0.48
// through the ring), for rows of up to 24 elements per lane.
inline bool pair_applies(const ag_ctx* ctx, int packets_per_row, int nv, bool backward) {
  const int kp2 = (packets_per_row + 63) / 64;
  if (!ctx->norm_pair || kp2 * nv > 24) return false;  // up to 24 row elements per lane: no register spills
  if (ctx->norm_pair == 1) return true;
  // bf16 storage, backward: the pair kernel holds the next row's packets in registers (a row ahead)
  if (nv == 8) return backward && ctx->norm_ring != 1;
  return nv == 4 && packets_per_row >= (backward ? 256 : 384);
}

inline int pick_kp(int packets_per_row) {
  const int need = (packets_per_row + 31) / 32;
  static const int kChoices[] = {1, 2, 3, 4, 5, 6, 8, 10, 12, 16};
  for (int k : kChoices)
    if (k >= need) return k;
  return 0;
}

// Persistent grid: exactly the number of CTAs that are resident at once (occupancy x SMs),
// so that no partial second wave forms; fewer when there are not enough rows.
// When every warp would visit only a few rows, a resident-sized grid quantises badly (2.3 rows
// per warp costs 3 iterations); then one CTA per 8 rows is launched instead and the hardware
// scheduler fills SMs as CTAs retire.  `max_grid` bounds the grid where each CTA owns a partial row.
inline int persistent_grid(const ag_ctx* ctx, int64_t N, int ctas_per_sm, int64_t max_grid = (1ll << 30),
                           int rows_per_cta = NORM_WARPS) {
  int64_t want = (N + rows_per_cta - 1) / rows_per_cta;
  if (ctas_per_sm < 1) ctas_per_sm = 1;
  if (ctas_per_sm > 8) ctas_per_sm = 8;
  int64_t cap = (int64_t)ctx->sm_count * ctas_per_sm;
  if (want < 1) want = 1;
  int64_t grid = want <= cap ? want : (want <= 6 * cap ? want : cap);
  if (grid > max_grid) grid = max_grid > cap ? max_grid / cap * cap : max_grid;
  return (int)grid;
}

// Resident CTAs per SM of one kernel instantiation at a given dynamic shared-memory size;
// queried once per (kernel, device, smem) and cached (single host thread per context).
template <typename K>
int resident_ctas(ag_ctx* ctx, K kern, size_t smem, int* cache, size_t* cache_smem, int threads = NORM_THREADS) {
  if (*cache > 0 && *cache_smem == smem) return *cache;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return -1;
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, smem) != cudaSuccess) return -1;
  *cache = occ < 1 ? 1 : occ;
  *cache_smem = smem;
  (void)ctx;
  return *cache;
}

template <typename T, int KIND, int KP>
int launch_fwd_kp(ag_ctx* ctx, const T* x, const T* r, const float* gamma, const float* beta, T* h, T* y, float* s0,
                  float* s1, int64_t N, int C, float eps) {
  const size_t smem = (size_t)2 * C * sizeof(float);
  auto kern = norm_forward_kernel<T, KP, KIND>;
  static int occ_cache[AG_MAX_DEVICES] = {};
  static size_t occ_smem[AG_MAX_DEVICES] = {};
  const int occ = resident_ctas(ctx, kern, smem, &occ_cache[ag_dev_slot(ctx)], &occ_smem[ag_dev_slot(ctx)]);
  if (occ < 0) AG_FAIL(ctx, AG_ERR_CUDA, "norm_forward_kernel: occupancy query failed: %s", cudaGetErrorString(cudaGetLastError()));
  const int grid = persistent_grid(ctx, N, occ);
  AG_LAUNCH_PDL(ctx, "norm_forward_kernel", kern, grid, NORM_THREADS, smem, x, r, gamma, beta, h, y, s0, s1, N, C, eps,
                take_stage_poll_limit(ctx), ctx->d_status, grid <= ctx->sm_count * occ ? 1 : 0);
  return AG_OK;
}

// Which shapes take the row ring.  Measured on B200 (back-to-back launches, operands rotated through
// more buffers than fit in L2): with fp32 storage the ring and the register kernels reach the same HBM
// rate on long inputs (32768 x 1280: 0.92 / 0.91 of the copy rate forward / backward with rows in
// registers, 0.86 / 0.92 through the ring) and the register kernels win on short ones (16384 x 384
// backward 0.68 vs 0.60; 8192 x 1536 backward 0.745 with two warps per row vs 0.70), so fp32 keeps its
// rows in registers.  With bf16 storage a lane's 16-byte packet holds half as many bytes per element in
// flight; there the ring wins over the one-warp kernels (8192 x 1536: forward 0.57 vs 0.53, backward 0.48 vs
// 0.38); the bf16 backward is taken by the pair kernel first where the row fits it (see pair_applies).
// ctx->norm_ring: 0 never, 1 always where the shape fits, 2 (default) this policy.
inline bool ring_applies(const ag_ctx* ctx, int kp, int nv, int64_t N, bool backward, int packets_per_row) {
  if (!ctx->norm_ring || kp <= 0 || kp * nv > RING_MAX_PER_LANE || N >= (1ll << 31)) return false;
  if (ctx->norm_ring == 1) return true;
  // bf16 storage: forward always; backward only for rows too wide for the pair kernel
  return nv == 8 && !(backward && pair_applies(ctx, packets_per_row, nv, true));
}

template <typename T, int KIND, int KP>
int launch_fwd_ring_kp(ag_ctx* ctx, const T* x, const T* r, const float* gamma, const float* beta, T* h, T* y,
                       float* s0, float* s1, int64_t N, int C, float eps) {
  if constexpr (KP * Pack<T>::N > RING_MAX_PER_LANE) {
    AG_FAIL(ctx, AG_ERR_INVALID, "norm_forward_ring_kernel: row too wide");
  } else {
    const RingPlan plan = ring_plan(C, sizeof(T), r ? 2 : 1, KIND == kLayerNorm ? 2 : 1, 0);
    if (plan.slots == 0) return -1;
    const int threads = (plan.consumers + 1) * 32;
    auto kern = norm_forward_ring_kernel<T, KP, KIND>;
    static int occ_cache[AG_MAX_DEVICES] = {};
    static size_t occ_smem[AG_MAX_DEVICES] = {};
    const int occ = resident_ctas(ctx, kern, plan.smem, &occ_cache[ag_dev_slot(ctx)], &occ_smem[ag_dev_slot(ctx)],
                                  threads);
    if (occ < 0)
      AG_FAIL(ctx, AG_ERR_CUDA, "norm_forward_ring_kernel: occupancy query failed: %s",
              cudaGetErrorString(cudaGetLastError()));
    const int64_t cap = (int64_t)ctx->sm_count * (occ > 8 ? 8 : occ);
    const int grid = (int)(N < cap ? N : cap);
    AG_LAUNCH_PDL(ctx, "norm_forward_ring_kernel", kern, grid, threads, plan.smem, x, r, gamma, beta, h, y, s0, s1,
                  N, C, eps, plan.slots, plan.consumers, plan.slot_bytes, take_stage_poll_limit(ctx), ctx->d_status, 1);
    return AG_OK;
  }
}

template <typename T, int KIND, int KP2>
int launch_fwd_pair_kp(ag_ctx* ctx, const T* x, const T* r, const float* gamma, const float* beta, T* h, T* y, float* s0,
                       float* s1, int64_t N, int C, float eps) {
  const size_t smem = (size_t)2 * C * sizeof(float);
  auto kern = norm_forward_pair_kernel<T, KP2, KIND>;
  static int occ_cache[AG_MAX_DEVICES] = {};
  static size_t occ_smem[AG_MAX_DEVICES] = {};
  const int occ = resident_ctas(ctx, kern, smem, &occ_cache[ag_dev_slot(ctx)], &occ_smem[ag_dev_slot(ctx)]);
  if (occ < 0)
    AG_FAIL(ctx, AG_ERR_CUDA, "norm_forward_pair_kernel: occupancy query failed: %s", cudaGetErrorString(cudaGetLastError()));
  const int grid = persistent_grid(ctx, N, occ, (1ll << 30), PAIR_TEAMS);
  AG_LAUNCH_PDL(ctx, "norm_forward_pair_kernel", kern, grid, NORM_THREADS, smem, x, r, gamma, beta, h, y, s0, s1, N, C, eps,
                take_stage_poll_limit(ctx), ctx->d_status, grid <= ctx->sm_count * occ ? 1 : 0);
  return AG_OK;
}

template <typename T, int KIND>
int launch_fwd(ag_ctx* ctx, const T* x, const T* r, const float* gamma, const float* beta, T* h, T* y, float* s0,
               float* s1, int64_t N, int C, float eps) {
  constexpr int NV = Pack<T>::N;
  const bool vec_ok = (C % NV == 0) && ag_aligned16(x) && ag_aligned16(r) && ag_aligned16(h) && ag_aligned16(y);
  const int kp = vec_ok ? pick_kp(C / NV) : 0;
  if (ring_applies(ctx, kp, NV, N, false, C / NV)) {
    int rc = -1;
#define AG_FWD_RING_CASE(K)                                                                   \
  case K:                                                                                     \
    rc = launch_fwd_ring_kp<T, KIND, K>(ctx, x, r, gamma, beta, h, y, s0, s1, N, C, eps);     \
    break;
    switch (kp) {
      AG_FWD_RING_CASE(1) AG_FWD_RING_CASE(2) AG_FWD_RING_CASE(3) AG_FWD_RING_CASE(4) AG_FWD_RING_CASE(5)
      AG_FWD_RING_CASE(6) AG_FWD_RING_CASE(8) AG_FWD_RING_CASE(10) AG_FWD_RING_CASE(12)
      default:
        break;
    }
#undef AG_FWD_RING_CASE
    if (rc >= 0) return rc;  // -1: the ring does not take this shape, the register kernels do
  }
  if (vec_ok && pair_applies(ctx, C / NV, NV, false)) {
#define AG_FWD_PAIR_CASE(K) \
  case K:                   \
    return launch_fwd_pair_kp<T, KIND, K>(ctx, x, r, gamma, beta, h, y, s0, s1, N, C, eps);
    switch ((C / NV + 63) / 64) {
      AG_FWD_PAIR_CASE(1) AG_FWD_PAIR_CASE(2) AG_FWD_PAIR_CASE(3) AG_FWD_PAIR_CASE(4) AG_FWD_PAIR_CASE(5)
      AG_FWD_PAIR_CASE(6)
      default:
        break;
    }
#undef AG_FWD_PAIR_CASE
  }
#define AG_FWD_CASE(K) \
  case K:              \
    return launch_fwd_kp<T, KIND, K>(ctx, x, r, gamma, beta, h, y, s0, s1, N, C, eps);
  switch (kp) {
    AG_FWD_CASE(1) AG_FWD_CASE(2) AG_FWD_CASE(3) AG_FWD_CASE(4) AG_FWD_CASE(5) AG_FWD_CASE(6) AG_FWD_CASE(8)
    AG_FWD_CASE(10) AG_FWD_CASE(12) AG_FWD_CASE(16)
    default:
      break;
  }
#undef AG_FWD_CASE
  int64_t cap = (int64_t)ctx->sm_count * 8;
  int grid = (int)(N < cap ? N : cap);
  norm_forward_generic_kernel<T, KIND><<<grid, NORM_THREADS, 0, ctx->stream>>>(x, r, gamma, beta, h, y, s0, s1, N, C, eps);
  AG_LAUNCHED(ctx, "norm_forward_generic_kernel");
  return AG_OK;
}

// Shared memory of the row-in-registers backward kernel, and whether it fits an SM.
template <int KIND>
size_t norm_bwd_smem(int C) { return (size_t)(1 + NORM_WARPS * norm_bwd_slots<KIND>()) * C * sizeof(float); }
constexpr size_t kNormSmemLimit = 200 * 1024;

// Largest grid any backward launch may use: bounds the partials workspace.
inline int max_partial_rows(const ag_ctx* ctx) { return ctx->sm_count * 8; }

template <typename T, int KIND, int KP>
int launch_bwd_kp(ag_ctx* ctx, const T* dy, const T* x, const float* gamma, const T* dres, T* dx, float* partials,
                  int wg, int wb, int64_t N, int C, float eps, int max_grid, int* grid_out) {
  const size_t smem = norm_bwd_smem<KIND>(C);
  auto kern = norm_backward_kernel<T, KP, KIND>;
  static int occ_cache[AG_MAX_DEVICES] = {};
  static size_t occ_smem[AG_MAX_DEVICES] = {};
  const int occ = resident_ctas(ctx, kern, smem, &occ_cache[ag_dev_slot(ctx)], &occ_smem[ag_dev_slot(ctx)]);
  if (occ < 0) AG_FAIL(ctx, AG_ERR_CUDA, "norm_backward_kernel: occupancy query failed: %s", cudaGetErrorString(cudaGetLastError()));
  const int grid = persistent_grid(ctx, N, occ, max_grid);
  AG_LAUNCH_PDL(ctx, "norm_backward_kernel", kern, grid, NORM_THREADS, smem, dy, x, gamma, dres, dx, partials, wg, wb, N, C,
                eps, take_stage_poll_limit(ctx), ctx->d_status, grid <= ctx->sm_count * occ ? 1 : 0);
  *grid_out = grid;
  return AG_OK;
}

template <int KIND>
size_t norm_bwd_pair_smem(int C) { return (size_t)(1 + PAIR_TEAMS * norm_bwd_slots<KIND>()) * C * sizeof(float); }

template <typename T, int KIND, int KP2>
int launch_bwd_pair_kp(ag_ctx* ctx, const T* dy, const T* x, const float* gamma, const T* dres, T* dx, float* partials,
                       int wg, int wb, int64_t N, int C, float eps, int max_grid, int* grid_out) {
  const size_t smem = norm_bwd_pair_smem<KIND>(C);
  auto kern = norm_backward_pair_kernel<T, KP2, KIND>;
  static int occ_cache[AG_MAX_DEVICES] = {};
  static size_t occ_smem[AG_MAX_DEVICES] = {};
  const int occ = resident_ctas(ctx, kern, smem, &occ_cache[ag_dev_slot(ctx)], &occ_smem[ag_dev_slot(ctx)]);
  if (occ < 0)
    AG_FAIL(ctx, AG_ERR_CUDA, "norm_backward_pair_kernel: occupancy query failed: %s", cudaGetErrorString(cudaGetLastError()));
  const int grid = persistent_grid(ctx, N, occ, max_grid, PAIR_TEAMS);
  AG_LAUNCH_PDL(ctx, "norm_backward_pair_kernel", kern, grid, NORM_THREADS, smem, dy, x, gamma, dres, dx, partials, wg, wb, N,
                C, eps, take_stage_poll_limit(ctx), ctx->d_status, grid <= ctx->sm_count * occ ? 1 : 0);
  *grid_out = grid;
  return AG_OK;
}

template <typename T, int KIND, int KP>
int launch_bwd_ring_kp(ag_ctx* ctx, const T* dy, const T* x, const float* gamma, const T* dres, T* dx, float* partials,
                       int wg, int wb, int64_t N, int C, float eps, int max_grid, int* grid_out) {
  if constexpr (KP * Pack<T>::N > RING_MAX_PER_LANE) {
    AG_FAIL(ctx, AG_ERR_INVALID, "norm_backward_ring_kernel: row too wide");
  } else {
    const RingPlan plan = ring_plan(C, sizeof(T), (dres && dx) ? 3 : 2, 1, norm_bwd_slots<KIND>());
    if (plan.slots == 0) return -1;
    const int threads = (plan.consumers + 1) * 32;
    auto kern = norm_backward_ring_kernel<T, KP, KIND>;
    static int occ_cache[AG_MAX_DEVICES] = {};
    static size_t occ_smem[AG_MAX_DEVICES] = {};
    const int occ = resident_ctas(ctx, kern, plan.smem, &occ_cache[ag_dev_slot(ctx)], &occ_smem[ag_dev_slot(ctx)],
                                  threads);
    if (occ < 0)
      AG_FAIL(ctx, AG_ERR_CUDA, "norm_backward_ring_kernel: occupancy query failed: %s",
              cudaGetErrorString(cudaGetLastError()));
    int64_t cap = (int64_t)ctx->sm_count * (occ > 8 ? 8 : occ);
    if (cap > max_grid) cap = max_grid;
    const int grid = (int)(N < cap ? N : cap);
    AG_LAUNCH_PDL(ctx, "norm_backward_ring_kernel", kern, grid, threads, plan.smem, dy, x, gamma, dres, dx, partials,
                  wg, wb, N, C, eps, plan.slots, plan.consumers, plan.slot_bytes, take_stage_poll_limit(ctx), ctx->d_status, 1);
    *grid_out = grid;
    return AG_OK;
  }
}

// `small_workspace`: the caller's workspace may hold fewer partial rows than ag_norm_partials_bytes
// asks for; the grid is then clipped to the rows that fit (the allocation-free entry point).
template <typename T, int KIND>
int launch_bwd(ag_ctx* ctx, const T* dy, const T* x, const float* gamma, const T* dres, T* dx, float* dgamma,
               float* dbeta, void* partials_v, size_t partials_bytes, int64_t N, int C, float eps,
               bool small_workspace = false) {
  constexpr int NV = Pack<T>::N;
  float* partials = static_cast<float*>(partials_v);
  const int wg = dgamma != nullptr, wb = (KIND == kLayerNorm) && dbeta != nullptr;
  int max_grid = max_partial_rows(ctx);
  if (wg || wb) {
    if (!partials || (!small_workspace && partials_bytes < ag_norm_partials_bytes(ctx, C)))
      AG_FAIL(ctx, AG_ERR_SCRATCH, "norm backward: partials workspace has %zu bytes, needs %zu", partials_bytes,
              ag_norm_partials_bytes(ctx, C));
    AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(partials) & 3u) == 0, "norm backward: partials not 4-byte aligned");
    const size_t fit = partials_bytes / ((size_t)2 * C * sizeof(float));
    if (fit < (size_t)max_grid) max_grid = (int)fit;
    if (max_grid < 1) AG_FAIL(ctx, AG_ERR_SCRATCH, "norm backward: partials workspace holds no row of %d columns", C);
  }
  const bool vec_ok = (C % NV == 0) && ag_aligned16(dy) && ag_aligned16(x) && ag_aligned16(dres) && ag_aligned16(dx) &&
                      norm_bwd_smem<KIND>(C) <= kNormSmemLimit;
  const int kp = vec_ok ? pick_kp(C / NV) : 0;
  int grid = 0;
  int rc = -1;
  if (ring_applies(ctx, kp, NV, N, true, C / NV)) {
#define AG_BWD_RING_CASE(K)                                                                                          \
  case K:                                                                                                            \
    rc = launch_bwd_ring_kp<T, KIND, K>(ctx, dy, x, gamma, dres, dx, partials, wg, wb, N, C, eps, max_grid, &grid);  \
    break;
    switch (kp) {
      AG_BWD_RING_CASE(1) AG_BWD_RING_CASE(2) AG_BWD_RING_CASE(3) AG_BWD_RING_CASE(4) AG_BWD_RING_CASE(5)
      AG_BWD_RING_CASE(6) AG_BWD_RING_CASE(8) AG_BWD_RING_CASE(10) AG_BWD_RING_CASE(12)
      default:
        break;
    }
#undef AG_BWD_RING_CASE
  }
  if (rc < 0 && vec_ok && pair_applies(ctx, C / NV, NV, true)) {
#define AG_BWD_PAIR_CASE(K)                                                                                          \
  case K:                                                                                                            \
    rc = launch_bwd_pair_kp<T, KIND, K>(ctx, dy, x, gamma, dres, dx, partials, wg, wb, N, C, eps, max_grid, &grid);  \
    break;
    switch ((C / NV + 63) / 64) {
      AG_BWD_PAIR_CASE(1) AG_BWD_PAIR_CASE(2) AG_BWD_PAIR_CASE(3) AG_BWD_PAIR_CASE(4) AG_BWD_PAIR_CASE(5)
      AG_BWD_PAIR_CASE(6)
      default:
        break;
    }
#undef AG_BWD_PAIR_CASE
  }
  if (rc < 0) {
#define AG_BWD_CASE(K)                                                                                            \
  case K:                                                                                                         \
    rc = launch_bwd_kp<T, KIND, K>(ctx, dy, x, gamma, dres, dx, partials, wg, wb, N, C, eps, max_grid, &grid);    \
    break;
  switch (kp) {
    AG_BWD_CASE(1) AG_BWD_CASE(2) AG_BWD_CASE(3) AG_BWD_CASE(4) AG_BWD_CASE(5) AG_BWD_CASE(6) AG_BWD_CASE(8)
    AG_BWD_CASE(10) AG_BWD_CASE(12) AG_BWD_CASE(16)
    default:
      break;
  }
#undef AG_BWD_CASE
  }
  if (rc > 0) return rc;
  if (rc < 0) {
    const size_t smem = (size_t)2 * C * sizeof(float);
    auto kern = norm_backward_generic_kernel<T, KIND>;
    if (smem > 48 * 1024)
      AG_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t cap = (int64_t)ctx->sm_count * 4;
    if (cap > max_grid) cap = max_grid;
    grid = (int)(N < cap ? N : cap);
    kern<<<grid, NORM_THREADS, smem, ctx->stream>>>(dy, x, gamma, dres, dx, partials, wg, wb, N, C, eps);
    AG_LAUNCHED(ctx, "norm_backward_generic_kernel");
  }
  if (wg || wb) {
    dim3 rgrid((C + 31) / 32, KIND == kLayerNorm ? 2 : 1);
    AG_LAUNCH_PDL(ctx, "norm_partials_reduce_kernel", norm_partials_reduce_kernel, rgrid, dim3(32, 32), 0,
                  (const float*)partials, grid, C, wg ? dgamma : (float*)nullptr, wb ? dbeta : (float*)nullptr);
  }
  return AG_OK;
}

}  // namespace

// =========================================================================================
extern "C" size_t ag_norm_partials_bytes(ag_ctx* ctx, int C) {
  if (!ctx || C <= 0) return 0;
  return (size_t)max_partial_rows(ctx) * 2 * (size_t)C * sizeof(float);
}

extern "C" int ag_add_layernorm_forward(ag_ctx* ctx, const float* x, const float* r, const float* gamma,
                                        const float* beta, float* h, float* y, float* mean, float* rstd, int64_t N,
                                        int C, float eps) {
  if (!ctx) return AG_ERR_INVALID;
  if (N == 0) return AG_OK;
  AG_REQUIRE(ctx, x && gamma && beta && y, "ag_add_layernorm_forward: null pointer");
  AG_REQUIRE(ctx, N > 0 && C > 0, "ag_add_layernorm_forward: bad shape N=%lld C=%d", (long long)N, C);
  AG_REQUIRE(ctx, (size_t)2 * C * 4 <= 200 * 1024, "ag_add_layernorm_forward: C=%d too large", C);
  return launch_fwd<float, kLayerNorm>(ctx, x, r, gamma, beta, h, y, mean, rstd, N, C, eps);
}

extern "C" int ag_layernorm_backward(ag_ctx* ctx, const float* dy, const float* x, const float* gamma,
                                     const float* dres, float* dx, float* dgamma, float* dbeta, void* partials,
                                     size_t partials_bytes, int64_t N, int C, float eps) {
  if (!ctx) return AG_ERR_INVALID;
  if (N == 0) return AG_OK;
  AG_REQUIRE(ctx, dy && x && gamma, "ag_layernorm_backward: null pointer");
  AG_REQUIRE(ctx, N > 0 && C > 0, "ag_layernorm_backward: bad shape N=%lld C=%d", (long long)N, C);
  AG_REQUIRE(ctx, (size_t)2 * C * 4 <= kNormSmemLimit, "ag_layernorm_backward: C=%d too large", C);
  return launch_bwd<float, kLayerNorm>(ctx, dy, x, gamma, dres, dx, dgamma, dbeta, partials, partials_bytes, N, C, eps);
}

extern "C" int ag_rmsnorm_forward(ag_ctx* ctx, const void* x, const float* gamma, void* y, float* inv_rms, int64_t N,
                                  int C, float eps, int dtype) {
  if (!ctx) return AG_ERR_INVALID;
  if (N == 0) return AG_OK;
  AG_REQUIRE(ctx, x && y, "ag_rmsnorm_forward: null pointer");
  AG_REQUIRE(ctx, N > 0 && C > 0, "ag_rmsnorm_forward: bad shape N=%lld C=%d", (long long)N, C);
  AG_REQUIRE(ctx, dtype == AG_F32 || dtype == AG_BF16, "ag_rmsnorm_forward: unknown dtype %d", dtype);
  AG_REQUIRE(ctx, (size_t)2 * C * 4 <= 200 * 1024, "ag_rmsnorm_forward: C=%d too large", C);
  if (dtype == AG_F32)
    return launch_fwd<float, kRmsNorm>(ctx, static_cast<const float*>(x), nullptr, gamma, nullptr, nullptr,
                                       static_cast<float*>(y), inv_rms, nullptr, N, C, eps);
  return launch_fwd<__nv_bfloat16, kRmsNorm>(ctx, static_cast<const __nv_bfloat16*>(x), nullptr, gamma, nullptr,
                                             nullptr, static_cast<__nv_bfloat16*>(y), inv_rms, nullptr, N, C, eps);
}

extern "C" int ag_rmsnorm_backward(ag_ctx* ctx, const void* dz, const void* x, const float* gamma, const void* dres,
                                   void* dx, float* dgamma, void* partials, size_t partials_bytes, int64_t N, int C,
                                   float eps, int dtype) {
  if (!ctx) return AG_ERR_INVALID;
  if (N == 0) return AG_OK;
  AG_REQUIRE(ctx, dz && x, "ag_rmsnorm_backward: null pointer");
  AG_REQUIRE(ctx, N > 0 && C > 0, "ag_rmsnorm_backward: bad shape N=%lld C=%d", (long long)N, C);
  AG_REQUIRE(ctx, dtype == AG_F32 || dtype == AG_BF16, "ag_rmsnorm_backward: unknown dtype %d", dtype);
  AG_REQUIRE(ctx, gamma || !dgamma, "ag_rmsnorm_backward: dgamma requested without gamma");
  AG_REQUIRE(ctx, (size_t)2 * C * 4 <= kNormSmemLimit, "ag_rmsnorm_backward: C=%d too large", C);
  if (dtype == AG_F32)
    return launch_bwd<float, kRmsNorm>(ctx, static_cast<const float*>(dz), static_cast<const float*>(x), gamma,
                                       static_cast<const float*>(dres), static_cast<float*>(dx), dgamma, nullptr,
                                       partials, partials_bytes, N, C, eps);
  return launch_bwd<__nv_bfloat16, kRmsNorm>(ctx, static_cast<const __nv_bfloat16*>(dz),
                                             static_cast<const __nv_bfloat16*>(x), gamma,
                                             static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx),
                                             dgamma, nullptr, partials, partials_bytes, N, C, eps);
}

// =========================================================================================
// LayerNorm backward for callers that cannot allocate device memory.
//
// Some hosts of this library hand it only the tensors of the op: a runtime whose arena was
// sized before this backend was registered, a plugin slot with no allocator callback, or a
// caller inside a region where cudaMalloc is forbidden.  ag_layernorm_backward needs a
// workspace for its per-CTA dgamma/dbeta partial rows; this variant keeps that workspace in
// a fixed array inside the library image instead.  Nothing is allocated or freed here, and
// no allocating library routine is called.
//
// The array costs AG_LN_NOALLOC_SCRATCH_BYTES of device memory on every GPU that loads the
// library, until the process exits.  It is shared by all calls: two calls whose kernels
// overlap on the GPU (different streams or contexts) race on it; calls on one stream are
// safe.  Nothing in it has to start at zero - every partial row the second pass reads is
// written in full by the first pass of the same call - so stale contents are harmless.
//
// In host code the array's name is only a stand-in for the symbol, not a device address.
// The address comes from cudaGetSymbolAddress, looked up once per device with that device
// current, on the first call made on that device; do that first call outside any stream
// capture.
// =========================================================================================
namespace {

constexpr size_t kLnNoallocScratchBytes = (size_t)AG_LN_NOALLOC_SCRATCH_BYTES;
constexpr int kLnNoallocMaxDevices = 64;

static __device__ __align__(256) float g_ln_noalloc_scratch[kLnNoallocScratchBytes / sizeof(float)];

float* g_ln_noalloc_addr[kLnNoallocMaxDevices] = {};

int ln_noalloc_scratch(ag_ctx* ctx, float** out) {
  AG_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kLnNoallocMaxDevices, "device ordinal %d out of range", ctx->device);
  if (!g_ln_noalloc_addr[ctx->device]) {
    int current = -1;
    AG_CUDA(ctx, cudaGetDevice(&current));
    if (current != ctx->device) AG_CUDA(ctx, cudaSetDevice(ctx->device));
    void* p = nullptr;
    AG_CUDA(ctx, cudaGetSymbolAddress(&p, g_ln_noalloc_scratch));
    if (current != ctx->device && current >= 0) AG_CUDA(ctx, cudaSetDevice(current));
    g_ln_noalloc_addr[ctx->device] = static_cast<float*>(p);
  }
  *out = g_ln_noalloc_addr[ctx->device];
  return AG_OK;
}

}  // namespace

extern "C" int ag_layernorm_backward_noalloc(ag_ctx* ctx, const float* dy, const float* x, const float* gamma,
                                             const float* dres, float* dx, float* dgamma, float* dbeta, int64_t N,
                                             int C, float eps) {
  if (!ctx) return AG_ERR_INVALID;
  if (N == 0) return AG_OK;
  AG_REQUIRE(ctx, dy && x && gamma, "ag_layernorm_backward_noalloc: null pointer");
  AG_REQUIRE(ctx, N > 0 && C > 0, "ag_layernorm_backward_noalloc: bad shape N=%lld C=%d", (long long)N, C);
  if (C > AG_LN_NOALLOC_MAX_C)
    AG_FAIL(ctx, AG_ERR_INVALID,
            "ag_layernorm_backward_noalloc: C=%d exceeds the built-in workspace limit of %d columns; use "
            "ag_layernorm_backward with a caller-provided workspace",
            C, AG_LN_NOALLOC_MAX_C);
  float* partials = nullptr;
  int rc = ln_noalloc_scratch(ctx, &partials);
  if (rc) return rc;
  // Same kernels as ag_layernorm_backward; the grid is clipped to the partial rows that fit the
  // fixed array, and every partial row the second pass reads is written by the first pass of
  // this call.
  return launch_bwd<float, kLayerNorm>(ctx, dy, x, gamma, dres, dx, dgamma, dbeta, partials, kLnNoallocScratchBytes, N, C,
                                       eps, /*small_workspace=*/true);
}

// Test hook for the unwind path of the gamma/beta staging (a wait that gives up): the next norm
// kernel launched through ctx that stages these vectors in shared memory (rows of more than 512 fp32
// columns, and every row-ring kernel) treats its staging wait as expired at once, records
// AG_STATUS_STAGE_FALLBACK, lets the copy land and fills the vectors with plain loads.
extern "C" int ag_debug_expire_staging(ag_ctx* ctx) {
  if (!ctx) return AG_ERR_INVALID;
  ctx->debug_stage_expire = 1;
  return AG_OK;
}
