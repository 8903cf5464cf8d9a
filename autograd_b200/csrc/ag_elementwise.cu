// Bandwidth-bound elementwise kernels: residual add, tanh-GELU, SwiGLU, AdamW.
// All use 16-byte packets, grid-stride loops with several independent packets in flight per
// thread, grids sized in multiples of the SM count, and IEEE math (no fast-math) so that
// fp32 results stay within 1e-5 of the numpy reference.
#include "ag_common.cuh"

namespace {

constexpr int EW_THREADS = 256;
constexpr int EW_UNROLL = 4;

// Grid of an elementwise kernel: one CTA per EW_THREADS * EW_UNROLL packets, at most cap_mult CTAs per
// SM (0: no limit, every thread makes one pass).  Measured at 32768 x 5120 fp32: the two- and
// three-stream kernels with light arithmetic (add, GELU forward, SwiGLU) run 4-13 % faster without a
// limit; GELU backward and AdamW (more live values per thread) are faster with a small resident grid.
inline int ew_grid(const ag_ctx* ctx, int64_t packets, int cap_mult) {
  int64_t want = (packets + (int64_t)EW_THREADS * EW_UNROLL - 1) / ((int64_t)EW_THREADS * EW_UNROLL);
  if (want < 1) want = 1;
  if (cap_mult > 0) {
    const int64_t cap = (int64_t)ctx->sm_count * cap_mult;
    if (want > cap) want = cap;
  }
  if (want > 0x7fffffff) want = 0x7fffffff;
  return (int)want;
}
// CTAs of `kern` that an SM holds at once (queried once per kernel and device): a kernel that loops over a
// resident grid wants exactly one wave of them.
template <typename K>
int ew_resident(const ag_ctx* ctx, K kern, int* cache) {
  if (*cache <= 0) {
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, EW_THREADS, 0) != cudaSuccess || occ < 1) {
      (void)cudaGetLastError();
      occ = 2;
    }
    *cache = occ > 8 ? 8 : occ;
  }
  (void)ctx;
  return *cache;
}

// Whether a grid is resident in one wave for certain (then the kernel lets its successor be scheduled early).
inline int ew_early(const ag_ctx* ctx, int grid) { return grid <= ctx->sm_count * 4 ? 1 : 0; }

// Generic driver: F is a functor with
//   template<int NV> void packet(int64_t elem_index)   - process one 16-byte packet
//   void scalar(int64_t elem_index)                    - process one element (ragged tail)
template <int NV, int UNROLL = EW_UNROLL, typename F>
__device__ __forceinline__ void ew_drive(int64_t n, F& f, int early) {
  ag_pdl_wait();
  if (early) ag_pdl_trigger();
  const int64_t packets = n / NV;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (UNROLL - 1) * stride < packets; i += UNROLL * stride) f.template packets<UNROLL>(i, stride);
  for (; i < packets; i += stride) f.template packets<1>(i, stride);
  const int64_t tail = packets * NV;
  for (int64_t j = tail + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) f.scalar(j);
}

// ---------------------------------------------------------------------------- add
struct AddFwd {
  const float* x;
  const float* y;
  float* out;
  template <int U>
  __device__ __forceinline__ void packets(int64_t i, int64_t stride) {
    float a[U][4], b[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      Pack<float>::load_stream(x + (i + u * stride) * 4, a[u]);
      Pack<float>::load_stream(y + (i + u * stride) * 4, b[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int e = 0; e < 4; ++e) a[u][e] += b[u][e];
      Pack<float>::store(out + (i + u * stride) * 4, a[u]);
    }
  }
  __device__ __forceinline__ void scalar(int64_t j) { out[j] = x[j] + y[j]; }
};

__global__ void __launch_bounds__(EW_THREADS) add_forward_kernel(AddFwd f, int64_t n, int early) { ew_drive<4>(n, f, early); }

struct AddBwd {
  const float* g;
  float* xg;
  float* yg;
  template <int U>
  __device__ __forceinline__ void packets(int64_t i, int64_t stride) {
    float gv[U][4], a[U][4], b[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      Pack<float>::load(g + (i + u * stride) * 4, gv[u]);
      if (xg) Pack<float>::load(xg + (i + u * stride) * 4, a[u]);
      if (yg) Pack<float>::load(yg + (i + u * stride) * 4, b[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (xg) {
#pragma unroll
        for (int e = 0; e < 4; ++e) a[u][e] += gv[u][e];
        Pack<float>::store(xg + (i + u * stride) * 4, a[u]);
      }
      if (yg) {
#pragma unroll
        for (int e = 0; e < 4; ++e) b[u][e] += gv[u][e];
        Pack<float>::store(yg + (i + u * stride) * 4, b[u]);
      }
    }
  }
  __device__ __forceinline__ void scalar(int64_t j) {
    if (xg) xg[j] += g[j];
    if (yg) yg[j] += g[j];
  }
};

__global__ void __launch_bounds__(EW_THREADS) add_backward_kernel(AddBwd f, int64_t n, int early) { ew_drive<4>(n, f, early); }

// ---------------------------------------------------------------------------- GELU
// backend.py:18-20
constexpr float kGeluC = 0.7978845608028654f;
constexpr float kGeluA = 0.044715f;
constexpr float kGeluA3 = 0.134145f;

// With e = e^(2b) and q = 2 / (1 + e):  1 - tanh(b) = q,  1 + tanh(b) = q e,  1 - tanh(b)^2 = q^2 e.
// Only products, so no cancellation at either end; e from the ex2-based exponential and q from the
// approximate division are each good to a few ulp, and q e = 2e / (1 + e) is insensitive to the error
// of e where e is large.  Modelled and measured error of both GELU outputs: about 4e-7 of their rms,
// against bounds of 1e-5 / 1e-4.  tanhf costs three to four times the instructions and made both
// kernels issue-bound.  b is capped at 40 (tanh is 1 to the last bit from 9 on) so that 1 + e stays
// inside the range of the approximate division; e underflowing to 0 gives 1 + t = 0, as it should.
__device__ __forceinline__ void gelu_tanh_parts(float x, float& one_plus_t, float& one_minus_t2) {
  // backend.py:380-385: ((x*x)*x)*A, + x, *C, tanh
  float b = x * x;
  b = b * x;
  b = b * kGeluA;
  b = x + b;
  b = b * kGeluC;
  b = fminf(b, 40.0f);
  const float e = __expf(2.0f * b);
  const float q = __fdividef(2.0f, 1.0f + e);
  one_plus_t = q * e;
  one_minus_t2 = q * one_plus_t;
}

__device__ __forceinline__ float gelu_fwd1(float x) {
  float opt, omt2;
  gelu_tanh_parts(x, opt, omt2);
  return (x * opt) * 0.5f;
}

__device__ __forceinline__ float gelu_grad1(float x) {
  // backend.py:396-411
  float opt, omt2;
  gelu_tanh_parts(x, opt, omt2);
  const float d_inner = kGeluC * (1.0f + kGeluA3 * x * x);
  return opt * 0.5f + omt2 * (0.5f * x * d_inner);
}

struct GeluFwd {
  const float* x;
  float* y;
  template <int U>
  __device__ __forceinline__ void packets(int64_t i, int64_t stride) {
    float a[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) Pack<float>::load_stream(x + (i + u * stride) * 4, a[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int e = 0; e < 4; ++e) a[u][e] = gelu_fwd1(a[u][e]);
      Pack<float>::store(y + (i + u * stride) * 4, a[u]);
    }
  }
  __device__ __forceinline__ void scalar(int64_t j) { y[j] = gelu_fwd1(x[j]); }
};

__global__ void __launch_bounds__(EW_THREADS) gelu_forward_kernel(GeluFwd f, int64_t n, int early) { ew_drive<4>(n, f, early); }

// HAS_RES: dx = dres + local (the accumulate-into-grad form); without it no registers are held for dres,
// which lets a third CTA share the SM (more loads in flight).
template <bool HAS_RES>
struct GeluBwd {
  const float* x;
  const float* dy;
  const float* dres;
  float* dx;
  template <int U>
  __device__ __forceinline__ void packets(int64_t i, int64_t stride) {
    float a[U][4], g[U][4], r[HAS_RES ? U : 1][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      Pack<float>::load_stream(x + (i + u * stride) * 4, a[u]);
      Pack<float>::load_stream(dy + (i + u * stride) * 4, g[u]);
      if constexpr (HAS_RES) Pack<float>::load(dres + (i + u * stride) * 4, r[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float local = g[u][e] * gelu_grad1(a[u][e]);
        if constexpr (HAS_RES) a[u][e] = r[u][e] + local;
        else a[u][e] = local;
      }
      Pack<float>::store(dx + (i + u * stride) * 4, a[u]);
    }
  }
  __device__ __forceinline__ void scalar(int64_t j) {
    const float local = dy[j] * gelu_grad1(x[j]);
    dx[j] = HAS_RES ? dres[j] + local : local;
  }
};

template <bool HAS_RES>
__global__ void __launch_bounds__(EW_THREADS) gelu_backward_kernel(GeluBwd<HAS_RES> f, int64_t n, int early) {
  ew_drive<4>(n, f, early);
}

// ---------------------------------------------------------------------------- SwiGLU
// backend.py:1117-1120: 1 / (exp(-g) + 1).  FAST: ex2-based __expf and the approximate reciprocal,
// relative error of the exponential (2 + 1.16 |g|) ulp, of the sigmoid at most a quarter of that
// (s (1 - s) damps it): below 5e-7 against the 1e-5 bound; the vector kernels use it for both storage
// types (with the accurate expf and the rounded reciprocal they were issue-bound).  FAST=false:
// accurate expf and a correctly rounded reciprocal (bit-identical to the IEEE division 1/x).
template <bool FAST>
__device__ __forceinline__ float sigmoid_ref(float g) {
  if (FAST) return __fdividef(1.0f, __expf(-g) + 1.0f);
  return __frcp_rn(expf(-g) + 1.0f);
}

// Position (row, packet in row) of a packet index that advances by a fixed step.
struct RowWalk {
  int64_t row, drow;
  int col, dcol;
  __device__ __forceinline__ void init(int64_t p, int ppr, int64_t step_packets) {
    row = p / ppr;
    col = (int)(p - row * ppr);
    drow = step_packets / ppr;
    dcol = (int)(step_packets - drow * ppr);
  }
  __device__ __forceinline__ void step(int ppr) {
    row += drow;
    col += dcol;
    if (col >= ppr) {
      col -= ppr;
      ++row;
    }
  }
};

// One thread handles packets of the same column range in the gate and up halves of a row.  Packets stay
// as loaded (16 bytes = 4 registers) until they are used, so that bf16 storage, whose packets widen to 8
// floats, can keep four packet pairs in flight per thread instead of two at the same register count.
template <typename T>
__global__ void __launch_bounds__(EW_THREADS) swiglu_forward_kernel(const T* __restrict__ gu, T* __restrict__ hidden,
                                                                    int64_t N, int I, int early) {
  ag_pdl_wait();
  if (early) ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  constexpr int K = NV == 8 ? 4 : 2;  // packet pairs in flight per thread
  const int ppr = I / NV;  // packets per row (I % NV == 0 on this path)
  const int64_t packets = N * (int64_t)ppr;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // (row, packet-in-row) of the packets of an iteration advance by a fixed step: one 64-bit
  // division per thread instead of one per packet (they would cost as much as the activation)
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  RowWalk w[K];
#pragma unroll
  for (int k = 0; k < K; ++k) w[k].init(i0 + k * stride, ppr, K * stride);
  for (int64_t i = i0; i < packets; i += K * stride) {
    typename Pack<T>::Raw g[K], u[K];
    bool live[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int64_t p = i + k * stride;
      live[k] = p < packets;
      if (live[k]) {
        const int64_t row = w[k].row;
        const int col = w[k].col * NV;
        g[k] = Pack<T>::load_raw_stream(gu + row * 2 * I + col);
        u[k] = Pack<T>::load_raw_stream(gu + row * 2 * I + I + col);
      }
      w[k].step(ppr);
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (live[k]) {
        float gv[NV], uv[NV];
        Pack<T>::unpack_raw(g[k], gv);
        Pack<T>::unpack_raw(u[k], uv);
#pragma unroll
        for (int e = 0; e < NV; ++e) gv[e] = (gv[e] * sigmoid_ref<true>(gv[e])) * uv[e];
        Pack<T>::store(hidden + (i + k * stride) * NV, gv);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS) swiglu_forward_scalar_kernel(const T* __restrict__ gu,
                                                                           T* __restrict__ hidden, int64_t N, int I) {
  const int64_t total = N * (int64_t)I;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / I;
    const int col = (int)(i - row * I);
    const float g = Pack<T>::load1(gu + row * 2 * I + col);
    const float u = Pack<T>::load1(gu + row * 2 * I + I + col);
    Pack<T>::store1(hidden + i, (g * sigmoid_ref<false>(g)) * u);
  }
}

template <bool FAST>
__device__ __forceinline__ void swiglu_bwd1(float g, float u, float dh, float& dg, float& du) {
  // backend.py:1202-1217
  const float s = sigmoid_ref<FAST>(g);
  float t = 1.0f - s;
  t = t * g;
  t = t + 1.0f;
  t = t * s;
  t = t * u;
  dg = t * dh;
  du = (g * s) * dh;
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS) swiglu_backward_kernel(T* __restrict__ gu, const T* __restrict__ dh,
                                                                     int64_t N, int I, int early) {
  ag_pdl_wait();
  if (early) ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  constexpr int K = NV == 8 ? 4 : 2;  // packet triples (gate, up, dh) in flight per thread, kept as loaded
  const int ppr = I / NV;
  const int64_t packets = N * (int64_t)ppr;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  RowWalk w[K];
#pragma unroll
  for (int k = 0; k < K; ++k) w[k].init(i0 + k * stride, ppr, K * stride);
  for (int64_t i = i0; i < packets; i += K * stride) {
    typename Pack<T>::Raw g[K], u[K], d[K];
    bool live[K];
    int64_t goff[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int64_t p = i + k * stride;
      live[k] = p < packets;
      if (live[k]) {
        goff[k] = w[k].row * 2 * I + w[k].col * NV;
        g[k] = Pack<T>::load_raw(gu + goff[k]);
        u[k] = Pack<T>::load_raw(gu + goff[k] + I);
        d[k] = Pack<T>::load_raw_stream(dh + p * NV);
      }
      w[k].step(ppr);
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (live[k]) {
        float gv[NV], uv[NV], dv[NV];
        Pack<T>::unpack_raw(g[k], gv);
        Pack<T>::unpack_raw(u[k], uv);
        Pack<T>::unpack_raw(d[k], dv);
#pragma unroll
        for (int e = 0; e < NV; ++e) {
          float dg, du;
          swiglu_bwd1<true>(gv[e], uv[e], dv[e], dg, du);
          gv[e] = dg;
          uv[e] = du;
        }
        Pack<T>::store(gu + goff[k], gv);
        Pack<T>::store(gu + goff[k] + I, uv);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS) swiglu_backward_scalar_kernel(T* __restrict__ gu,
                                                                            const T* __restrict__ dh, int64_t N,
                                                                            int I) {
  const int64_t total = N * (int64_t)I;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / I;
    const int col = (int)(i - row * I);
    T* pg = gu + row * 2 * I + col;
    const float g = Pack<T>::load1(pg);
    const float u = Pack<T>::load1(pg + I);
    float dg, du;
    swiglu_bwd1<false>(g, u, Pack<T>::load1(dh + i), dg, du);
    Pack<T>::store1(pg, dg);
    Pack<T>::store1(pg + I, du);
  }
}

// ---------------------------------------------------------------------------- AdamW
// GT = float, or uint16_t for gradients stored as bf16 bit patterns (the reference's
// grad_dtype="bf16" storage, backend.py:5128-5140: the kernel widens g before anything else).
template <typename GT>
struct AdamW {
  float* p;
  const GT* g;
  float* m;
  float* v;
  float lr_wd, lr_t, b1, b2, one_minus_b1, one_minus_b2, eps, grad_scale;
  bool decay;
  __device__ __forceinline__ void one(float& pp, float gg, float& mm, float& vv) const {
    // backend.py:2021-2038, statement order kept
    gg = gg * grad_scale;
    if (decay) pp = pp - pp * lr_wd;
    mm = mm * b1 + gg * one_minus_b1;
    vv = vv * b2 + (gg * gg) * one_minus_b2;
    pp = pp - (mm / (sqrtf(vv) + eps)) * lr_t;
  }
  template <int U>
  __device__ __forceinline__ void packets(int64_t i, int64_t stride) {
    float pv[U][4], gv[U][4], mv[U][4], vv[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t o = (i + u * stride) * 4;
      Pack<float>::load(p + o, pv[u]);
      if constexpr (sizeof(GT) == 4) {
        Pack<float>::load_stream(reinterpret_cast<const float*>(g) + o, gv[u]);
      } else {
        const uint2 w = __ldcs(reinterpret_cast<const uint2*>(g + o));
        gv[u][0] = __uint_as_float(w.x << 16); gv[u][1] = __uint_as_float(w.x & 0xffff0000u);
        gv[u][2] = __uint_as_float(w.y << 16); gv[u][3] = __uint_as_float(w.y & 0xffff0000u);
      }
      Pack<float>::load(m + o, mv[u]);
      Pack<float>::load(v + o, vv[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t o = (i + u * stride) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) one(pv[u][e], gv[u][e], mv[u][e], vv[u][e]);
      Pack<float>::store(p + o, pv[u]);
      Pack<float>::store(m + o, mv[u]);
      Pack<float>::store(v + o, vv[u]);
    }
  }
  __device__ __forceinline__ void scalar(int64_t j) {
    float gg;
    if constexpr (sizeof(GT) == 4) gg = g[j];
    else gg = __uint_as_float((uint32_t)g[j] << 16);
    one(p[j], gg, m[j], v[j]);
  }
};

// Two packets of p, g, m, v per thread (eight loads in flight) rather than four: half the registers, so
// three CTAs share an SM instead of one and more bytes are in flight per SM.
template <typename GT>
__global__ void __launch_bounds__(EW_THREADS) adamw_kernel(AdamW<GT> f, int64_t n, int early) { ew_drive<4, 2>(n, f, early); }

// ------------------------------------------------------- fp32 <-> bf16 gradient storage
// Round to nearest, ties to even; Inf kept, NaN stays NaN after the cut (utils.py:20-27,
// metal_ops.metal:12010-12041).
__device__ __forceinline__ uint32_t bf16_bits_rne(float value) {
  const uint32_t bits = __float_as_uint(value);
  if ((bits & 0x7f800000u) == 0x7f800000u) return ((bits >> 16) | ((bits & 0x007fffffu) ? 0x0040u : 0u)) & 0xffffu;
  return ((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16) & 0xffffu;
}

// dst = bf16(src), or bf16(src + float(dst)) when accumulate: 8 elements per packet (two 16-byte loads,
// one 16-byte store)
// 32 bytes of fp32 per lane in one store (a whole sector; two 16-byte stores of a lane each fill half a
// sector per request): bf16 -> fp32 went from 47 to 41 us on 41.9 M elements.  The same width on the load
// side of fp32 -> bf16 measured slower (47 against 43 us) and is not used.  Needs a 32-byte aligned pointer.
__device__ __forceinline__ void st_v8_f32(float* p, const float (&v)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
               "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

struct F32ToBf16 {
  const float* src;
  uint16_t* dst;
  bool accumulate;
  template <int U>
  __device__ __forceinline__ void packets(int64_t i, int64_t stride) {
    float a[U][8];
    uint4 old[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t o = (i + u * stride) * 8;
      const float4 x = __ldcs(reinterpret_cast<const float4*>(src + o));
      const float4 y = __ldcs(reinterpret_cast<const float4*>(src + o + 4));
      a[u][0] = x.x; a[u][1] = x.y; a[u][2] = x.z; a[u][3] = x.w;
      a[u][4] = y.x; a[u][5] = y.y; a[u][6] = y.z; a[u][7] = y.w;
      if (accumulate) old[u] = *reinterpret_cast<const uint4*>(dst + o);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t o = (i + u * stride) * 8;
      if (accumulate) {
        const uint32_t w[4] = {old[u].x, old[u].y, old[u].z, old[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          a[u][2 * e] += __uint_as_float(w[e] << 16);
          a[u][2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
        }
      }
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) w[e] = bf16_bits_rne(a[u][2 * e]) | (bf16_bits_rne(a[u][2 * e + 1]) << 16);
      *reinterpret_cast<uint4*>(dst + o) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  __device__ __forceinline__ void scalar(int64_t j) {
    float v = src[j];
    if (accumulate) v += __uint_as_float((uint32_t)dst[j] << 16);
    dst[j] = (uint16_t)bf16_bits_rne(v);
  }
};

__global__ void __launch_bounds__(EW_THREADS) f32_to_bf16_kernel(F32ToBf16 f, int64_t n, int early) { ew_drive<8>(n, f, early); }

template <bool WIDE>
struct Bf16ToF32 {
  const uint16_t* src;
  float* dst;
  template <int U>
  __device__ __forceinline__ void packets(int64_t i, int64_t stride) {
    uint4 t[U];
#pragma unroll
    for (int u = 0; u < U; ++u) t[u] = __ldcs(reinterpret_cast<const uint4*>(src + (i + u * stride) * 8));
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t o = (i + u * stride) * 8;
      const uint32_t w[4] = {t[u].x, t[u].y, t[u].z, t[u].w};
      float v[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[2 * e] = __uint_as_float(w[e] << 16);
        v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
      }
      if constexpr (WIDE) {
        st_v8_f32(dst + o, v);
      } else {
        *reinterpret_cast<float4*>(dst + o) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + o + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    }
  }
  __device__ __forceinline__ void scalar(int64_t j) { dst[j] = __uint_as_float((uint32_t)src[j] << 16); }
};

template <bool WIDE>
__global__ void __launch_bounds__(EW_THREADS) bf16_to_f32_kernel(Bf16ToF32<WIDE> f, int64_t n, int early) { ew_drive<8>(n, f, early); }

template <typename... P>
bool all_aligned16(P... p) {
  return (ag_aligned16(p) && ...);
}

}  // namespace

// =========================================================================================
extern "C" int ag_add_forward(ag_ctx* ctx, const float* x, const float* y, float* out, int64_t n) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, x && y && out && n > 0, "ag_add_forward: null pointer or negative n");
  AG_REQUIRE(ctx, all_aligned16(x, y, out), "ag_add_forward: pointers must be 16-byte aligned");
  {
    const int grid = ew_grid(ctx, n / 4, 0);
    AG_LAUNCH_PDL(ctx, "add_forward_kernel", add_forward_kernel, grid, EW_THREADS, 0, AddFwd{x, y, out}, n, ew_early(ctx, grid));
  }
  return AG_OK;
}

extern "C" int ag_add_backward(ag_ctx* ctx, const float* g, float* xgrad, float* ygrad, int64_t n) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0 || (!xgrad && !ygrad)) return AG_OK;
  AG_REQUIRE(ctx, g && n > 0, "ag_add_backward: null g or negative n");
  AG_REQUIRE(ctx, all_aligned16(g, xgrad, ygrad), "ag_add_backward: pointers must be 16-byte aligned");
  {
    const int grid = ew_grid(ctx, n / 4, 0);
    AG_LAUNCH_PDL(ctx, "add_backward_kernel", add_backward_kernel, grid, EW_THREADS, 0, AddBwd{g, xgrad, ygrad}, n, ew_early(ctx, grid));
  }
  return AG_OK;
}

extern "C" int ag_gelu_forward(ag_ctx* ctx, const float* x, float* y, int64_t n) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, x && y && n > 0, "ag_gelu_forward: null pointer or negative n");
  AG_REQUIRE(ctx, all_aligned16(x, y), "ag_gelu_forward: pointers must be 16-byte aligned");
  {
    const int grid = ew_grid(ctx, n / 4, 0);
    AG_LAUNCH_PDL(ctx, "gelu_forward_kernel", gelu_forward_kernel, grid, EW_THREADS, 0, GeluFwd{x, y}, n, ew_early(ctx, grid));
  }
  return AG_OK;
}

extern "C" int ag_gelu_backward(ag_ctx* ctx, const float* x, const float* dy, const float* dres, float* dx,
                                int64_t n) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, x && dy && dx && n > 0, "ag_gelu_backward: null pointer or negative n");
  AG_REQUIRE(ctx, all_aligned16(x, dy, dres, dx), "ag_gelu_backward: pointers must be 16-byte aligned");
  {
    // One resident wave exactly (three CTAs per SM without the residual operand, two with it): a grid of eight
    // CTAs per SM ran as 2.67 waves, the last one a third empty (6.87 -> 6.57 ms per benchmark step, 49.8 ->
    // 48.5 us at 16384 x 1536).
    static int occ_res[AG_MAX_DEVICES] = {}, occ_plain[AG_MAX_DEVICES] = {};
    if (dres) {
      const int grid = ew_grid(ctx, n / 4, ew_resident(ctx, gelu_backward_kernel<true>, &occ_res[ag_dev_slot(ctx)]));
      AG_LAUNCH_PDL(ctx, "gelu_backward_kernel", gelu_backward_kernel<true>, grid, EW_THREADS, 0,
                    GeluBwd<true>{x, dy, dres, dx}, n, ew_early(ctx, grid));
    } else {
      const int grid = ew_grid(ctx, n / 4, ew_resident(ctx, gelu_backward_kernel<false>, &occ_plain[ag_dev_slot(ctx)]));
      AG_LAUNCH_PDL(ctx, "gelu_backward_kernel", gelu_backward_kernel<false>, grid, EW_THREADS, 0,
                    GeluBwd<false>{x, dy, dres, dx}, n, ew_early(ctx, grid));
    }
  }
  return AG_OK;
}

template <typename T>
static int swiglu_forward_t(ag_ctx* ctx, const void* gu, void* hidden, int64_t N, int I) {
  constexpr int NV = Pack<T>::N;
  if (I % NV == 0 && all_aligned16(gu, hidden)) {
    const int64_t packets = N * (int64_t)(I / NV);
    const int grid = ew_grid(ctx, packets * 2, NV > 4 ? 8 : 0);  // bf16 packets carry twice the arithmetic
    AG_LAUNCH_PDL(ctx, "swiglu_forward_kernel", swiglu_forward_kernel<T>, grid, EW_THREADS, 0, static_cast<const T*>(gu),
                  static_cast<T*>(hidden), N, I, ew_early(ctx, grid));
  } else {
    swiglu_forward_scalar_kernel<T><<<ew_grid(ctx, N * (int64_t)I, 8), EW_THREADS, 0, ctx->stream>>>(
        static_cast<const T*>(gu), static_cast<T*>(hidden), N, I);
    AG_LAUNCHED(ctx, "swiglu_forward_scalar_kernel");
  }
  return AG_OK;
}

template <typename T>
static int swiglu_backward_t(ag_ctx* ctx, void* gu, const void* dh, int64_t N, int I) {
  constexpr int NV = Pack<T>::N;
  if (I % NV == 0 && all_aligned16(gu, dh)) {
    const int64_t packets = N * (int64_t)(I / NV);
    const int grid = ew_grid(ctx, packets * 2, NV > 4 ? 8 : 0);
    AG_LAUNCH_PDL(ctx, "swiglu_backward_kernel", swiglu_backward_kernel<T>, grid, EW_THREADS, 0, static_cast<T*>(gu),
                  static_cast<const T*>(dh), N, I, ew_early(ctx, grid));
  } else {
    swiglu_backward_scalar_kernel<T><<<ew_grid(ctx, N * (int64_t)I, 8), EW_THREADS, 0, ctx->stream>>>(
        static_cast<T*>(gu), static_cast<const T*>(dh), N, I);
    AG_LAUNCHED(ctx, "swiglu_backward_scalar_kernel");
  }
  return AG_OK;
}

extern "C" int ag_swiglu_forward(ag_ctx* ctx, const void* gu, void* hidden, int64_t N, int I, int dtype) {
  if (!ctx) return AG_ERR_INVALID;
  if (N == 0 || I == 0) return AG_OK;
  AG_REQUIRE(ctx, gu && hidden && N > 0 && I > 0, "ag_swiglu_forward: null pointer or negative size");
  AG_REQUIRE(ctx, dtype == AG_F32 || dtype == AG_BF16, "ag_swiglu_forward: unknown dtype %d", dtype);
  return dtype == AG_F32 ? swiglu_forward_t<float>(ctx, gu, hidden, N, I)
                         : swiglu_forward_t<__nv_bfloat16>(ctx, gu, hidden, N, I);
}

extern "C" int ag_swiglu_backward(ag_ctx* ctx, void* gu, const void* dhidden, int64_t N, int I, int dtype) {
  if (!ctx) return AG_ERR_INVALID;
  if (N == 0 || I == 0) return AG_OK;
  AG_REQUIRE(ctx, gu && dhidden && N > 0 && I > 0, "ag_swiglu_backward: null pointer or negative size");
  AG_REQUIRE(ctx, dtype == AG_F32 || dtype == AG_BF16, "ag_swiglu_backward: unknown dtype %d", dtype);
  return dtype == AG_F32 ? swiglu_backward_t<float>(ctx, gu, dhidden, N, I)
                         : swiglu_backward_t<__nv_bfloat16>(ctx, gu, dhidden, N, I);
}

namespace {
template <typename GT>
int adamw_launch(ag_ctx* ctx, float* p, const GT* g, float* m, float* v, int64_t n, double lr, double lr_t, double b1,
                 double b2, double eps, double weight_decay, double grad_scale) {
  AdamW<GT> f;
  f.p = p; f.g = g; f.m = m; f.v = v;
  // the reference multiplies fp32 arrays by python doubles: the scalar expression is
  // evaluated in double, then rounded once to fp32 (backend.py:2022, :2026, :2031)
  f.lr_wd = (float)(lr * weight_decay);
  f.lr_t = (float)lr_t; f.b1 = (float)b1; f.b2 = (float)b2;
  f.one_minus_b1 = (float)(1.0 - b1);
  f.one_minus_b2 = (float)(1.0 - b2);
  f.eps = (float)eps; f.grad_scale = (float)grad_scale;
  f.decay = weight_decay > 0.0;
  const int grid = ew_grid(ctx, n / 4, 8);
  AG_LAUNCH_PDL(ctx, "adamw_kernel", adamw_kernel<GT>, grid, EW_THREADS, 0, f, n, ew_early(ctx, grid));
  return AG_OK;
}
}  // namespace

extern "C" int ag_adamw_step(ag_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, double lr,
                             double lr_t, double b1, double b2, double eps, double weight_decay,
                             double grad_scale) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, p && g && m && v && n > 0, "ag_adamw_step: null pointer or negative n");
  AG_REQUIRE(ctx, all_aligned16(p, g, m, v), "ag_adamw_step: pointers must be 16-byte aligned");
  return adamw_launch<float>(ctx, p, g, m, v, n, lr, lr_t, b1, b2, eps, weight_decay, grad_scale);
}

extern "C" int ag_adamw_step_bf16grad(ag_ctx* ctx, float* p, const uint16_t* g, float* m, float* v, int64_t n,
                                      double lr, double lr_t, double b1, double b2, double eps,
                                      double weight_decay, double grad_scale) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, p && g && m && v && n > 0, "ag_adamw_step_bf16grad: null pointer or negative n");
  AG_REQUIRE(ctx, all_aligned16(p, g, m, v), "ag_adamw_step_bf16grad: pointers must be 16-byte aligned");
  return adamw_launch<uint16_t>(ctx, p, g, m, v, n, lr, lr_t, b1, b2, eps, weight_decay, grad_scale);
}

extern "C" int ag_f32_to_bf16(ag_ctx* ctx, const float* src, uint16_t* dst, int64_t n, int accumulate) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, src && dst && n > 0, "ag_f32_to_bf16: null pointer or negative n");
  AG_REQUIRE(ctx, all_aligned16(src, dst), "ag_f32_to_bf16: pointers must be 16-byte aligned");
  const int grid = ew_grid(ctx, n / 8, 0);
  F32ToBf16 f{src, dst, accumulate != 0};
  AG_LAUNCH_PDL(ctx, "f32_to_bf16_kernel", f32_to_bf16_kernel, grid, EW_THREADS, 0, f, n, ew_early(ctx, grid));
  return AG_OK;
}

extern "C" int ag_bf16_to_f32(ag_ctx* ctx, const uint16_t* src, float* dst, int64_t n) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, src && dst && n > 0, "ag_bf16_to_f32: null pointer or negative n");
  AG_REQUIRE(ctx, all_aligned16(src, dst), "ag_bf16_to_f32: pointers must be 16-byte aligned");
  const int grid = ew_grid(ctx, n / 8, 0);
  if ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
    Bf16ToF32<true> f{src, dst};
    AG_LAUNCH_PDL(ctx, "bf16_to_f32_kernel", bf16_to_f32_kernel<true>, grid, EW_THREADS, 0, f, n, ew_early(ctx, grid));
  } else {
    Bf16ToF32<false> f{src, dst};
    AG_LAUNCH_PDL(ctx, "bf16_to_f32_kernel", bf16_to_f32_kernel<false>, grid, EW_THREADS, 0, f, n, ew_early(ctx, grid));
  }
  return AG_OK;
}
