// Rotate-half RoPE applied in place to q (B,T,H,D) and k (B,T,HKV,D).
//
// Work item = (token, group of four heads, 16-byte packet of the low half).  A thread loads the cos/sin
// entries of its packet once and applies them to the matching packets of up to four heads (q heads
// first, then k heads): the table traffic per data byte is a quarter of one lookup per head, which
// matters for bf16 storage, where a 16-byte data packet needs 64 bytes of fp32 table entries.  Both
// halves of a head are read once and written once; all loads of a thread (eight packets and the
// table entries) are issued in one burst before the first store: there is no shared-memory stage and
// no barrier.  Consecutive threads take consecutive packets of one head half (256 / 128 contiguous
// bytes at head_dim 128).  Shapes where D/2 is not a multiple of the packet width use a scalar kernel.
#include "ag_common.cuh"

namespace {

constexpr int ROPE_THREADS = 256;
constexpr int ROPE_HEADS = 4;  // heads per work item

template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kernel(T* q, T* k, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int64_t tokens, int T_len,
            int H, int HKV, int D, int64_t q_stride, int64_t k_stride, float sgn) {
  ag_pdl_wait();
  ag_pdl_trigger();
  constexpr int NV = Pack<T>::N;
  const int d2 = D >> 1;
  const int ppd = d2 / NV;                                  // packets per half head
  const int groups = (H + HKV + ROPE_HEADS - 1) / ROPE_HEADS;
  const int64_t total = tokens * groups * ppd;              // work items, token-major
  const int64_t g = (int64_t)blockIdx.x * ROPE_THREADS + threadIdx.x;
  if (g >= total) return;
  const int col = (int)(g % ppd) * NV;
  const int64_t rest = g / ppd;
  const int group = (int)(rest % groups);
  const int64_t tok = rest / groups;
  const int t = (int)(tok % T_len);
  typename Pack<T>::Raw lo[ROPE_HEADS], hi[ROPE_HEADS];  // kept as loaded: bf16 packets are widened one head at a time
  float c[NV], s[NV];
  T* ptr[ROPE_HEADS];
#pragma unroll
  for (int u = 0; u < ROPE_HEADS; ++u) {
    const int head = group * ROPE_HEADS + u;
    ptr[u] = nullptr;
    if (head < H + HKV) {
      T* hp = head < H ? q + tok * q_stride + (int64_t)head * D : k + tok * k_stride + (int64_t)(head - H) * D;
      ptr[u] = hp + col;
      lo[u] = Pack<T>::load_raw(ptr[u]);
      hi[u] = Pack<T>::load_raw(ptr[u] + d2);
    }
  }
  {
    const float* crow = cos_tab + (int64_t)t * d2 + col;   // L2-resident tables (T * D/2 floats)
    const float* srow = sin_tab + (int64_t)t * d2 + col;
#pragma unroll
    for (int e = 0; e < NV; e += 4) {
      const float4 cv = __ldg(reinterpret_cast<const float4*>(crow + e));
      const float4 sv = __ldg(reinterpret_cast<const float4*>(srow + e));
      c[e] = cv.x; c[e + 1] = cv.y; c[e + 2] = cv.z; c[e + 3] = cv.w;
      s[e] = sgn * sv.x; s[e + 1] = sgn * sv.y; s[e + 2] = sgn * sv.z; s[e + 3] = sgn * sv.w;
    }
  }
#pragma unroll
  for (int u = 0; u < ROPE_HEADS; ++u) {
    if (ptr[u]) {
      float vlo[NV], vhi[NV], olo[NV], ohi[NV];
      Pack<T>::unpack_raw(lo[u], vlo);
      Pack<T>::unpack_raw(hi[u], vhi);
#pragma unroll
      for (int e = 0; e < NV; ++e) {
        // sgn=+1: lo*c - hi*s , lo*s + hi*c   (backend.py:1413-1414)
        // sgn=-1: lo*c + hi*s , -lo*s + hi*c  (backend.py:1396-1397)
        olo[e] = vlo[e] * c[e] - vhi[e] * s[e];
        ohi[e] = vlo[e] * s[e] + vhi[e] * c[e];
      }
      Pack<T>::store(ptr[u], olo);
      Pack<T>::store(ptr[u] + d2, ohi);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_scalar_kernel(T* q, T* k, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int T_len, int H,
                   int HKV, int D, int64_t q_stride, int64_t k_stride, float sgn) {
  const int d2 = D >> 1;
  const int64_t tok = blockIdx.x;
  const int t = (int)(tok % T_len);
  const int items = (H + HKV) * d2;
  for (int it = threadIdx.x; it < items; it += ROPE_THREADS) {
    const int head = it / d2;
    const int c0 = it - head * d2;
    T* hp = head < H ? q + tok * q_stride + (int64_t)head * D : (k ? k + tok * k_stride + (int64_t)(head - H) * D : nullptr);
    if (!hp) continue;
    const float c = cos_tab[(int64_t)t * d2 + c0];
    const float s = sgn * sin_tab[(int64_t)t * d2 + c0];
    const float lo = Pack<T>::load1(hp + c0), hi = Pack<T>::load1(hp + c0 + d2);
    Pack<T>::store1(hp + c0, lo * c - hi * s);
    Pack<T>::store1(hp + c0 + d2, lo * s + hi * c);
  }
}

template <typename T>
int rope_t(ag_ctx* ctx, void* qv, void* kv, const float* cos_tab, const float* sin_tab, int B, int T_len, int H,
           int HKV, int D, int64_t qs, int64_t ks, int sin_sign) {
  constexpr int NV = Pack<T>::N;
  T* q = static_cast<T*>(qv);
  T* k = static_cast<T*>(kv);
  const int d2 = D / 2;
  const int64_t tokens = (int64_t)B * T_len;
  const float sgn = sin_sign >= 0 ? 1.0f : -1.0f;
  const bool vec_ok = (d2 % NV == 0) && ag_aligned16(q) && ag_aligned16(k) && (qs % NV == 0) && (ks % NV == 0) &&
                      ag_aligned16(cos_tab) && ag_aligned16(sin_tab);
  if (vec_ok) {
    const int hkv = k ? HKV : 0;
    const int64_t total = tokens * (int64_t)((H + hkv + ROPE_HEADS - 1) / ROPE_HEADS) * (d2 / NV);
    AG_LAUNCH_PDL(ctx, "rope_kernel", rope_kernel<T>, (unsigned)((total + ROPE_THREADS - 1) / ROPE_THREADS), ROPE_THREADS, 0, q, k,
                  cos_tab, sin_tab, tokens, T_len, H, hkv, D, qs, ks, sgn);
  } else {
    rope_scalar_kernel<T><<<(unsigned)tokens, ROPE_THREADS, 0, ctx->stream>>>(q, k, cos_tab, sin_tab, T_len, H,
                                                                              k ? HKV : 0, D, qs, ks, sgn);
    AG_LAUNCHED(ctx, "rope_scalar_kernel");
  }
  return AG_OK;
}

}  // namespace

extern "C" int ag_rope_qk(ag_ctx* ctx, void* q, void* k, const float* cos_tab, const float* sin_tab, int B, int T,
                          int H, int HKV, int D, int64_t q_token_stride, int64_t k_token_stride, int sin_sign,
                          int dtype) {
  if (!ctx) return AG_ERR_INVALID;
  if (B == 0 || T == 0) return AG_OK;
  AG_REQUIRE(ctx, q && cos_tab && sin_tab, "ag_rope_qk: null pointer");
  AG_REQUIRE(ctx, B > 0 && T > 0 && H > 0 && D > 0 && (D % 2) == 0 && (k == nullptr || HKV > 0),
             "ag_rope_qk: bad shape B=%d T=%d H=%d HKV=%d D=%d", B, T, H, HKV, D);
  AG_REQUIRE(ctx, dtype == AG_F32 || dtype == AG_BF16, "ag_rope_qk: unknown dtype %d", dtype);
  AG_REQUIRE(ctx, q_token_stride >= (int64_t)H * D && (k == nullptr || k_token_stride >= (int64_t)HKV * D),
             "ag_rope_qk: token stride smaller than heads*D");
  AG_REQUIRE(ctx, (int64_t)B * T < (1ll << 31), "ag_rope_qk: too many tokens");
  AG_REQUIRE(ctx, D <= 8192, "ag_rope_qk: D=%d too large", D);
  return dtype == AG_F32
             ? rope_t<float>(ctx, q, k, cos_tab, sin_tab, B, T, H, HKV, D, q_token_stride, k_token_stride, sin_sign)
             : rope_t<__nv_bfloat16>(ctx, q, k, cos_tab, sin_tab, B, T, H, HKV, D, q_token_stride, k_token_stride,
                                     sin_sign);
}
