// Shared declarations of the sm_100a kernels: context object, error plumbing, 16-byte
// vector access, warp reductions and the bounded mbarrier / bulk-copy helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "autograd_b200.h"

struct ag_ctx {
  int device;
  cudaStream_t stream;
  bool own_stream;
  int sm_count;
  int cc_major, cc_minor;
  size_t l2_bytes;
  size_t total_bytes;
  int* d_status;  // device status word (AG_STATUS_* bits), set by kernels with atomicOr
  int* h_status;  // pinned mirror
  cudaEvent_t ev_begin, ev_end;
  cudaEvent_t* ev_pool;  // ag_event_record / ag_event_elapsed
  int ev_pool_size;
  int64_t launches;
  int pdl;              // 1: kernels are launched with programmatic stream serialization
  int tc_pair;          // 1: the split-operand tensor-core GEMMs run on CTA pairs (cta_group::2)
  int norm_ring;        // norm kernels stream rows through a shared-memory ring: 0 never, 1 always, 2 per shape
  int norm_pair;        // norm backward with two warps per row: 0 never, 1 always, 2 per shape
  int scatter_group;    // sorted entries per group of the scatter-add: 32, 64, or 0 = by the number of ids
  int debug_stage_expire;  // ag_debug_expire_staging: the next staging wait gives up at once (tests)
  int linear_k_chunk;   // contraction elements per accumulation chain, forward of the linear+bias+residual op
  int tc_timing;        // ag_tc_timing: bracket tensor-core GEMM launches with pool events
  int tc_timing_base;
  int tc_timing_count;
  char err[512];
};

#define AG_FAIL(ctx, code, ...)                                \
  do {                                                         \
    snprintf((ctx)->err, sizeof((ctx)->err), __VA_ARGS__);     \
    return (code);                                             \
  } while (0)

#define AG_CUDA(ctx, call)                                                                    \
  do {                                                                                        \
    cudaError_t e_ = (call);                                                                  \
    if (e_ != cudaSuccess)                                                                    \
      AG_FAIL(ctx, AG_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, \
              __LINE__);                                                                      \
  } while (0)

#define AG_REQUIRE(ctx, cond, ...)                        \
  do {                                                    \
    if (!(cond)) AG_FAIL(ctx, AG_ERR_INVALID, __VA_ARGS__); \
  } while (0)

// To be called right after a kernel launch.
#define AG_LAUNCHED(ctx, name)                                                              \
  do {                                                                                      \
    cudaError_t e_ = cudaGetLastError();                                                    \
    if (e_ != cudaSuccess)                                                                  \
      AG_FAIL(ctx, AG_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e_));  \
    (ctx)->launches++;                                                                      \
  } while (0)

// Launch with programmatic stream serialization: the grid may be scheduled while the tail of the
// previous kernel of the stream is still running, which hides the launch latency of short kernels.
// A kernel launched this way must execute ag_pdl_wait() before its first access to global memory
// (it returns once every earlier grid has completed and its writes are visible) and should execute
// ag_pdl_trigger() early so that its own successor can be scheduled in the same way.
#define AG_LAUNCH_PDL(ctx, name, kern, grid, block, smem, ...)                                  \
  do {                                                                                          \
    cudaLaunchConfig_t cfg_ = {};                                                               \
    cfg_.gridDim = (grid);                                                                      \
    cfg_.blockDim = (block);                                                                    \
    cfg_.dynamicSmemBytes = (smem);                                                             \
    cfg_.stream = (ctx)->stream;                                                                \
    cudaLaunchAttribute at_[1];                                                                 \
    at_[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                             \
    at_[0].val.programmaticStreamSerializationAllowed = 1;                                      \
    cfg_.attrs = at_;                                                                           \
    cfg_.numAttrs = (ctx)->pdl ? 1 : 0;                                                         \
    cudaError_t e_ = cudaLaunchKernelEx(&cfg_, kern, __VA_ARGS__);                              \
    if (e_ != cudaSuccess)                                                                      \
      AG_FAIL(ctx, AG_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e_));      \
    (ctx)->launches++;                                                                          \
  } while (0)

#ifdef __CUDACC__
__device__ __forceinline__ void ag_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ag_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// Per-device slots of the small host-side caches (function attributes and occupancy are per device).
constexpr int AG_MAX_DEVICES = 64;
static inline int ag_dev_slot(const ag_ctx* ctx) { return ctx->device >= 0 && ctx->device < AG_MAX_DEVICES ? ctx->device : 0; }

static inline bool ag_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline int ag_ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// ---------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float ag_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float ag_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 16-byte packets of activations: 4 fp32 or 8 bf16, always widened to fp32 registers.
template <typename T>
struct Pack;

template <>
struct Pack<float> {
  static constexpr int N = 4;
  // a packet as it lies in memory, for kernels that keep many packets in flight before widening them
  using Raw = float4;
  __device__ __forceinline__ static Raw load_raw(const float* p) { return *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ static Raw load_raw_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
  __device__ __forceinline__ static void unpack_raw(const Raw& t, float (&v)[4]) {
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ __forceinline__ static void load(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  // streaming variant for data that is read exactly once
  __device__ __forceinline__ static void load_stream(const float* p, float (&v)[4]) {
    float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ __forceinline__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  __device__ __forceinline__ static void store_stream(float* p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
  __device__ __forceinline__ static float load1(const float* p) { return *p; }
  __device__ __forceinline__ static void store1(float* p, float v) { *p = v; }
};

template <>
struct Pack<__nv_bfloat16> {
  static constexpr int N = 8;
  using Raw = uint4;
  __device__ __forceinline__ static Raw load_raw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ static Raw load_raw_stream(const __nv_bfloat16* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
  }
  __device__ __forceinline__ static void unpack_raw(const Raw& t, float (&v)[8]) { unpack(t, v); }
  __device__ __forceinline__ static void unpack(const uint4& t, float (&v)[8]) {
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static uint4 pack(const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // round-to-nearest-even, the reference's bf16 storage rule (utils.py:20-27)
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    unpack(*reinterpret_cast<const uint4*>(p), v);
  }
  __device__ __forceinline__ static void load_stream(const __nv_bfloat16* p, float (&v)[8]) {
    unpack(__ldcs(reinterpret_cast<const uint4*>(p)), v);
  }
  __device__ __forceinline__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(p) = pack(v);
  }
  __device__ __forceinline__ static void store_stream(__nv_bfloat16* p, const float (&v)[8]) {
    __stcs(reinterpret_cast<uint4*>(p), pack(v));
  }
  __device__ __forceinline__ static float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ __forceinline__ static void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// ---- mbarrier + bulk (TMA 1-D) copy, every wait bounded ---------------------------------
__device__ __forceinline__ uint32_t ag_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ag_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ag_smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void ag_fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void ag_fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void ag_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ag_smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void ag_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ag_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool ag_mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(ag_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Spins at most `limit` polls.  Returns false when the limit was hit; the caller must
// then raise AG_STATUS_WAIT_EXPIRED and unwind without touching the awaited data.
__device__ __forceinline__ bool ag_mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (ag_mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
  }
  return false;
}

// 1-D bulk copy global -> shared (TMA engine).  dst, src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void ag_bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          ag_smem_u32(dst_smem)),
      "l"(src), "r"(bytes), "r"(ag_smem_u32(bar))
      : "memory");
}

// Ask the copy engine to pull `bytes` (multiple of 16, 16-byte aligned) into L2; no registers or
// shared memory are tied up and nothing waits on it.
__device__ __forceinline__ void ag_prefetch_l2_bulk(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Stage up to two fp32 vectors of n floats each (src1 may be null) into shared memory
// through the bulk-copy engine when alignment allows, else with plain loads.  Called by all
// threads of the CTA; returns after a __syncthreads() with the data visible.
// `bar` must point to an 8-byte aligned uint64_t in shared memory used for nothing else.
// `poll_limit` bounds the wait for the copy; when it runs out the CTA records
// AG_STATUS_STAGE_FALLBACK, gives the copy that is still in flight a second bounded wait to
// land (nothing may write this CTA's shared memory behind its back) and fills the vectors with
// plain loads.  A limit of 0 takes that path at once (used by the tests).
__device__ __forceinline__ void ag_stage_vectors(float* dst0, const float* src0, float* dst1, const float* src1,
                                                 int n, uint64_t* bar, int* status, uint32_t poll_limit = 1u << 20) {
  const uint32_t bytes = (uint32_t)n * 4u;
  const bool bulk_ok = (bytes % 16u == 0) && ((reinterpret_cast<uintptr_t>(src0) & 15u) == 0) &&
                       (src1 == nullptr || (reinterpret_cast<uintptr_t>(src1) & 15u) == 0) &&
                       ((ag_smem_u32(dst0) & 15u) == 0) && (src1 == nullptr || (ag_smem_u32(dst1) & 15u) == 0);
  bool done = false;
  if (bulk_ok) {
    if (threadIdx.x == 0) {
      ag_mbar_init(bar, 1);
      ag_fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      ag_mbar_expect_tx(bar, bytes * (src1 ? 2u : 1u));
      ag_bulk_g2s(dst0, src0, bytes, bar);
      if (src1) ag_bulk_g2s(dst1, src1, bytes, bar);
    }
    done = ag_mbar_wait_bounded(bar, 0, poll_limit);
    // all threads agree on the outcome
    done = __syncthreads_and(done ? 1 : 0) != 0;
    if (!done) {
      if (threadIdx.x == 0) {
        atomicOr(status, AG_STATUS_STAGE_FALLBACK);
        if (!ag_mbar_wait_bounded(bar, 0, 1u << 20)) atomicOr(status, AG_STATUS_WAIT_EXPIRED);
      }
      __syncthreads();
    }
  }
  if (!done) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      dst0[i] = src0[i];
      if (src1) dst1[i] = src1[i];
    }
    __syncthreads();
  }
}

#endif  // __CUDACC__
