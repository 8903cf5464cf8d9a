// Context, memory, copies, fills, event timing: the typed CUDA counterpart of the
// reference's MetalContext (metal_ext.mm:770-796).  One context = one device + one stream;
// every kernel of this library is enqueued on that stream in call order.
#include "ag_common.cuh"

#include <stdlib.h>
#include <string.h>

static thread_local char g_create_err[512] = "";

extern "C" const char* ag_last_error(const ag_ctx* ctx) { return ctx ? ctx->err : g_create_err; }

extern "C" int ag_ctx_create(int device, void* stream, ag_ctx** out) {
  if (!out) {
    snprintf(g_create_err, sizeof g_create_err, "ag_ctx_create: out is NULL");
    return AG_ERR_INVALID;
  }
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || device < 0 || device >= count) {
    snprintf(g_create_err, sizeof g_create_err, "ag_ctx_create: no CUDA device %d (%d visible%s%s)", device, count,
             e != cudaSuccess ? ": " : "", e != cudaSuccess ? cudaGetErrorString(e) : "");
    return AG_ERR_CUDA;
  }
  ag_ctx* c = new ag_ctx();
  memset(c, 0, sizeof *c);
  c->device = device;
#define CREATE_CUDA(call)                                                                     \
  do {                                                                                        \
    cudaError_t e2 = (call);                                                                  \
    if (e2 != cudaSuccess) {                                                                  \
      snprintf(g_create_err, sizeof g_create_err, "%s failed: %s", #call, cudaGetErrorString(e2)); \
      delete c;                                                                               \
      return AG_ERR_CUDA;                                                                     \
    }                                                                                         \
  } while (0)
  CREATE_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  CREATE_CUDA(cudaGetDeviceProperties(&prop, device));
  c->sm_count = prop.multiProcessorCount;
  c->cc_major = prop.major;
  c->cc_minor = prop.minor;
  c->l2_bytes = (size_t)prop.l2CacheSize;
  c->total_bytes = prop.totalGlobalMem;
  if (prop.major != 10) {
    snprintf(g_create_err, sizeof g_create_err,
             "ag_ctx_create: device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major,
             prop.minor);
    delete c;
    return AG_ERR_INVALID;
  }
  if (stream) {
    c->stream = (cudaStream_t)stream;
    c->own_stream = false;
  } else {
    CREATE_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    c->own_stream = true;
  }
  {
    // AG_B200_PDL=0 launches every kernel fully serialized (diagnostics)
    const char* e = getenv("AG_B200_PDL");
    c->pdl = (e && e[0] == '0') ? 0 : 1;
    // AG_B200_TC_PAIR=0 runs the tensor-core GEMMs on single CTAs (diagnostics)
    e = getenv("AG_B200_TC_PAIR");
    c->tc_pair = (e && e[0] == '0') ? 0 : 1;
    // AG_B200_NORM_RING: 0 = rows in registers everywhere, 1 = the shared-memory row ring wherever the
    // shape fits, unset = the measured choice per shape (diagnostics, A/B measurements)
    e = getenv("AG_B200_NORM_RING");
    c->norm_ring = !e ? 2 : (e[0] == '0' ? 0 : 1);
    c->debug_stage_expire = 0;
    // AG_B200_NORM_PAIR: norm backward with two warps per row: 0 never, 1 whenever the shape fits, unset =
    // fp32 rows of 1024 columns and more (diagnostics, A/B measurements)
    e = getenv("AG_B200_NORM_PAIR");
    c->norm_pair = !e ? 2 : (e[0] == '0' ? 0 : 1);
    // AG_B200_SCATTER_GROUP: 32, 64 or 128 sorted entries per group of the scatter-add; unset = by the number of ids
    e = getenv("AG_B200_SCATTER_GROUP");
    c->scatter_group = 0;
    if (e && (atoi(e) == 32 || atoi(e) == 64 || atoi(e) == 128)) c->scatter_group = atoi(e);
    // AG_B200_LINEAR_K_CHUNK: longest tensor-core accumulation chain (contraction elements) in the forward
    // of the linear + bias + residual op; shorter chains = smaller error, more launches.  A multiple of 32.
    e = getenv("AG_B200_LINEAR_K_CHUNK");
    c->linear_k_chunk = 384;
    if (e) {
      const int v = atoi(e);
      if (v >= 64 && v % 32 == 0) c->linear_k_chunk = v;
    }
  }
  CREATE_CUDA(cudaMalloc(&c->d_status, sizeof(int)));
  CREATE_CUDA(cudaMemset(c->d_status, 0, sizeof(int)));
  CREATE_CUDA(cudaDeviceSynchronize());  // the memset ran on the default stream, the kernels use the context's own
  CREATE_CUDA(cudaMallocHost(&c->h_status, sizeof(int)));
  CREATE_CUDA(cudaEventCreate(&c->ev_begin));
  CREATE_CUDA(cudaEventCreate(&c->ev_end));
#undef CREATE_CUDA
  *out = c;
  return AG_OK;
}

extern "C" int ag_ctx_destroy(ag_ctx* ctx) {
  if (!ctx) return AG_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  cudaEventDestroy(ctx->ev_begin);
  cudaEventDestroy(ctx->ev_end);
  for (int i = 0; i < ctx->ev_pool_size; ++i) cudaEventDestroy(ctx->ev_pool[i]);
  free(ctx->ev_pool);
  cudaFree(ctx->d_status);
  cudaFreeHost(ctx->h_status);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return AG_OK;
}

extern "C" int ag_set_stream(ag_ctx* ctx, void* stream) {
  if (!ctx) return AG_ERR_INVALID;
  if (ctx->own_stream) {
    AG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    AG_CUDA(ctx, cudaStreamDestroy(ctx->stream));
    ctx->own_stream = false;
  }
  if (stream) {
    ctx->stream = (cudaStream_t)stream;
  } else {
    AG_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    ctx->own_stream = true;
  }
  return AG_OK;
}

extern "C" int ag_device_info(ag_ctx* ctx, int* sm_count, int64_t* l2_bytes, int64_t* total_bytes, int* cc_major,
                              int* cc_minor) {
  if (!ctx) return AG_ERR_INVALID;
  if (sm_count) *sm_count = ctx->sm_count;
  if (l2_bytes) *l2_bytes = (int64_t)ctx->l2_bytes;
  if (total_bytes) *total_bytes = (int64_t)ctx->total_bytes;
  if (cc_major) *cc_major = ctx->cc_major;
  if (cc_minor) *cc_minor = ctx->cc_minor;
  return AG_OK;
}

extern "C" int ag_alloc(ag_ctx* ctx, size_t bytes, void** out) {
  if (!ctx || !out) return AG_ERR_INVALID;
  *out = nullptr;
  if (bytes == 0) return AG_OK;
  AG_CUDA(ctx, cudaSetDevice(ctx->device));
  AG_CUDA(ctx, cudaMalloc(out, bytes));
  return AG_OK;
}

extern "C" int ag_free(ag_ctx* ctx, void* ptr) {
  if (!ctx) return AG_ERR_INVALID;
  if (!ptr) return AG_OK;
  AG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  AG_CUDA(ctx, cudaFree(ptr));
  return AG_OK;
}

extern "C" int ag_copy_h2d(ag_ctx* ctx, void* dst, const void* src, size_t bytes) {
  if (!ctx) return AG_ERR_INVALID;
  if (bytes == 0) return AG_OK;
  AG_REQUIRE(ctx, dst && src, "ag_copy_h2d: null pointer");
  AG_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return AG_OK;
}

extern "C" int ag_copy_d2h(ag_ctx* ctx, void* dst, const void* src, size_t bytes) {
  if (!ctx) return AG_ERR_INVALID;
  if (bytes == 0) return AG_OK;
  AG_REQUIRE(ctx, dst && src, "ag_copy_d2h: null pointer");
  AG_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  AG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return AG_OK;
}

extern "C" int ag_synchronize(ag_ctx* ctx) {
  if (!ctx) return AG_ERR_INVALID;
  AG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return AG_OK;
}

extern "C" int ag_status(ag_ctx* ctx, int* flags) {
  if (!ctx || !flags) return AG_ERR_INVALID;
  AG_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  AG_CUDA(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
  AG_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  *flags = *ctx->h_status;
  return AG_OK;
}

extern "C" int64_t ag_launch_count(const ag_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int ag_pass_begin_profiled(ag_ctx* ctx) {
  if (!ctx) return AG_ERR_INVALID;
  AG_CUDA(ctx, cudaEventRecord(ctx->ev_begin, ctx->stream));
  return AG_OK;
}

extern "C" int ag_pass_end_profiled(ag_ctx* ctx, float* ms) {
  if (!ctx || !ms) return AG_ERR_INVALID;
  AG_CUDA(ctx, cudaEventRecord(ctx->ev_end, ctx->stream));
  AG_CUDA(ctx, cudaEventSynchronize(ctx->ev_end));
  AG_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_begin, ctx->ev_end));
  return AG_OK;
}

extern "C" int ag_event_record(ag_ctx* ctx, int index) {
  if (!ctx) return AG_ERR_INVALID;
  AG_REQUIRE(ctx, index >= 0 && index < (1 << 22), "ag_event_record: bad index %d", index);
  if (index >= ctx->ev_pool_size) {
    int n = ctx->ev_pool_size ? ctx->ev_pool_size : 256;
    while (n <= index) n *= 2;
    cudaEvent_t* p = (cudaEvent_t*)realloc(ctx->ev_pool, sizeof(cudaEvent_t) * n);
    if (!p) AG_FAIL(ctx, AG_ERR_INVALID, "ag_event_record: out of host memory");
    ctx->ev_pool = p;
    for (int i = ctx->ev_pool_size; i < n; ++i) {
      cudaError_t e = cudaEventCreate(&ctx->ev_pool[i]);
      if (e != cudaSuccess) {
        ctx->ev_pool_size = i;
        AG_FAIL(ctx, AG_ERR_CUDA, "cudaEventCreate failed: %s", cudaGetErrorString(e));
      }
    }
    ctx->ev_pool_size = n;
  }
  AG_CUDA(ctx, cudaEventRecord(ctx->ev_pool[index], ctx->stream));
  return AG_OK;
}

extern "C" int ag_event_elapsed(ag_ctx* ctx, int start_index, int end_index, float* ms) {
  if (!ctx || !ms) return AG_ERR_INVALID;
  AG_REQUIRE(ctx, start_index >= 0 && end_index >= 0 && start_index < ctx->ev_pool_size && end_index < ctx->ev_pool_size,
             "ag_event_elapsed: event not recorded");
  AG_CUDA(ctx, cudaEventSynchronize(ctx->ev_pool[end_index]));
  AG_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_pool[start_index], ctx->ev_pool[end_index]));
  return AG_OK;
}

extern "C" int ag_tc_timing(ag_ctx* ctx, int enable, int first_event_index) {
  if (!ctx) return AG_ERR_INVALID;
  AG_REQUIRE(ctx, first_event_index >= 0, "ag_tc_timing: negative event index");
  ctx->tc_timing = enable ? 1 : 0;
  if (enable) {
    ctx->tc_timing_base = first_event_index;
    ctx->tc_timing_count = 0;
  }
  return AG_OK;
}

extern "C" int ag_tc_timing_count(const ag_ctx* ctx) { return ctx ? ctx->tc_timing_count : 0; }

extern "C" int ag_alloc_host(ag_ctx* ctx, size_t bytes, void** out) {
  if (!ctx || !out) return AG_ERR_INVALID;
  *out = nullptr;
  if (bytes == 0) return AG_OK;
  AG_CUDA(ctx, cudaHostAlloc(out, bytes, cudaHostAllocDefault));
  return AG_OK;
}

extern "C" int ag_free_host(ag_ctx* ctx, void* ptr) {
  if (!ctx) return AG_ERR_INVALID;
  if (ptr) AG_CUDA(ctx, cudaFreeHost(ptr));
  return AG_OK;
}

// ---------------------------------------------------------------------------------------
// fills
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fill_u32_kernel(uint32_t* __restrict__ dst, uint32_t v, int64_t n) {
  // n counts 32-bit words; the 16-byte aligned body is written as uint4
  const int64_t n4 = n >> 2;
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  const uint4 v4 = make_uint4(v, v, v, v);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) d4[i] = v4;
  const int64_t tail = n4 << 2;
  for (int64_t i = tail + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = v;
}

__global__ void __launch_bounds__(256) fill_small_kernel(uint8_t* __restrict__ dst, uint32_t pattern, int itemsize,
                                                          int64_t n_items) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_items; i += stride) {
    if (itemsize == 1)
      dst[i] = (uint8_t)pattern;
    else
      reinterpret_cast<uint16_t*>(dst)[i] = (uint16_t)pattern;
  }
}

static int fill_words(ag_ctx* ctx, void* dst, uint32_t word, int64_t n_words) {
  // head: bring dst to 16-byte alignment with a tiny scalar launch folded into the kernel
  // by offsetting; arena slots are 256-byte aligned so the common case has no head.
  uint32_t* p = static_cast<uint32_t*>(dst);
  if (word == 0 || word == 0xffffffffu) {
    AG_CUDA(ctx, cudaMemsetAsync(dst, word ? 0xff : 0, (size_t)n_words * 4, ctx->stream));
    return AG_OK;
  }
  int64_t head = 0;
  while (head < n_words && !ag_aligned16(p + head)) ++head;
  if (head) {
    fill_u32_kernel<<<1, 32, 0, ctx->stream>>>(p, word, head < 4 ? head : 3);
    AG_LAUNCHED(ctx, "fill_u32_kernel(head)");
  }
  const int64_t body = n_words - head;
  if (body > 0) {
    int64_t want = (body / 4 + 255) / 256;
    int grid = (int)(want < 1 ? 1 : (want > (int64_t)ctx->sm_count * 8 ? (int64_t)ctx->sm_count * 8 : want));
    fill_u32_kernel<<<grid, 256, 0, ctx->stream>>>(p + head, word, body);
    AG_LAUNCHED(ctx, "fill_u32_kernel");
  }
  return AG_OK;
}

extern "C" int ag_fill_f32(ag_ctx* ctx, float* dst, float value, int64_t n) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, dst && n > 0, "ag_fill_f32: null dst or negative n");
  AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(dst) & 3u) == 0, "ag_fill_f32: dst not 4-byte aligned");
  uint32_t w;
  memcpy(&w, &value, 4);
  return fill_words(ctx, dst, w, n);
}

extern "C" int ag_fill_pattern(ag_ctx* ctx, void* dst, uint32_t pattern, int itemsize, int64_t n) {
  if (!ctx) return AG_ERR_INVALID;
  if (n == 0) return AG_OK;
  AG_REQUIRE(ctx, dst && n > 0, "ag_fill_pattern: null dst or negative n");
  AG_REQUIRE(ctx, itemsize == 1 || itemsize == 2 || itemsize == 4, "ag_fill_pattern: itemsize %d not in {1,2,4}",
             itemsize);
  if (itemsize == 4) {
    AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(dst) & 3u) == 0, "ag_fill_pattern: dst not 4-byte aligned");
    return fill_words(ctx, dst, pattern, n);
  }
  if (itemsize == 2) AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(dst) & 1u) == 0, "ag_fill_pattern: dst not 2-byte aligned");
  const uint32_t lo = itemsize == 1 ? (pattern & 0xffu) : (pattern & 0xffffu);
  if (lo == 0) {
    AG_CUDA(ctx, cudaMemsetAsync(dst, 0, (size_t)n * itemsize, ctx->stream));
    return AG_OK;
  }
  int64_t want = (n + 255) / 256;
  int grid = (int)(want > (int64_t)ctx->sm_count * 8 ? (int64_t)ctx->sm_count * 8 : want);
  fill_small_kernel<<<grid, 256, 0, ctx->stream>>>(static_cast<uint8_t*>(dst), lo, itemsize, n);
  AG_LAUNCHED(ctx, "fill_small_kernel");
  return AG_OK;
}
