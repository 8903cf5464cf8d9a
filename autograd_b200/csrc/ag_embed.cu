// Token-embedding gather and its deterministic scatter-add backward.
//
// Forward: out[i,:] = table[ids[i],:], a pure copy (bit-exact).  One warp per token row,
// all 16-byte loads of a row chunk issued before the stores.
//
// Backward: dtable[ids[i],:] += dout[i,:] with a summation order that does not depend on
// scheduling.  No float atomics are used anywhere:
//   1. stable LSD radix sort of (id, position) pairs, 9 bits per pass, so that equal ids end
//      up adjacent and in ascending position order;
//   2. the sorted list is cut into groups of SEG_GROUP consecutive entries.  A CTA walks one
//      group (for one 512-column slice), summing each run of equal ids in list order.  A run
//      that is a complete segment (its id neither continues from the previous group nor
//      into the next one) starts from the current dtable row and is written back directly:
//      for such rows the result is bit-identical to numpy's sequential np.add.at.  A run cut
//      by a group boundary is written to a per-group partial slot instead;
//   3. a combine kernel adds, for every segment that spans several groups, its partial slots
//      in group order onto the dtable row.
// Ids outside [0,V) are dropped and flagged in the status word.
#include "ag_common.cuh"

namespace {

// ------------------------------------------------------------------------------ gather
constexpr int GATHER_THREADS = 256;

__global__ void __launch_bounds__(GATHER_THREADS)
gather_forward_kernel(const int32_t* __restrict__ ids, const float* __restrict__ table, float* __restrict__ out,
                      int64_t n_ids, int C, int V, int* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = ((int64_t)blockIdx.x * GATHER_THREADS + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * GATHER_THREADS) >> 5;
  const int c4 = C >> 2;
  for (int64_t i = warp_global; i < n_ids; i += n_warps) {
    const int id = ids[i];
    const bool ok = id >= 0 && id < V;
    if (!ok && lane == 0) atomicOr(status, AG_STATUS_BAD_INDEX);
    const float4* src = reinterpret_cast<const float4*>(table + (int64_t)(ok ? id : 0) * C);
    float4* dst = reinterpret_cast<float4*>(out + i * C);
    for (int p = lane; p < c4; p += 32 * 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (p + u * 32 < c4) v[u] = ok ? __ldg(src + p + u * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (p + u * 32 < c4) __stcs(dst + p + u * 32, v[u]);
    }
  }
}

__global__ void __launch_bounds__(GATHER_THREADS)
gather_forward_scalar_kernel(const int32_t* __restrict__ ids, const float* __restrict__ table,
                             float* __restrict__ out, int64_t n_ids, int C, int V, int* status) {
  const int64_t total = n_ids * C;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int64_t i = e / C;
    const int c = (int)(e - i * C);
    const int id = ids[i];
    const bool ok = id >= 0 && id < V;
    if (!ok && c == 0) atomicOr(status, AG_STATUS_BAD_INDEX);
    out[e] = ok ? table[(int64_t)id * C + c] : 0.0f;
  }
}

// ------------------------------------------------------------------------------ radix sort
constexpr int SORT_BITS = 9;
constexpr int SORT_DIGITS = 1 << SORT_BITS;  // 512
constexpr int SORT_TILE = 1024;              // keys per CTA, one per thread
constexpr int SORT_WARPS = SORT_TILE / 32;

// Out-of-range ids get the key V (sorted behind every valid id, dropped later).
__global__ void __launch_bounds__(SORT_TILE)
sort_init_kernel(const int32_t* __restrict__ ids, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals, int64_t n,
                 int V, int* status) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  const bool ok = id >= 0 && id < V;
  if (!ok) atomicOr(status, AG_STATUS_BAD_INDEX);
  keys[i] = ok ? (uint32_t)id : (uint32_t)V;
  vals[i] = (uint32_t)i;
}

// Per-tile digit histogram: hist[digit * n_tiles + tile].
__global__ void __launch_bounds__(SORT_TILE)
sort_hist_kernel(const uint32_t* __restrict__ keys, uint32_t* __restrict__ hist, int64_t n, int shift, int n_tiles) {
  __shared__ uint32_t s_cnt[SORT_DIGITS];
  for (int d = threadIdx.x; d < SORT_DIGITS; d += SORT_TILE) s_cnt[d] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * SORT_TILE + threadIdx.x;
  if (i < n) atomicAdd(&s_cnt[(keys[i] >> shift) & (SORT_DIGITS - 1)], 1u);  // integer: order-free
  __syncthreads();
  for (int d = threadIdx.x; d < SORT_DIGITS; d += SORT_TILE) hist[(int64_t)d * n_tiles + blockIdx.x] = s_cnt[d];
}

// Exclusive scan of hist (digit-major, SORT_DIGITS*n_tiles entries) by a single CTA.
__global__ void __launch_bounds__(1024) sort_scan_kernel(uint32_t* __restrict__ hist, int64_t total) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t base = 0; base < total; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const uint32_t v = i < total ? hist[i] : 0u;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      uint32_t w = s_warp[lane];
      uint32_t winc = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += t;
      }
      s_warp[lane] = winc - w;  // exclusive prefix of warp totals
    }
    __syncthreads();
    const uint32_t carry = s_carry;
    if (i < total) hist[i] = carry + s_warp[warp] + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = carry + s_warp[31] + inc;
    __syncthreads();
  }
}

// Stable scatter of one tile: rank inside the tile = (#equal digits in earlier warps) +
// (#equal digits in lower lanes of the own warp).
__global__ void __launch_bounds__(SORT_TILE)
sort_scatter_kernel(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                    uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                    const uint32_t* __restrict__ hist, int64_t n, int shift, int n_tiles) {
  __shared__ uint16_t s_cnt[SORT_WARPS][SORT_DIGITS];  // 32 KB
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int d = lane; d < SORT_DIGITS; d += 32) s_cnt[warp][d] = 0;
  __syncwarp();
  const int64_t i = (int64_t)blockIdx.x * SORT_TILE + threadIdx.x;
  const bool live = i < n;
  uint32_t key = 0, val = 0;
  int digit = 0;
  if (live) {
    key = keys_in[i];
    val = vals_in[i];
    digit = (key >> shift) & (SORT_DIGITS - 1);
  }
  // peers: live lanes of this warp holding the same digit
  const uint32_t live_mask = __ballot_sync(0xffffffffu, live);
  uint32_t peers = 0;
  if (live) peers = __match_any_sync(live_mask, digit);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (live && rank_in_warp == 0) s_cnt[warp][digit] = (uint16_t)__popc(peers);
  __syncthreads();
  if (live) {
    uint32_t before = 0;
    for (int w = 0; w < warp; ++w) before += s_cnt[w][digit];
    const uint32_t dst = hist[(int64_t)digit * n_tiles + blockIdx.x] + before + rank_in_warp;
    keys_out[dst] = key;
    vals_out[dst] = val;
  }
}

// ------------------------------------------------------------------------------ scatter-add
constexpr int SEG_GROUP = 32;       // sorted entries per group
constexpr int SEG_THREADS = 128;    // one float4 per thread: 512 columns per CTA
constexpr int SEG_COLS = SEG_THREADS * 4;

__device__ __forceinline__ float4 f4_add(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// grid = (n_groups, ceil(C/512)).  VEC: C % 4 == 0 and pointers 16-byte aligned.
// partials: [n_groups][2][C] floats; slot 0 = the group's first run when it continues from
// the previous group or is the cut part of a longer segment, slot 1 = its last run when
// that run started inside this group and continues into the next one.
template <bool VEC>
__global__ void __launch_bounds__(SEG_THREADS)
scatter_groups_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ pos,
                      const float* __restrict__ dout, float* dtable, float* __restrict__ partials, int64_t n, int C,
                      int V) {
  __shared__ uint32_t s_key[SEG_GROUP + 2];  // [0] = key before the group, [1..G] group, [G+1] = key after
  __shared__ uint32_t s_pos[SEG_GROUP];
  const int64_t g0 = (int64_t)blockIdx.x * SEG_GROUP;
  const int cnt = (int)((n - g0) < SEG_GROUP ? (n - g0) : SEG_GROUP);
  if (threadIdx.x < SEG_GROUP + 2) {
    const int64_t j = g0 - 1 + threadIdx.x;
    // sentinel 0xffffffff never equals a key (keys are <= V)
    s_key[threadIdx.x] = (j >= 0 && j < n && (int)threadIdx.x <= cnt + 1) ? keys[j] : 0xffffffffu;
  }
  if (threadIdx.x < SEG_GROUP) s_pos[threadIdx.x] = threadIdx.x < cnt ? pos[g0 + threadIdx.x] : 0u;
  __syncthreads();

  const int col = blockIdx.y * SEG_COLS + threadIdx.x * (VEC ? 4 : 1);
  // scalar mode: a thread covers columns col, col+128, col+256, col+384
  int e = 0;
  while (e < cnt) {
    const uint32_t key = s_key[e + 1];
    int end = e + 1;
    while (end < cnt && s_key[end + 1] == key) ++end;
    const bool from_prev = (e == 0) && (s_key[0] == key);
    const bool into_next = (end == cnt) && (s_key[cnt + 1] == key);
    if (key < (uint32_t)V) {
      const bool complete = !from_prev && !into_next;
      float* drow = dtable + (int64_t)key * C;
      float* prow = partials + ((int64_t)blockIdx.x * 2 + (from_prev || e == 0 ? 0 : 1)) * C;
      if (VEC) {
        if (col < C) {
          float4 acc = complete ? *reinterpret_cast<const float4*>(drow + col) : make_float4(0.f, 0.f, 0.f, 0.f);
          int j = e;
          for (; j + 4 <= end; j += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
              v[u] = __ldcs(reinterpret_cast<const float4*>(dout + (int64_t)s_pos[j + u] * C + col));
#pragma unroll
            for (int u = 0; u < 4; ++u) acc = f4_add(acc, v[u]);
          }
          for (; j < end; ++j)
            acc = f4_add(acc, __ldcs(reinterpret_cast<const float4*>(dout + (int64_t)s_pos[j] * C + col)));
          *reinterpret_cast<float4*>((complete ? drow : prow) + col) = acc;
        }
      } else {
        for (int c = col; c < C && c < (int)(blockIdx.y + 1) * SEG_COLS; c += SEG_THREADS) {
          float acc = complete ? drow[c] : 0.0f;
          for (int j = e; j < end; ++j) acc += dout[(int64_t)s_pos[j] * C + c];
          (complete ? drow : prow)[c] = acc;
        }
      }
    }
    e = end;
  }
}

// One CTA per (group, column slice): if the group's LAST run opens a multi-group segment
// (or the group's only run is the head of one), add the partial slots of that segment in
// group order onto the dtable row.
template <bool VEC>
__global__ void __launch_bounds__(SEG_THREADS)
scatter_combine_kernel(const uint32_t* __restrict__ keys, float* dtable, const float* __restrict__ partials, int64_t n,
                       int n_groups, int C, int V) {
  const int64_t grp = blockIdx.x;
  const int64_t g0 = grp * SEG_GROUP;
  const int cnt = (int)((n - g0) < SEG_GROUP ? (n - g0) : SEG_GROUP);
  const int64_t last = g0 + cnt - 1;
  if (last + 1 >= n) return;                 // nothing after this group
  const uint32_t key = keys[last];
  if (keys[last + 1] != key) return;         // last run does not continue
  if (key >= (uint32_t)V) return;            // dropped ids
  // is this group the head of the segment?  The run containing `last` must start here:
  // either it starts after the group's first entry, or at entry 0 with a different key before.
  int64_t start = last;
  while (start > g0 && keys[start - 1] == key) --start;
  if (start == g0 && g0 > 0 && keys[g0 - 1] == key) return;  // a continuation, an earlier group is the head
  const int head_slot = (start == g0) ? 0 : 1;

  // number of following groups whose first run continues this segment (same for every thread;
  // found by binary search over the sorted keys: the last entry of the segment)
  int64_t lo_i = last, hi_i = n - 1;
  while (lo_i < hi_i) {
    const int64_t mid = (lo_i + hi_i + 1) >> 1;
    if (keys[mid] == key) lo_i = mid; else hi_i = mid - 1;
  }
  const int64_t g_end = lo_i / SEG_GROUP;  // last group that holds entries of this segment
  const int col = blockIdx.y * SEG_COLS + threadIdx.x * (VEC ? 4 : 1);
  float* drow = dtable + (int64_t)key * C;
  if (VEC) {
    if (col >= C) return;
    float4 acc = *reinterpret_cast<const float4*>(drow + col);
    acc = f4_add(acc, *reinterpret_cast<const float4*>(partials + (grp * 2 + head_slot) * C + col));
    int64_t g = grp + 1;
    // loads of 8 partial rows are independent and in flight together; the adds stay in group order
    for (; g + 8 <= g_end + 1; g += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcs(reinterpret_cast<const float4*>(partials + ((g + u) * 2 + 0) * C + col));
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = f4_add(acc, v[u]);
    }
    for (; g <= g_end; ++g) acc = f4_add(acc, *reinterpret_cast<const float4*>(partials + (g * 2 + 0) * C + col));
    *reinterpret_cast<float4*>(drow + col) = acc;
  } else {
    for (int c = col; c < C && c < (int)(blockIdx.y + 1) * SEG_COLS; c += SEG_THREADS) {
      float acc = drow[c] + partials[(grp * 2 + head_slot) * C + c];
      for (int64_t g = grp + 1; g <= g_end; ++g) acc += partials[(g * 2 + 0) * C + c];
      drow[c] = acc;
    }
  }
}

struct ScatterPlan {
  int64_t n_tiles, n_groups;
  size_t off_keys[2], off_vals[2], off_hist, off_partials, total;
};

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

inline ScatterPlan scatter_plan(int64_t n, int C) {
  ScatterPlan p;
  p.n_tiles = (n + SORT_TILE - 1) / SORT_TILE;
  p.n_groups = (n + SEG_GROUP - 1) / SEG_GROUP;
  size_t off = 0;
  for (int b = 0; b < 2; ++b) {
    p.off_keys[b] = off; off += align256((size_t)n * 4);
    p.off_vals[b] = off; off += align256((size_t)n * 4);
  }
  p.off_hist = off; off += align256((size_t)SORT_DIGITS * p.n_tiles * 4);
  p.off_partials = off; off += align256((size_t)p.n_groups * 2 * C * 4);
  p.total = off;
  return p;
}

}  // namespace

// =========================================================================================
extern "C" int ag_gather_forward(ag_ctx* ctx, const int32_t* ids, const float* table, float* out, int64_t n_ids,
                                 int C, int V) {
  if (!ctx) return AG_ERR_INVALID;
  if (n_ids == 0) return AG_OK;
  AG_REQUIRE(ctx, ids && table && out, "ag_gather_forward: null pointer");
  AG_REQUIRE(ctx, n_ids > 0 && C > 0 && V > 0, "ag_gather_forward: bad shape n=%lld C=%d V=%d", (long long)n_ids, C, V);
  if (C % 4 == 0 && ag_aligned16(table) && ag_aligned16(out)) {
    int64_t want = (n_ids * 32 + GATHER_THREADS - 1) / GATHER_THREADS;
    int64_t cap = (int64_t)ctx->sm_count * 8;
    gather_forward_kernel<<<(int)(want < cap ? want : cap), GATHER_THREADS, 0, ctx->stream>>>(ids, table, out, n_ids,
                                                                                               C, V, ctx->d_status);
    AG_LAUNCHED(ctx, "gather_forward_kernel");
  } else {
    int64_t want = (n_ids * C + GATHER_THREADS - 1) / GATHER_THREADS;
    int64_t cap = (int64_t)ctx->sm_count * 8;
    gather_forward_scalar_kernel<<<(int)(want < cap ? want : cap), GATHER_THREADS, 0, ctx->stream>>>(
        ids, table, out, n_ids, C, V, ctx->d_status);
    AG_LAUNCHED(ctx, "gather_forward_scalar_kernel");
  }
  return AG_OK;
}

extern "C" size_t ag_scatter_add_scratch_bytes(int64_t n_ids, int C, int V) {
  (void)V;
  if (n_ids <= 0 || C <= 0) return 0;
  return scatter_plan(n_ids, C).total;
}

extern "C" int ag_gather_backward(ag_ctx* ctx, const int32_t* ids, const float* dout, float* dtable, void* scratch,
                                  size_t scratch_bytes, int64_t n_ids, int C, int V) {
  if (!ctx) return AG_ERR_INVALID;
  if (n_ids == 0) return AG_OK;
  AG_REQUIRE(ctx, ids && dout && dtable, "ag_gather_backward: null pointer");
  AG_REQUIRE(ctx, n_ids > 0 && C > 0 && V > 0, "ag_gather_backward: bad shape n=%lld C=%d V=%d", (long long)n_ids, C, V);
  AG_REQUIRE(ctx, n_ids < (1ll << 31) && (int64_t)V < (1ll << 31) - 1, "ag_gather_backward: sizes exceed 32-bit keys");
  const ScatterPlan p = scatter_plan(n_ids, C);
  if (!scratch || scratch_bytes < p.total)
    AG_FAIL(ctx, AG_ERR_SCRATCH, "ag_gather_backward: scratch has %zu bytes, needs %zu", scratch_bytes, p.total);
  AG_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "ag_gather_backward: scratch not 256-byte aligned");
  AG_REQUIRE(ctx, (int64_t)SORT_DIGITS * p.n_tiles < (1ll << 31) && p.n_groups < (1ll << 31) - 1,
             "ag_gather_backward: too many ids");
  unsigned char* base = static_cast<unsigned char*>(scratch);
  uint32_t* keys[2] = {reinterpret_cast<uint32_t*>(base + p.off_keys[0]), reinterpret_cast<uint32_t*>(base + p.off_keys[1])};
  uint32_t* vals[2] = {reinterpret_cast<uint32_t*>(base + p.off_vals[0]), reinterpret_cast<uint32_t*>(base + p.off_vals[1])};
  uint32_t* hist = reinterpret_cast<uint32_t*>(base + p.off_hist);
  float* partials = reinterpret_cast<float*>(base + p.off_partials);
  const int n_tiles = (int)p.n_tiles;

  sort_init_kernel<<<n_tiles, SORT_TILE, 0, ctx->stream>>>(ids, keys[0], vals[0], n_ids, V, ctx->d_status);
  AG_LAUNCHED(ctx, "sort_init_kernel");
  // keys are in [0, V]: sort just enough 9-bit digits to cover V
  int bits = 1;
  while (((int64_t)1 << bits) <= (int64_t)V) ++bits;
  int cur = 0;
  for (int shift = 0; shift < bits; shift += SORT_BITS) {
    sort_hist_kernel<<<n_tiles, SORT_TILE, 0, ctx->stream>>>(keys[cur], hist, n_ids, shift, n_tiles);
    AG_LAUNCHED(ctx, "sort_hist_kernel");
    sort_scan_kernel<<<1, 1024, 0, ctx->stream>>>(hist, (int64_t)SORT_DIGITS * n_tiles);
    AG_LAUNCHED(ctx, "sort_scan_kernel");
    sort_scatter_kernel<<<n_tiles, SORT_TILE, 0, ctx->stream>>>(keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1], hist,
                                                                 n_ids, shift, n_tiles);
    AG_LAUNCHED(ctx, "sort_scatter_kernel");
    cur ^= 1;
  }
  const bool vec = (C % 4 == 0) && ag_aligned16(dout) && ag_aligned16(dtable);
  dim3 grid((unsigned)p.n_groups, (unsigned)((C + SEG_COLS - 1) / SEG_COLS));
  if (vec) {
    scatter_groups_kernel<true><<<grid, SEG_THREADS, 0, ctx->stream>>>(keys[cur], vals[cur], dout, dtable, partials,
                                                                        n_ids, C, V);
    AG_LAUNCHED(ctx, "scatter_groups_kernel");
    scatter_combine_kernel<true><<<grid, SEG_THREADS, 0, ctx->stream>>>(keys[cur], dtable, partials, n_ids,
                                                                         (int)p.n_groups, C, V);
    AG_LAUNCHED(ctx, "scatter_combine_kernel");
  } else {
    scatter_groups_kernel<false><<<grid, SEG_THREADS, 0, ctx->stream>>>(keys[cur], vals[cur], dout, dtable, partials,
                                                                         n_ids, C, V);
    AG_LAUNCHED(ctx, "scatter_groups_kernel");
    scatter_combine_kernel<false><<<grid, SEG_THREADS, 0, ctx->stream>>>(keys[cur], dtable, partials, n_ids,
                                                                          (int)p.n_groups, C, V);
    AG_LAUNCHED(ctx, "scatter_combine_kernel");
  }
  return AG_OK;
}
