// Token-embedding gather and its deterministic scatter-add backward.
//
// Forward: out[i,:] = table[ids[i],:], a pure copy (bit-exact).  One warp per token row,
// all 16-byte loads of a row chunk issued before the stores.
//
// Backward: dtable[ids[i],:] += dout[i,:] with a summation order that does not depend on
// scheduling.  No float atomics are used anywhere:
//   1. stable LSD radix sort of (id, position) pairs, 9 bits per pass, so that equal ids end
//      up adjacent and in ascending position order (up to 262144 ids: one histogram launch and
//      one launch per pass; beyond that a histogram, a scan and a scatter launch per pass);
//   2. the sorted list is cut into groups of 32 consecutive entries (64 from 49152 ids on: half as
//      many partial slots for step 3).  A CTA walks one group (for one 512-column slice), every
//      thread keeping a ring of 8 row requests in flight, summing each run of equal ids in list order.  A run
//      that is a complete segment (its id neither continues from the previous group nor
//      into the next one) starts from the current dtable row and is written back directly:
//      for such rows the result is bit-identical to numpy's sequential np.add.at.  A run cut
//      by a group boundary is written to a per-group partial slot instead;
//   3. a combine kernel finds the segments that span several groups and adds their partial slots
//      in group order onto the dtable row.
// Ids outside [0,V) are dropped and flagged in the status word.
#include "ag_common.cuh"

namespace {

// ------------------------------------------------------------------------------ gather
constexpr int GATHER_THREADS = 256;

__global__ void __launch_bounds__(GATHER_THREADS)
gather_forward_kernel(const int32_t* __restrict__ ids, const float* __restrict__ table, float* __restrict__ out,
                      int64_t n_ids, int C, int V, int* status) {
  ag_pdl_wait();
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
sort_init_kernel(const int32_t* __restrict__ ids, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals,
                 uint32_t* __restrict__ head_count, int64_t n, int V, int* status) {
  ag_pdl_wait();
  if (gridDim.x * gridDim.y <= 148) ag_pdl_trigger();  // single-wave grids let the next kernel be scheduled early
  if (blockIdx.x == 0 && threadIdx.x == 0) *head_count = 0u;  // the list of head groups starts empty
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
  ag_pdl_wait();
  if (gridDim.x * gridDim.y <= 148) ag_pdl_trigger();  // single-wave grids let the next kernel be scheduled early
  __shared__ uint32_t s_cnt[SORT_DIGITS];
  for (int d = threadIdx.x; d < SORT_DIGITS; d += SORT_TILE) s_cnt[d] = 0;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * SORT_TILE + threadIdx.x;
  if (i < n) atomicAdd(&s_cnt[(keys[i] >> shift) & (SORT_DIGITS - 1)], 1u);  // integer: order-free
  __syncthreads();
  for (int d = threadIdx.x; d < SORT_DIGITS; d += SORT_TILE) hist[(int64_t)d * n_tiles + blockIdx.x] = s_cnt[d];
}

// Exclusive scan of hist (digit-major, SORT_DIGITS*n_tiles entries) by a single CTA.  Blocks of
// 32768 entries: warp w owns entries [1024 w, 1024 w + 1024) of the block, loads them all at once
// (32 coalesced loads per lane in flight), scans them in registers with a running carry, then the 32
// warp totals are scanned and every warp writes its segment with its offset.
__global__ void __launch_bounds__(1024) sort_scan_kernel(uint32_t* __restrict__ hist, int64_t total) {
  ag_pdl_wait();
  ag_pdl_trigger();
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_carry;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t base = 0; base < total; base += 32768) {
    const int64_t seg = base + (int64_t)warp * 1024 + lane;
    uint32_t v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const int64_t i = seg + k * 32;
      v[k] = i < total ? hist[i] : 0u;
    }
    uint32_t run = 0;  // sum of the warp's entries before row k
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const uint32_t x = v[k];
      uint32_t inc = x;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      v[k] = run + inc - x;  // exclusive prefix inside the warp's segment
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) s_warp[warp] = run;
    __syncthreads();
    const uint32_t carry = s_carry;
    uint32_t before = 0, all = 0;
    for (int w = 0; w < 32; ++w) {  // 32 shared-memory broadcasts; same values for every thread
      const uint32_t t = s_warp[w];
      if (w < warp) before += t;
      all += t;
    }
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const int64_t i = seg + k * 32;
      if (i < total) hist[i] = carry + before + v[k];
    }
    __syncthreads();
    if (threadIdx.x == 0) s_carry = carry + all;
    __syncthreads();
  }
}

// Stable scatter of one tile: rank inside the tile = (#equal digits in earlier warps) +
// (#equal digits in lower lanes of the own warp).
__global__ void __launch_bounds__(SORT_TILE)
sort_scatter_kernel(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                    uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                    const uint32_t* __restrict__ hist, int64_t n, int shift, int n_tiles) {
  ag_pdl_wait();
  if (gridDim.x * gridDim.y <= 148) ag_pdl_trigger();  // single-wave grids let the next kernel be scheduled early
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

// ------------------------------------------------------------------------------ radix sort, few launches
// For up to SORT_FUSED_MAX_TILES tiles (262144 ids) a pass needs no scan launch and no separate
// histogram launch after the first one:
//   * sort_hist_ids_kernel reads the ids themselves (key = id, or V for an id outside the table;
//     value = position), writes the per-tile histogram of the first digit and zeroes the
//     histograms of the later passes;
//   * sort_scatter_fused_kernel derives its tile's digit offsets from the whole histogram
//     (n_tiles x SORT_DIGITS counters, tile-major, a few hundred KB in L2: thread d walks digit d
//     down the tiles with coalesced loads, then the CTA scans the 512 digit totals), places its
//     keys stably, and counts the next pass's per-tile histogram as it goes - integer atomics on
//     counters, aggregated per warp, whose final values do not depend on the order of the additions.
// The order of the sorted list is the one the unfused kernels produce: stable by digit, tile, rank.
constexpr int SORT_FUSED_MAX_TILES = 256;
constexpr int SORT_MAX_PASSES = 4;

__device__ __forceinline__ uint32_t sort_key_of(int id, int V) { return (id >= 0 && id < V) ? (uint32_t)id : (uint32_t)V; }

// hist0 and hist_later are tile-major: counter of (tile, digit) at [tile * SORT_DIGITS + digit].
__global__ void __launch_bounds__(SORT_TILE)
sort_hist_ids_kernel(const int32_t* __restrict__ ids, uint32_t* __restrict__ hist0, uint32_t* __restrict__ hist_later,
                     int64_t later_entries, uint32_t* __restrict__ head_count, int64_t n, int V, int* status) {
  ag_pdl_wait();
  if (gridDim.x <= 148) ag_pdl_trigger();
  if (blockIdx.x == 0 && threadIdx.x == 0) *head_count = 0u;  // the list of head groups starts empty
  __shared__ uint32_t s_cnt[SORT_DIGITS];
  for (int d = threadIdx.x; d < SORT_DIGITS; d += SORT_TILE) s_cnt[d] = 0;
  // the histograms of the later passes start at zero: this CTA clears its share
  for (int64_t e = (int64_t)blockIdx.x * SORT_TILE + threadIdx.x; e < later_entries; e += (int64_t)gridDim.x * SORT_TILE)
    hist_later[e] = 0u;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * SORT_TILE + threadIdx.x;
  if (i < n) {
    const int id = ids[i];
    if (id < 0 || id >= V) atomicOr(status, AG_STATUS_BAD_INDEX);
    atomicAdd(&s_cnt[sort_key_of(id, V) & (SORT_DIGITS - 1)], 1u);  // integer: order-free
  }
  __syncthreads();
  for (int d = threadIdx.x; d < SORT_DIGITS; d += SORT_TILE) hist0[(int64_t)blockIdx.x * SORT_DIGITS + d] = s_cnt[d];
}

// FIRST: keys and values come from the ids (pass 0); otherwise from keys_in / vals_in.
// hist: this pass's per-tile histogram; hist_next: the next pass's (NULL on the last pass), counted
// per tile of the OUTPUT positions.  Both tile-major.
template <bool FIRST>
__global__ void __launch_bounds__(SORT_TILE)
sort_scatter_fused_kernel(const int32_t* __restrict__ ids, const uint32_t* __restrict__ keys_in,
                          const uint32_t* __restrict__ vals_in, uint32_t* __restrict__ keys_out,
                          uint32_t* __restrict__ vals_out, const uint32_t* __restrict__ hist,
                          uint32_t* __restrict__ hist_next, int64_t n, int V, int shift, int n_tiles) {
  ag_pdl_wait();
  if (gridDim.x <= 148) ag_pdl_trigger();
  __shared__ uint16_t s_cnt[SORT_WARPS][SORT_DIGITS];  // 32 KB
  __shared__ uint32_t s_tot[2][SORT_DIGITS], s_bef[2][SORT_DIGITS];
  __shared__ uint32_t s_base[SORT_DIGITS];             // first output position of (digit, this tile)
  __shared__ uint32_t s_wsum[SORT_DIGITS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int d = lane; d < SORT_DIGITS; d += 32) s_cnt[warp][d] = 0;
  // the tile's own key and position are requested first; they arrive while the offsets are computed
  const int64_t i = (int64_t)blockIdx.x * SORT_TILE + threadIdx.x;
  const bool live = i < n;
  uint32_t key = 0, val = 0;
  int digit = 0;
  if (live) {
    if (FIRST) {
      key = sort_key_of(ids[i], V);
      val = (uint32_t)i;
    } else {
      key = keys_in[i];
      val = vals_in[i];
    }
    digit = (key >> shift) & (SORT_DIGITS - 1);
  }

  // ---- offsets: total[d] = count of digit d over all tiles, before[d] = over the tiles before this one.
  // Thread (half, d) walks digit d down one half of the tiles; a warp's loads are 32 consecutive counters.
  {
    const int d = threadIdx.x & (SORT_DIGITS - 1), half = threadIdx.x >> 9;
    const int t0 = half ? (n_tiles + 1) / 2 : 0, t1 = half ? n_tiles : (n_tiles + 1) / 2;
    uint32_t total = 0, before = 0;
    for (int t = t0; t < t1; t += 8) {
      uint32_t v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (t + u < t1) ? hist[(int64_t)(t + u) * SORT_DIGITS + d] : 0u;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        total += v[u];
        if (t + u < (int)blockIdx.x) before += v[u];
      }
    }
    s_tot[half][d] = total;
    s_bef[half][d] = before;
  }
  __syncthreads();
  if (threadIdx.x < SORT_DIGITS) {
    // exclusive scan of the 512 digit totals: 16 warps of 32 digits
    const int d = threadIdx.x;
    const uint32_t total = s_tot[0][d] + s_tot[1][d];
    uint32_t inc = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) s_wsum[warp] = inc;
    s_base[d] = inc - total + s_bef[0][d] + s_bef[1][d];  // the warps' offsets are added below
  }
  __syncthreads();
  if (threadIdx.x < SORT_DIGITS) {
    uint32_t wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += s_wsum[w];
    s_base[threadIdx.x] += wbase;
  }

  const uint32_t live_mask = __ballot_sync(0xffffffffu, live);
  uint32_t peers = 0;
  if (live) peers = __match_any_sync(live_mask, digit);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (live && rank_in_warp == 0) s_cnt[warp][digit] = (uint16_t)__popc(peers);
  __syncthreads();
  if (live) {
    uint32_t before = 0;
    for (int w = 0; w < warp; ++w) before += s_cnt[w][digit];
    const uint32_t dst = s_base[digit] + before + rank_in_warp;
    keys_out[dst] = key;
    vals_out[dst] = val;
    if (hist_next) {
      // one atomic per distinct counter and warp (a hot id fills whole warps with the same counter)
      const uint32_t counter = (dst >> 10) * SORT_DIGITS + ((key >> (shift + SORT_BITS)) & (SORT_DIGITS - 1));
      const uint32_t same = __match_any_sync(live_mask, counter);
      if ((same & ((1u << lane) - 1u)) == 0) atomicAdd(&hist_next[counter], (uint32_t)__popc(same));  // order-free
    }
  }
}

// ------------------------------------------------------------------------------ scatter-add
constexpr int SEG_GROUP_MIN = 32;   // sorted entries per group: 32 or 64 (template parameter G of the two kernels)
constexpr int SEG_THREADS = 128;    // one float4 per thread: 512 columns per CTA
constexpr int SEG_COLS = SEG_THREADS * 4;

__device__ __forceinline__ float4 f4_add(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

// Table-gradient rows are fp32, or bf16 bit patterns (TT = uint16_t: the reference's bf16
// parameter-gradient storage, metal_ops.metal:12395-12446: the sum of a row's contributions is
// formed in fp32 from zero, in position order, and the row becomes bf16(old + sum), rounded once,
// to nearest even).
__device__ __forceinline__ uint32_t seg_bf16_rne(float value) {
  const uint32_t bits = __float_as_uint(value);
  if ((bits & 0x7f800000u) == 0x7f800000u) return ((bits >> 16) | ((bits & 0x007fffffu) ? 0x0040u : 0u)) & 0xffffu;
  return ((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16) & 0xffffu;
}
__device__ __forceinline__ float4 seg_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 seg_load4(const uint16_t* p) {
  const uint2 w = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                     __uint_as_float(w.y & 0xffff0000u));
}
__device__ __forceinline__ void seg_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void seg_store4(uint16_t* p, float4 v) {
  *reinterpret_cast<uint2*>(p) = make_uint2(seg_bf16_rne(v.x) | (seg_bf16_rne(v.y) << 16),
                                            seg_bf16_rne(v.z) | (seg_bf16_rne(v.w) << 16));
}
__device__ __forceinline__ float seg_load1(const float* p) { return *p; }
__device__ __forceinline__ float seg_load1(const uint16_t* p) { return __uint_as_float((uint32_t)*p << 16); }
__device__ __forceinline__ void seg_store1(float* p, float v) { *p = v; }
__device__ __forceinline__ void seg_store1(uint16_t* p, float v) { *p = (uint16_t)seg_bf16_rne(v); }

// grid = (n_groups, ceil(C/512)).  VEC: C % 4 == 0 and pointers 16-byte aligned.
// partials: [n_groups][2][C] floats; slot 0 = the group's first run when it continues from
// the previous group or is the cut part of a longer segment, slot 1 = its last run when
// that run started inside this group and continues into the next one.
// Per-entry run information of a group, computed once per CTA.
constexpr uint32_t RUN_BEGIN = 1u, RUN_END = 2u, RUN_COMPLETE = 4u, RUN_SLOT1 = 8u, RUN_VALID = 16u;
constexpr int SEG_BATCH = 8;  // sorted entries whose rows are requested together

template <bool VEC, typename TT, int SEG_GROUP>
__global__ void __launch_bounds__(SEG_THREADS)
scatter_groups_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ pos,
                      const float* __restrict__ dout, TT* dtable, float* __restrict__ partials,
                      long long* __restrict__ heads, uint32_t* __restrict__ head_count,
                      uint32_t* __restrict__ head_list, int n_groups, int64_t n, int C, int V) {
  constexpr bool BF = sizeof(TT) == 2;  // rounded storage: sum from zero, add the old row last
  ag_pdl_wait();
  __shared__ uint32_t s_key[SEG_GROUP + 2];  // [0] = key before the group, [1..G] group, [G+1] = key after
  __shared__ uint32_t s_pos[SEG_GROUP];
  __shared__ uint32_t s_info[SEG_GROUP];
  const int64_t g0 = (int64_t)blockIdx.x * SEG_GROUP;
  const int cnt = (int)((n - g0) < SEG_GROUP ? (n - g0) : SEG_GROUP);
  for (int t = threadIdx.x; t < SEG_GROUP + 2; t += SEG_THREADS) {
    const int64_t j = g0 - 1 + t;
    // sentinel 0xffffffff never equals a key (keys are <= V)
    s_key[t] = (j >= 0 && j < n && t <= cnt + 1) ? keys[j] : 0xffffffffu;
  }
  for (int t = threadIdx.x; t < SEG_GROUP; t += SEG_THREADS) s_pos[t] = t < cnt ? pos[g0 + t] : 0u;
  __syncthreads();
  for (int j = threadIdx.x; j < cnt; j += SEG_THREADS) {
    // the run (equal keys) around entry j: where it begins and ends inside the group, whether it is cut
    // by the group boundary on either side
    const uint32_t key = s_key[j + 1];
    int rb = j, re = j;
    while (rb > 0 && s_key[rb] == key) --rb;
    while (re + 1 < cnt && s_key[re + 2] == key) ++re;
    const bool from_prev = rb == 0 && s_key[0] == key;
    const bool into_next = re == cnt - 1 && s_key[cnt + 1] == key;
    uint32_t info = 0;
    if (j == rb) info |= RUN_BEGIN;
    if (j == re) info |= RUN_END;
    if (!from_prev && !into_next) info |= RUN_COMPLETE;
    if (!(from_prev || rb == 0)) info |= RUN_SLOT1;
    if (key < (uint32_t)V) info |= RUN_VALID;
    s_info[j] = info;
  }
  __syncthreads();

  const int col = blockIdx.y * SEG_COLS + threadIdx.x * (VEC ? 4 : 1);
  if (VEC) {
    if (col < C) {
    // A ring of SEG_BATCH row requests per thread: the row of entry j + SEG_BATCH (and the dtable row of
    // a complete run that begins there) is requested as soon as entry j has been added, so that a
    // thread always has SEG_BATCH - 1 or SEG_BATCH rows in flight.  The adds run in sorted (= position)
    // order, each complete run starting from its dtable row: the same sequence of additions as an
    // unbuffered add-at.
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 old = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 v[SEG_BATCH], d[SEG_BATCH];
    auto request = [&](int u, int j) {
      v[u] = d[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < cnt) {
        const uint32_t info = s_info[j];
        if (info & RUN_VALID) {
          v[u] = __ldcs(reinterpret_cast<const float4*>(dout + (int64_t)s_pos[j] * C + col));
          if ((info & (RUN_BEGIN | RUN_COMPLETE)) == (RUN_BEGIN | RUN_COMPLETE))
            d[u] = seg_load4(dtable + (int64_t)s_key[j + 1] * C + col);
        }
      }
    };
#pragma unroll
    for (int u = 0; u < SEG_BATCH; ++u) request(u, u);
    for (int j0 = 0; j0 < cnt; j0 += SEG_BATCH) {
#pragma unroll
      for (int u = 0; u < SEG_BATCH; ++u) {
        const int j = j0 + u;
        if (j < cnt) {
          const uint32_t info = s_info[j];
          if (info & RUN_VALID) {
            if (info & RUN_BEGIN) {
              if (BF) { old = d[u]; acc = make_float4(0.f, 0.f, 0.f, 0.f); }
              else acc = d[u];  // zero for a cut run
            }
            acc = f4_add(acc, v[u]);
            if (info & RUN_END) {
              if (info & RUN_COMPLETE)
                seg_store4(dtable + (int64_t)s_key[j + 1] * C + col, BF ? f4_add(old, acc) : acc);
              else
                *reinterpret_cast<float4*>(partials + ((int64_t)blockIdx.x * 2 + ((info & RUN_SLOT1) ? 1 : 0)) * C + col) = acc;
            }
          }
        }
        request(u, j + SEG_BATCH);
      }
    }
    }
  } else {
    // scalar mode: a thread covers columns col, col+128, col+256, col+384
    for (int j = 0; j < cnt; ++j) {
      const uint32_t info = s_info[j];
      if (!(info & RUN_VALID) || !(info & RUN_BEGIN)) continue;
      int end = j;
      while (!(s_info[end] & RUN_END)) ++end;
      const bool complete = (info & RUN_COMPLETE) != 0;
      TT* drow = dtable + (int64_t)s_key[j + 1] * C;
      float* prow = partials + ((int64_t)blockIdx.x * 2 + ((info & RUN_SLOT1) ? 1 : 0)) * C;
      for (int c = col; c < C && c < (int)(blockIdx.y + 1) * SEG_COLS; c += SEG_THREADS) {
        float acc = (complete && !BF) ? seg_load1(drow + c) : 0.0f;
        for (int e = j; e <= end; ++e) acc += dout[(int64_t)s_pos[e] * C + c];
        if (complete) seg_store1(drow + c, BF ? seg_load1(drow + c) + acc : acc);
        else prow[c] = acc;
      }
    }
  }

  // The first warp of the group's first column slice leaves the group's head record for the combine
  // kernel (after its own share of the sums, so that it costs the CTA nothing): 2 * (last group holding entries of the segment) + (partial slot of the head run) when the
  // group's LAST run opens a segment that continues into following groups and starts in this group,
  // else -1.  The decision comes from the keys already in shared memory; only a head group (rare)
  // probes the first keys of the following groups, 32 per ballot.
  if (blockIdx.y == 0 && threadIdx.x < 32) {
    const int lane = threadIdx.x;
    long long rec = -1;
    if (cnt > 0 && g0 + cnt < n) {
      const uint32_t k_last = s_key[cnt];
      int rb = cnt - 1;
      while (rb > 0 && s_key[rb] == k_last) --rb;
      const bool from_prev = rb == 0 && s_key[0] == k_last;
      if (s_key[cnt + 1] == k_last && k_last < (uint32_t)V && !from_prev) {  // warp-uniform
        long long g_end = blockIdx.x;
        for (long long gb = (long long)blockIdx.x + 1;; gb += 32) {
          const long long gq = gb + lane;
          const bool same = gq < n_groups && keys[gq * SEG_GROUP] == k_last;
          const int m = __popc(__ballot_sync(0xffffffffu, same));
          g_end = gb + m - 1;
          if (m < 32) break;
        }
        rec = g_end * 2 + (rb == 0 ? 0 : 1);
      }
    }
    if (lane == 0) {
      heads[blockIdx.x] = rec;
      // head groups are also listed, so that the combine kernel visits nothing else; the order of the
      // list varies from run to run, the work done per entry and its result do not
      if (rec >= 0) head_list[atomicAdd(head_count, 1u)] = blockIdx.x;
    }
  }
}

constexpr int64_t SEG_GROUP64_MIN_IDS = 49152;  // ids from which groups of 64 entries are used
constexpr int SEG_SPLIT = 4;  // sub-ranges of a segment's groups summed side by side in the combine kernel

// Block (SEG_THREADS, SEG_SPLIT), grid (about one resident wave, column slices): a CTA takes entries
// blockIdx.x, blockIdx.x + gridDim.x, ... of the list of head groups (the heads of segments that span
// several groups; few) for its column slice.  For a head group, the
// partial slots of the segment's following groups are split into SEG_SPLIT consecutive sub-ranges; thread
// row y adds its sub-range in group order (8 loads in flight), then row 0 adds
// dtable row + head partial + sub-sum 0 + ... + sub-sum 3 and writes the dtable row.  Fixed order; a
// table row is written by exactly one CTA.
template <bool VEC, typename TT, int SEG_GROUP>
__global__ void __launch_bounds__(SEG_THREADS * SEG_SPLIT)
scatter_combine_kernel(const uint32_t* __restrict__ keys, const long long* __restrict__ heads,
                       const uint32_t* __restrict__ head_count, const uint32_t* __restrict__ head_list, TT* dtable,
                       const float* __restrict__ partials, int64_t n, int C) {
  constexpr bool BF = sizeof(TT) == 2;
  ag_pdl_wait();
  __shared__ float4 s_sub[SEG_SPLIT][SEG_THREADS];
  const int col = blockIdx.y * SEG_COLS + threadIdx.x * (VEC ? 4 : 1);
  const int y = threadIdx.y;
  const uint32_t n_heads = *head_count;
  {
    for (uint32_t hi = blockIdx.x; hi < n_heads; hi += gridDim.x) {
      const int64_t grp = head_list[hi];
      const long long rec = heads[grp];
      const int64_t g_end = rec >> 1;
      const int head_slot = (int)(rec & 1);
      const int64_t g0 = grp * SEG_GROUP;
      const int cnt = (int)((n - g0) < SEG_GROUP ? (n - g0) : SEG_GROUP);
      const uint32_t key = keys[g0 + cnt - 1];
      TT* drow = dtable + (int64_t)key * C;
      if (VEC) {
        const int64_t chunk = (g_end - grp + SEG_SPLIT - 1) / SEG_SPLIT;
        float4 sub = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col < C) {
          int64_t g = grp + 1 + y * chunk;
          int64_t ge = g + chunk;
          if (ge > g_end + 1) ge = g_end + 1;
          for (; g + 8 <= ge; g += 8) {
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
              v[k] = __ldcs(reinterpret_cast<const float4*>(partials + ((g + k) * 2 + 0) * C + col));
#pragma unroll
            for (int k = 0; k < 8; ++k) sub = f4_add(sub, v[k]);
          }
          for (; g < ge; ++g) sub = f4_add(sub, *reinterpret_cast<const float4*>(partials + (g * 2 + 0) * C + col));
        }
        __syncthreads();  // the previous head's sub-sums have been read
        s_sub[y][threadIdx.x] = sub;
        __syncthreads();
        if (y == 0 && col < C) {
          const float4 old = seg_load4(drow + col);
          const float4 head = *reinterpret_cast<const float4*>(partials + (grp * 2 + head_slot) * C + col);
          float4 acc = BF ? head : f4_add(old, head);
#pragma unroll
          for (int q = 0; q < SEG_SPLIT; ++q) acc = f4_add(acc, s_sub[q][threadIdx.x]);
          seg_store4(drow + col, BF ? f4_add(old, acc) : acc);
        }
      } else if (y == 0) {
        for (int c = col; c < C && c < (int)(blockIdx.y + 1) * SEG_COLS; c += SEG_THREADS) {
          const float old = seg_load1(drow + c);
          float acc = BF ? partials[(grp * 2 + head_slot) * C + c] : old + partials[(grp * 2 + head_slot) * C + c];
          for (int64_t g = grp + 1; g <= g_end; ++g) acc += partials[(g * 2 + 0) * C + c];
          seg_store1(drow + c, BF ? old + acc : acc);
        }
      }
    }
  }
}

struct ScatterPlan {
  int64_t n_tiles, n_groups;
  size_t off_keys[2], off_vals[2], off_hist, off_heads, off_partials, total;
};

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

inline ScatterPlan scatter_plan(int64_t n, int C, int group = SEG_GROUP_MIN) {
  ScatterPlan p;
  p.n_tiles = (n + SORT_TILE - 1) / SORT_TILE;
  p.n_groups = (n + group - 1) / group;
  size_t off = 0;
  for (int b = 0; b < 2; ++b) {
    p.off_keys[b] = off; off += align256((size_t)n * 4);
    p.off_vals[b] = off; off += align256((size_t)n * 4);
  }
  p.off_hist = off;  // one histogram per pass when the passes are fused (few tiles), else one in all
  off += align256((size_t)SORT_DIGITS * p.n_tiles * 4 * (p.n_tiles <= SORT_FUSED_MAX_TILES ? SORT_MAX_PASSES : 1));
  // head records: a counter (256 bytes), the record of every group, the list of head groups
  p.off_heads = off; off += 256 + align256((size_t)p.n_groups * 8) + align256((size_t)p.n_groups * 4);
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
    // one row per warp up to 32 CTAs per SM: many short CTAs keep the load/store queues fuller than a resident
    // grid whose warps loop (65536 x 1536, Zipf ids: 80.0 us against 87.4 us with 8 CTAs per SM; 16: 82.2, 64: 79.9)
    int64_t cap = (int64_t)ctx->sm_count * 32;
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

namespace {
// The segmented sum over groups of G sorted entries and the combine over the listed head groups.
template <typename TT, int G>
int launch_groups_combine(ag_ctx* ctx, const ScatterPlan& p, const uint32_t* keys, const uint32_t* pos, const float* dout,
                           TT* dtable, float* partials, long long* heads, uint32_t* head_count, uint32_t* head_list,
                           int64_t n_ids, int C, int V, bool vec) {
  dim3 grid((unsigned)p.n_groups, (unsigned)((C + SEG_COLS - 1) / SEG_COLS));
  // combine: about one resident wave of 512-thread CTAs (four per SM) over all column slices
  int64_t cx = (int64_t)ctx->sm_count * 4 / grid.y;
  cx = cx < 1 ? 1 : (cx > p.n_groups ? p.n_groups : cx);
  dim3 cgrid((unsigned)cx, grid.y);
  if (vec) {
    auto groups_vec = scatter_groups_kernel<true, TT, G>;
    auto combine_vec = scatter_combine_kernel<true, TT, G>;
    AG_LAUNCH_PDL(ctx, "scatter_groups_kernel", groups_vec, grid, SEG_THREADS, 0, keys, pos, dout, dtable, partials, heads,
                  head_count, head_list, (int)p.n_groups, n_ids, C, V);
    AG_LAUNCH_PDL(ctx, "scatter_combine_kernel", combine_vec, cgrid, dim3(SEG_THREADS, SEG_SPLIT), 0, keys,
                  (const long long*)heads, (const uint32_t*)head_count, (const uint32_t*)head_list, dtable,
                  (const float*)partials, n_ids, C);
  } else {
    scatter_groups_kernel<false, TT, G><<<grid, SEG_THREADS, 0, ctx->stream>>>(keys, pos, dout, dtable, partials, heads,
                                                                               head_count, head_list, (int)p.n_groups,
                                                                               n_ids, C, V);
    AG_LAUNCHED(ctx, "scatter_groups_kernel");
    scatter_combine_kernel<false, TT, G><<<cgrid, dim3(SEG_THREADS, SEG_SPLIT), 0, ctx->stream>>>(
        keys, heads, head_count, head_list, dtable, partials, n_ids, C);
    AG_LAUNCHED(ctx, "scatter_combine_kernel");
  }
  return AG_OK;
}

template <typename TT>
int gather_backward_t(ag_ctx* ctx, const int32_t* ids, const float* dout, TT* dtable, void* scratch,
                      size_t scratch_bytes, int64_t n_ids, int C, int V) {
  if (!ctx) return AG_ERR_INVALID;
  if (n_ids == 0) return AG_OK;
  AG_REQUIRE(ctx, ids && dout && dtable, "ag_gather_backward: null pointer");
  AG_REQUIRE(ctx, n_ids > 0 && C > 0 && V > 0, "ag_gather_backward: bad shape n=%lld C=%d V=%d", (long long)n_ids, C, V);
  AG_REQUIRE(ctx, n_ids < (1ll << 31) && (int64_t)V < (1ll << 31) - 1, "ag_gather_backward: sizes exceed 32-bit keys");
  // Groups of 64 entries halve the partial rows a long segment leaves for the combine kernel; they pay
  // once the groups still fill the GPU several times over.  The scratch size is the one of groups of 32.
  const int group = ctx->scatter_group ? ctx->scatter_group : (n_ids >= SEG_GROUP64_MIN_IDS ? 64 : 32);
  const ScatterPlan p = scatter_plan(n_ids, C, group);
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
  uint32_t* head_count = reinterpret_cast<uint32_t*>(base + p.off_heads);
  long long* heads = reinterpret_cast<long long*>(base + p.off_heads + 256);
  uint32_t* head_list = reinterpret_cast<uint32_t*>(base + p.off_heads + 256 + align256((size_t)p.n_groups * 8));
  const int n_tiles = (int)p.n_tiles;
  // keys are in [0, V]: sort just enough 9-bit digits to cover V
  int bits = 1;
  while (((int64_t)1 << bits) <= (int64_t)V) ++bits;
  const int passes = (bits + SORT_BITS - 1) / SORT_BITS;
  int cur = 0;
  if (n_tiles <= SORT_FUSED_MAX_TILES) {
    // passes + 1 launches: no key/position initialisation, no scan, no histogram launch after the first
    const int64_t hist_entries = (int64_t)SORT_DIGITS * n_tiles;
    AG_LAUNCH_PDL(ctx, "sort_hist_ids_kernel", sort_hist_ids_kernel, n_tiles, SORT_TILE, 0, ids, hist, hist + hist_entries,
                  hist_entries * (passes - 1), head_count, n_ids, V, ctx->d_status);
    for (int pass = 0; pass < passes; ++pass) {
      uint32_t* h = hist + hist_entries * pass;
      uint32_t* h_next = pass + 1 < passes ? h + hist_entries : nullptr;
      if (pass == 0) {
        AG_LAUNCH_PDL(ctx, "sort_scatter_fused_kernel", sort_scatter_fused_kernel<true>, n_tiles, SORT_TILE, 0, ids,
                      (const uint32_t*)nullptr, (const uint32_t*)nullptr, keys[1], vals[1], (const uint32_t*)h, h_next,
                      n_ids, V, 0, n_tiles);
        cur = 1;
      } else {
        AG_LAUNCH_PDL(ctx, "sort_scatter_fused_kernel", sort_scatter_fused_kernel<false>, n_tiles, SORT_TILE, 0,
                      (const int32_t*)nullptr, (const uint32_t*)keys[cur], (const uint32_t*)vals[cur], keys[cur ^ 1],
                      vals[cur ^ 1], (const uint32_t*)h, h_next, n_ids, V, pass * SORT_BITS, n_tiles);
        cur ^= 1;
      }
    }
  } else {
    AG_LAUNCH_PDL(ctx, "sort_init_kernel", sort_init_kernel, n_tiles, SORT_TILE, 0, ids, keys[0], vals[0], head_count,
                  n_ids, V, ctx->d_status);
    for (int shift = 0; shift < bits; shift += SORT_BITS) {
      AG_LAUNCH_PDL(ctx, "sort_hist_kernel", sort_hist_kernel, n_tiles, SORT_TILE, 0, (const uint32_t*)keys[cur], hist,
                    n_ids, shift, n_tiles);
      AG_LAUNCH_PDL(ctx, "sort_scan_kernel", sort_scan_kernel, 1, 1024, 0, hist, (int64_t)SORT_DIGITS * n_tiles);
      AG_LAUNCH_PDL(ctx, "sort_scatter_kernel", sort_scatter_kernel, n_tiles, SORT_TILE, 0, (const uint32_t*)keys[cur],
                    (const uint32_t*)vals[cur], keys[cur ^ 1], vals[cur ^ 1], (const uint32_t*)hist, n_ids, shift, n_tiles);
      cur ^= 1;
    }
  }
  // 4-element packets of a table row: 16 bytes in fp32, 8 bytes in bf16 storage
  const bool vec = (C % 4 == 0) && ag_aligned16(dout) && ag_aligned16(dtable);
  if (group == 128)
    return launch_groups_combine<TT, 128>(ctx, p, keys[cur], vals[cur], dout, dtable, partials, heads, head_count,
                                          head_list, n_ids, C, V, vec);
  if (group == 64)
    return launch_groups_combine<TT, 64>(ctx, p, keys[cur], vals[cur], dout, dtable, partials, heads, head_count,
                                         head_list, n_ids, C, V, vec);
  return launch_groups_combine<TT, 32>(ctx, p, keys[cur], vals[cur], dout, dtable, partials, heads, head_count, head_list,
                                       n_ids, C, V, vec);
}
}  // namespace

extern "C" int ag_gather_backward(ag_ctx* ctx, const int32_t* ids, const float* dout, float* dtable, void* scratch,
                                  size_t scratch_bytes, int64_t n_ids, int C, int V) {
  return gather_backward_t<float>(ctx, ids, dout, dtable, scratch, scratch_bytes, n_ids, C, V);
}

extern "C" int ag_gather_backward_bf16(ag_ctx* ctx, const int32_t* ids, const float* dout, uint16_t* dtable,
                                       void* scratch, size_t scratch_bytes, int64_t n_ids, int C, int V) {
  return gather_backward_t<uint16_t>(ctx, ids, dout, dtable, scratch, scratch_bytes, n_ids, C, V);
}
