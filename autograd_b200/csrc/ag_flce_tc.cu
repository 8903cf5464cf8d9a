// tcgen05 tensor-core panels of the fused linear + cross-entropy head.
//
// One persistent GEMM kernel, D[M,N] (+)= A[M,K] . B[N,K]^T with both operands K-major:
//   warp 0      : TMA producer  - cp.async.bulk.tensor tiles (128-byte swizzle) into a ring of
//                 shared-memory stages, completion on mbarriers;
//   warp 1      : allocates TMEM, then one elected lane issues tcgen05.mma (cta_group::1,
//                 M = 128, N = BN) from shared-memory descriptors into one of two TMEM
//                 accumulators; tcgen05.commit releases stages and publishes accumulators;
//   warps 2..9  : epilogue - tcgen05.ld of the finished accumulator (one TMEM lane = one output
//                 row per thread), store / accumulate to global memory, while the MMA warp
//                 already works on the next tile in the other accumulator.
// Precision modes:
//   3xTF32 : every fp32 operand is split once into hi = tf32(x), lo = tf32(x - hi); each k-step
//            issues hi*lo + lo*hi + hi*hi into the same fp32 accumulator (error ~2^-22 of the
//            product, i.e. fp32-grade logits from tf32 tensor cores);
//   BF16   : operands rounded to bf16 once, a single MMA per k-step.
// All three GEMMs of the head are expressed K-major by keeping transposed operand copies:
//   logits  = X   . W^T       A = X  [rows,C]    B = W  [vc,C]
//   dX     += dl  . W         A = dl [rows,vc]   B = W^T[C,vc]
//   dW     += dl^T. X         A = dl^T[vc,rows]  B = X^T[C,rows]
// Every output tile has exactly one writer, so accumulation order is fixed.
// Every mbarrier wait is bounded; on expiry the CTA raises AG_STATUS_WAIT_EXPIRED, all roles
// leave their loops, TMEM is released and the kernel returns.  Every CTA loads its own tiles; no thread-block clusters.
#include <cuda.h>

#include "ag_flce.cuh"

namespace {

constexpr int TC_BM = 128;
constexpr int TC_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;
constexpr int TC_MAX_STAGES = 6;
constexpr int TC_SMEM_LIMIT = 227 * 1024;

struct TcParams {
  int M, N, K;
  int BN;          // tile width, multiple of 32, <= 256
  int BK;          // elements per stage along K: 128 bytes worth (32 fp32 / 64 bf16)
  int umma_k;      // elements per MMA along K: 32 bytes worth (8 / 16)
  int split;       // 1: operands come as (hi, lo) pairs and 3 MMAs are issued per k-step
  int stages;
  int tiles_m, tiles_n, k_iters;
  int splits;      // split-K: each output tile is computed by `splits` CTAs over disjoint k ranges
  int k_per_split; // k iterations per split (the last one may be shorter)
  int64_t split_stride;  // elements between the partial outputs of consecutive splits
  int n_fastest;   // tile order
  uint32_t idesc;
  uint32_t a_bytes, b_bytes;  // bytes of one A / B tile in a stage
  float* D;
  int64_t ldd;
  int accumulate;
  int* status;
  // EPI_STORE extras of the linear+bias+residual op: out = acc + bias[col] + resid[row][col]
  const float* bias;
  const float* resid;
  int64_t ld_resid;
  // fused cross-entropy epilogues (EPI_STATS / EPI_DLOGITS); row-indexed arrays start at A's row 0
  const int32_t* targets;
  int v0;                  // vocabulary index of column 0 of this panel
  int V;
  float2* part;            // EPI_STATS: per (column tile, row) partial (max, sum exp), [tiles_n][part_ld]
  int64_t part_ld;
  float* tgt_logit;        // EPI_STATS: logit of the target column, written by the tile that holds it
  const float* lse;        // EPI_DLOGITS
  const float* row_scale;
  const float* dloss;
  const float* denom;
  int ignore_mode;
  void* dl_hi;             // EPI_DLOGITS outputs: dl [M][ld_dl] and dl^T [N][ld_dlT], (hi, lo) or bf16
  void* dl_lo;
  int64_t ld_dl;
  void* dlT_hi;
  void* dlT_lo;
  int64_t ld_dlT;
};

enum { EPI_STORE = 0, EPI_STATS = 1, EPI_DLOGITS = 2 };

// ---------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void tc_tma_load_2d(const CUtensorMap* tm, void* smem_dst, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          ag_smem_u32(smem_dst)),
      "l"(tm), "r"(ag_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ag_smem_u32(bar))
               : "memory");
}

template <bool TF32>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  if (TF32) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, groups of
// 8 rows 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tc_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tc_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded wait that also gives up when another role of the CTA has already given up.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
    if (ag_mbar_try_wait(bar, parity)) return true;
    if ((i & 127u) == 127u) {
      if (*abort_flag) return false;
      __nanosleep(20);
    }
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tc_tile_coords(const TcParams& p, int tile, int& tm, int& tn, int& k_begin,
                                               int& k_end, int& split) {
  const int per_split = p.tiles_m * p.tiles_n;
  split = tile / per_split;
  tile -= split * per_split;
  k_begin = split * p.k_per_split;
  k_end = k_begin + p.k_per_split < p.k_iters ? k_begin + p.k_per_split : p.k_iters;
  if (p.n_fastest) {
    tm = tile / p.tiles_n;
    tn = tile - tm * p.tiles_n;
  } else {
    tn = tile / p.tiles_m;
    tm = tile - tn * p.tiles_m;
  }
}

// ---------------------------------------------------------------------------- the kernel
__device__ __forceinline__ float tc_tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

template <bool TF32, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA_hi, const __grid_constant__ CUtensorMap tmA_lo,
               const __grid_constant__ CUtensorMap tmB_hi, const __grid_constant__ CUtensorMap tmB_lo,
               const TcParams p) {
  extern __shared__ unsigned char tc_smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t stage_bytes = (p.a_bytes + p.b_bytes) * (p.split ? 2u : 1u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + (size_t)p.stages * stage_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + TC_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * TC_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ag_mbar_init(&full[s], 1);
      ag_mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ag_mbar_init(&acc_full[b], 1);
      ag_mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    ag_fence_mbar_init();
  }
  __syncthreads();
  if (warp == 1) {
    // 512 columns: two accumulators of up to 256 fp32 columns each (this kernel owns the SM)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ag_smem_u32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = p.tiles_m * p.tiles_n * p.splits;
  bool expired = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !expired; tile += gridDim.x) {
        int tm, tn, k_begin, k_end, split_id;
        tc_tile_coords(p, tile, tm, tn, k_begin, k_end, split_id);
        const int m0 = tm * TC_BM, n0 = tn * p.BN;
        for (int k = k_begin; k < k_end; ++k) {
          if (!tc_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            expired = true;
            break;
          }
          unsigned char* s = tiles + (size_t)stage * stage_bytes;
          ag_mbar_expect_tx(&full[stage], stage_bytes);
          const int kx = k * p.BK;
          tc_tma_load_2d(&tmA_hi, s, &full[stage], kx, m0);
          if (p.split) {
            tc_tma_load_2d(&tmA_lo, s + p.a_bytes, &full[stage], kx, m0);
            tc_tma_load_2d(&tmB_hi, s + 2 * p.a_bytes, &full[stage], kx, n0);
            tc_tma_load_2d(&tmB_lo, s + 2 * p.a_bytes + p.b_bytes, &full[stage], kx, n0);
          } else {
            tc_tma_load_2d(&tmB_hi, s + p.a_bytes, &full[stage], kx, n0);
          }
          if (++stage == (uint32_t)p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t acc_par[2] = {0, 0};
      int local = 0;
      const int k_sub = p.BK / p.umma_k;  // MMAs per stage along K (4)
      for (int tile = blockIdx.x; tile < total_tiles && !expired; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        if (!tc_wait(&acc_empty[buf], acc_par[buf] ^ 1u, abort_flag)) {
          expired = true;
          break;
        }
        acc_par[buf] ^= 1u;
        tc_fence_after();
        const uint32_t tacc = tmem_base + (uint32_t)buf * 256u;
        int tm, tn, k_begin, k_end, split_id;
        tc_tile_coords(p, tile, tm, tn, k_begin, k_end, split_id);
        for (int k = k_begin; k < k_end; ++k) {
          if (!tc_wait(&full[stage], phase, abort_flag)) {
            expired = true;
            break;
          }
          tc_fence_after();
          const uint32_t s = ag_smem_u32(tiles + (size_t)stage * stage_bytes);
          const uint32_t a_hi = s, a_lo = s + p.a_bytes;
          const uint32_t b_hi = p.split ? s + 2 * p.a_bytes : s + p.a_bytes;
          const uint32_t b_lo = b_hi + p.b_bytes;
          for (int kk = 0; kk < k_sub; ++kk) {
            const uint32_t off = (uint32_t)kk * 32u;  // 32 bytes of K per MMA inside the 128-byte row
            const uint32_t first = (k == k_begin && kk == 0) ? 0u : 1u;
            if (p.split) {
              tc_mma<TF32>(tacc, tc_smem_desc(a_hi + off), tc_smem_desc(b_lo + off), p.idesc, first);
              tc_mma<TF32>(tacc, tc_smem_desc(a_lo + off), tc_smem_desc(b_hi + off), p.idesc, 1u);
              tc_mma<TF32>(tacc, tc_smem_desc(a_hi + off), tc_smem_desc(b_hi + off), p.idesc, 1u);
            } else {
              tc_mma<TF32>(tacc, tc_smem_desc(a_hi + off), tc_smem_desc(b_hi + off), p.idesc, first);
            }
          }
          tc_commit(&empty[stage]);  // stage reusable once these MMAs have read it
          if (++stage == (uint32_t)p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (expired) break;
        tc_commit(&acc_full[buf]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Two warps share each TMEM lane quarter and take alternate 32-column chunks of the tile: the
    // epilogues run one warp per scheduler, so their latency is exposed and more warps hide it.
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are this warp's
    const int half = (warp - 2) >> 2;
    const int c_first = half * 32;
    uint32_t full_par[2] = {0, 0};
    int local = 0;
    const bool vec_ok = ((p.ldd & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0) &&
                        (!p.bias || (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0) &&
                        (!p.resid || (((p.ld_resid & 3) == 0) && (reinterpret_cast<uintptr_t>(p.resid) & 15u) == 0));
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      int tm, tn, k_begin, k_end, split_id;
      tc_tile_coords(p, tile, tm, tn, k_begin, k_end, split_id);
      const int m0 = tm * TC_BM, n0 = tn * p.BN;
      if (!tc_wait(&acc_full[buf], full_par[buf], abort_flag)) {
        expired = true;
        break;
      }
      full_par[buf] ^= 1u;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * 256u;
      if (EPI == EPI_STORE) {
        float* drow = p.D + (int64_t)split_id * p.split_stride + (int64_t)row * p.ldd;
        for (int c0 = c_first; c0 < p.BN; c0 += 64) {
          uint32_t r[32];
          tc_tmem_ld32(tacc + (uint32_t)c0, r);
          tc_tmem_ld_wait();
          const int col = n0 + c0;
          if (row < p.M && col < p.N) {
            if (vec_ok && col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                       __uint_as_float(r[j + 3]));
                float4* dst = reinterpret_cast<float4*>(drow + col + j);
                if (p.accumulate) {
                  const float4 o = *dst;
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                if (p.bias) {
                  const float4 bv = *reinterpret_cast<const float4*>(p.bias + col + j);
                  v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
                }
                if (p.resid) {
                  const float4 rv = *reinterpret_cast<const float4*>(p.resid + (int64_t)row * p.ld_resid + col + j);
                  v.x += rv.x; v.y += rv.y; v.z += rv.z; v.w += rv.w;
                }
                *dst = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col + j < p.N) {
                  float v = __uint_as_float(r[j]);
                  if (p.accumulate) v += drow[col + j];
                  if (p.bias) v += p.bias[col + j];
                  if (p.resid) v += p.resid[(int64_t)row * p.ld_resid + col + j];
                  drow[col + j] = v;
                }
              }
            }
          }
        }
      } else if (EPI == EPI_STATS) {
        // (max, sum exp) of this row over the tile's columns, straight from TMEM: two sweeps
        const int tcol = row < p.M ? p.targets[row] - p.v0 : -1;  // panel-relative target column
        float mx = -INFINITY;
        for (int c0 = c_first; c0 < p.BN; c0 += 64) {
          uint32_t r[32];
          tc_tmem_ld32(tacc + (uint32_t)c0, r);
          tc_tmem_ld_wait();
          const int col = n0 + c0;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col + j < p.N) mx = fmaxf(mx, __uint_as_float(r[j]));
        }
        float sum = 0.0f, tl = 0.0f;
        bool have_t = false;
        for (int c0 = c_first; c0 < p.BN; c0 += 64) {
          uint32_t r[32];
          tc_tmem_ld32(tacc + (uint32_t)c0, r);
          tc_tmem_ld_wait();
          const int col = n0 + c0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col + j < p.N) {
              const float v = __uint_as_float(r[j]);
              sum += __expf(v - mx);
              if (col + j == tcol) { tl = v; have_t = true; }
            }
          }
        }
        if (row < p.M) {
          // a half that saw no valid column (narrow last tile) contributes (max -inf, sum 0)
          p.part[(int64_t)(tn * 2 + half) * p.part_ld + row] = make_float2(mx, sum);
          if (have_t) p.tgt_logit[row] = tl;
        }
      } else {
        // dlogits of this row, written in operand form: dl (row-major) and dl^T
        float sc = 0.0f, e = 0.0f;
        int tcol = -1;
        if (row < p.M) {
          const int t = p.targets[row];
          const bool valid = t >= 0 && t < p.V;
          sc = p.row_scale ? p.dloss[0] * p.row_scale[row] : p.dloss[0] / p.denom[0];
          if (!valid && p.ignore_mode == AG_CE_IGNORE_MASKED) sc = 0.0f;
          e = p.lse[row];
          tcol = valid ? t - p.v0 : -1;
        }
        const bool row_vec = ((p.ld_dl & 7) == 0);
        for (int c0 = c_first; c0 < p.BN; c0 += 64) {
          uint32_t r[32];
          tc_tmem_ld32(tacc + (uint32_t)c0, r);
          tc_tmem_ld_wait();
          const int col = n0 + c0;
          if (row >= p.M || col >= p.N) continue;
          float hi[32], lo[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float d = 0.0f;
            if (sc != 0.0f) {
              float pr = __expf(__uint_as_float(r[j]) - e);
              if (col + j == tcol) pr -= 1.0f;
              d = pr * sc;
            }
            if (TF32) {
              hi[j] = tc_tf32_rna(d);
              lo[j] = tc_tf32_rna(d - hi[j]);
            } else {
              hi[j] = d;
            }
          }
          if (TF32) {
            float* dh = static_cast<float*>(p.dl_hi) + (int64_t)row * p.ld_dl + col;
            float* dlo = static_cast<float*>(p.dl_lo) + (int64_t)row * p.ld_dl + col;
            if (row_vec && col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                *reinterpret_cast<float4*>(dh + j) = make_float4(hi[j], hi[j + 1], hi[j + 2], hi[j + 3]);
                *reinterpret_cast<float4*>(dlo + j) = make_float4(lo[j], lo[j + 1], lo[j + 2], lo[j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) { dh[j] = hi[j]; dlo[j] = lo[j]; }
            }
            float* th = static_cast<float*>(p.dlT_hi) + (int64_t)col * p.ld_dlT + row;
            float* tlo = static_cast<float*>(p.dlT_lo) + (int64_t)col * p.ld_dlT + row;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col + j < p.N) {  // lanes of a warp hold consecutive rows: each store is one 128-byte line
                th[(int64_t)j * p.ld_dlT] = hi[j];
                tlo[(int64_t)j * p.ld_dlT] = lo[j];
              }
            }
          } else {
            __nv_bfloat16* dh = static_cast<__nv_bfloat16*>(p.dl_hi) + (int64_t)row * p.ld_dl + col;
            if (row_vec && col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint32_t w[4];
#pragma unroll
                for (int q2 = 0; q2 < 4; ++q2) {
                  __nv_bfloat162 h2 = __floats2bfloat162_rn(hi[j + 2 * q2], hi[j + 2 * q2 + 1]);
                  w[q2] = *reinterpret_cast<uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(dh + j) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N) dh[j] = __float2bfloat16_rn(hi[j]);
            }
            __nv_bfloat16* th = static_cast<__nv_bfloat16*>(p.dlT_hi) + (int64_t)col * p.ld_dlT + row;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N) th[(int64_t)j * p.ld_dlT] = __float2bfloat16_rn(hi[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) ag_mbar_arrive(&acc_empty[buf]);
    }
  }
  if (expired && lane == 0) atomicOr(p.status, AG_STATUS_WAIT_EXPIRED);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------------------- host side
struct TcOperand {
  const void* hi;
  const void* lo;   // null in bf16 mode
  int64_t ld;       // elements between consecutive rows
};

// The driver API is reached through the runtime (cudaGetDriverEntryPoint) so that the library has
// no link-time dependency on libcuda and still loads on a machine without a driver.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn tc_encode_fn(ag_ctx* ctx) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
      snprintf(ctx->err, sizeof ctx->err, "cuTensorMapEncodeTiled is not available from this driver: %s",
               cudaGetErrorString(e));
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int tc_encode(ag_ctx* ctx, CUtensorMap* tm, const void* ptr, bool bf16, int64_t k_extent, int64_t rows, int64_t ld,
              int box_k, int box_rows) {
  EncodeTiledFn encode = tc_encode_fn(ctx);
  if (!encode) return AG_ERR_CUDA;
  const size_t es = bf16 ? 2 : 4;
  cuuint64_t dims[2] = {(cuuint64_t)k_extent, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * es};
  cuuint32_t box[2] = {(cuuint32_t)box_k, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                                      const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    AG_FAIL(ctx, AG_ERR_CUDA, "cuTensorMapEncodeTiled failed: CUresult %d (ptr %p, k %lld, rows %lld, ld %lld, box %dx%d)",
            (int)r, ptr, (long long)k_extent, (long long)rows, (long long)ld, box_k, box_rows);
  return AG_OK;
}

// D[M,N] (+)= A[M,K] . B[N,K]^T on the tensor cores.
// D[m][n] (+)= sum over splits, in split order, of the partial outputs P[s][m][n].
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ P, int splits, int M, int N, float* D, int64_t ldd, int accumulate) {
  const int64_t total = (int64_t)M * N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int m = (int)(i / N), n = (int)(i - (int64_t)m * N);
    float* d = D + (int64_t)m * ldd + n;
    float acc = accumulate ? *d : 0.0f;
    for (int sp = 0; sp < splits; ++sp) acc += P[(int64_t)sp * total + i];
    *d = acc;
  }
}

template <bool TF32, int EPI>
int tc_launch(ag_ctx* ctx, int grid, size_t smem, const CUtensorMap& a_hi, const CUtensorMap& a_lo,
              const CUtensorMap& b_hi, const CUtensorMap& b_lo, const TcParams& p) {
  static bool attr_done = false;
  if (!attr_done) {
    AG_CUDA(ctx, cudaFuncSetAttribute(tc_gemm_kernel<TF32, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      TC_SMEM_LIMIT));
    attr_done = true;
  }
  int rc_ev;
  if (ctx->tc_timing && (rc_ev = ag_event_record(ctx, ctx->tc_timing_base + 2 * ctx->tc_timing_count))) return rc_ev;
  tc_gemm_kernel<TF32, EPI><<<grid, TC_THREADS, smem, ctx->stream>>>(a_hi, a_lo, b_hi, b_lo, p);
  AG_LAUNCHED(ctx, "tc_gemm_kernel");
  if (ctx->tc_timing) {
    if ((rc_ev = ag_event_record(ctx, ctx->tc_timing_base + 2 * ctx->tc_timing_count + 1))) return rc_ev;
    ctx->tc_timing_count++;
  }
  return AG_OK;
}

// `epi` (may be null = EPI_STORE) carries the fields of the fused cross-entropy epilogues.
int tc_gemm(ag_ctx* ctx, bool bf16, const TcOperand& A, const TcOperand& B, float* D, int64_t ldd, int M, int N, int K,
            bool accumulate, int epi_kind = EPI_STORE, const TcParams* epi = nullptr, int* tiles_n_out = nullptr,
            float* splitk_ws = nullptr, size_t splitk_ws_bytes = 0) {
  TcParams p = {};
  if (epi) p = *epi;
  p.M = M; p.N = N; p.K = K;
  p.BK = bf16 ? 64 : 32;
  p.umma_k = bf16 ? 16 : 8;
  p.split = bf16 ? 0 : 1;
  // Tile width and split-K factor.  Measured behaviour of this kernel: a k-step costs time in
  // proportion to the operand bytes it pulls through shared memory (128 + BN rows), a tile costs
  // about 8 k-steps of prologue / epilogue on top, and CTAs work in rounds over the SMs.  Split-K
  // is only considered for plain accumulate outputs with a workspace and few tiles.
  const int cand[] = {256, 192, 160, 128};
  int best_bn = 128, best_s = 1;
  double best_cost = 1e300;
  const int tiles_m = (M + TC_BM - 1) / TC_BM;
  const int k_iters_all = (K + p.BK - 1) / p.BK;
  for (int bn : cand) {
    const int tn = (N + bn - 1) / bn;
    const int64_t tiles = (int64_t)tiles_m * tn;
    int s_max = 1;
    if (epi_kind == EPI_STORE && splitk_ws && tiles < 2 * (int64_t)ctx->sm_count) {
      s_max = k_iters_all / 16;
      if (s_max > 16) s_max = 16;
      const int64_t fit = (int64_t)(splitk_ws_bytes / ((size_t)M * N * sizeof(float)));
      if (s_max > fit) s_max = (int)fit;
      if (s_max < 1) s_max = 1;
    }
    for (int sp = 1; sp <= s_max; ++sp) {
      const int k_per = (k_iters_all + sp - 1) / sp;
      const int s_eff = (k_iters_all + k_per - 1) / k_per;
      const int64_t rounds = (tiles * s_eff + ctx->sm_count - 1) / ctx->sm_count;
      double cost = (double)rounds * (k_per + 8) * (128 + bn);
      if (s_eff > 1) cost += 0.02 * cost;  // the ordered reduction of the partial outputs
      if (cost < best_cost) {
        best_cost = cost;
        best_bn = bn;
        best_s = s_eff;
      }
    }
  }
  p.BN = best_bn;
  p.tiles_m = tiles_m;
  p.tiles_n = (N + p.BN - 1) / p.BN;
  if (tiles_n_out) *tiles_n_out = p.tiles_n;
  p.k_iters = k_iters_all;
  p.k_per_split = (p.k_iters + best_s - 1) / best_s;
  p.splits = (p.k_iters + p.k_per_split - 1) / p.k_per_split;
  p.split_stride = 0;
  p.a_bytes = (uint32_t)TC_BM * 128u;
  p.b_bytes = (uint32_t)p.BN * 128u;
  const uint32_t stage_bytes = (p.a_bytes + p.b_bytes) * (p.split ? 2u : 1u);
  int stages = (TC_SMEM_LIMIT - 1024 - 256) / (int)stage_bytes;
  if (stages > TC_MAX_STAGES) stages = TC_MAX_STAGES;
  AG_REQUIRE(ctx, stages >= 2, "tc_gemm: tile does not fit shared memory");
  p.stages = stages;
  // per-wave operand footprint decides the tile order (keep the re-read operand in L2)
  {
    const int64_t sm = ctx->sm_count;
    const int64_t fp_m_fast = (tiles_m < sm ? tiles_m : sm) * (int64_t)p.a_bytes + ((sm + tiles_m - 1) / tiles_m) * (int64_t)p.b_bytes;
    const int64_t fp_n_fast = (p.tiles_n < sm ? p.tiles_n : sm) * (int64_t)p.b_bytes + ((sm + p.tiles_n - 1) / p.tiles_n) * (int64_t)p.a_bytes;
    p.n_fastest = fp_n_fast <= fp_m_fast ? 1 : 0;
  }
  // instruction descriptor: D fp32, A/B tf32 or bf16, both K-major, N>>3 at bit 17, M>>4 at bit 24
  const uint32_t fmt = bf16 ? 1u : 2u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
  p.D = D; p.ldd = ldd; p.accumulate = accumulate ? 1 : 0;
  if (p.splits > 1) {  // partial outputs [splits][M][N] in the workspace, summed in order afterwards
    p.D = splitk_ws;
    p.ldd = N;
    p.accumulate = 0;
    p.split_stride = (int64_t)M * N;
  }
  p.status = ctx->d_status;

  CUtensorMap tA_hi, tA_lo, tB_hi, tB_lo;
  int rc;
  if ((rc = tc_encode(ctx, &tA_hi, A.hi, bf16, K, M, A.ld, p.BK, TC_BM))) return rc;
  if ((rc = tc_encode(ctx, &tB_hi, B.hi, bf16, K, N, B.ld, p.BK, p.BN))) return rc;
  if (p.split) {
    if ((rc = tc_encode(ctx, &tA_lo, A.lo, bf16, K, M, A.ld, p.BK, TC_BM))) return rc;
    if ((rc = tc_encode(ctx, &tB_lo, B.lo, bf16, K, N, B.ld, p.BK, p.BN))) return rc;
  } else {
    tA_lo = tA_hi;
    tB_lo = tB_hi;
  }
  const size_t smem = 1024 + (size_t)stages * stage_bytes + 256;
  const int64_t total = (int64_t)p.tiles_m * p.tiles_n * p.splits;
  const int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
  if (epi_kind == EPI_STATS) {
    AG_REQUIRE(ctx, p.part_ld >= M, "tc_gemm: partial-statistics rows too short");
    return bf16 ? tc_launch<false, EPI_STATS>(ctx, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p)
                : tc_launch<true, EPI_STATS>(ctx, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p);
  }
  if (epi_kind == EPI_DLOGITS)
    return bf16 ? tc_launch<false, EPI_DLOGITS>(ctx, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p)
                : tc_launch<true, EPI_DLOGITS>(ctx, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p);
  rc = bf16 ? tc_launch<false, EPI_STORE>(ctx, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p)
            : tc_launch<true, EPI_STORE>(ctx, grid, smem, tA_hi, tA_lo, tB_hi, tB_lo, p);
  if (rc || p.splits == 1) return rc;
  const int64_t n4 = ((int64_t)M * N + 3) / 4;
  int64_t want = (n4 + 255) / 256;
  if (want > (int64_t)ctx->sm_count * 8) want = (int64_t)ctx->sm_count * 8;
  splitk_reduce_kernel<<<(int)want, 256, 0, ctx->stream>>>(splitk_ws, p.splits, M, N, D, ldd, accumulate ? 1 : 0);
  AG_LAUNCHED(ctx, "splitk_reduce_kernel");
  return AG_OK;
}

// ---------------------------------------------------------------------------- operand preparation
__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  hi = tf32_rna(x);
  lo = tf32_rna(x - hi);
}

// src[R][Cc] (row stride lds) -> hi/lo [R][Cc] (row stride ldo) and, when the T pointers are given,
// hiT/loT [Cc][R] (row stride ldt).  32x32 tiles through shared memory; block (32, 8).
// BF16: the outputs are bf16 (hi only).
template <bool BF16>
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ src, int64_t lds, void* __restrict__ hi, void* __restrict__ lo,
                       int64_t ldo, void* __restrict__ hiT, void* __restrict__ loT, int64_t ldt, int R, int Cc) {
  __shared__ float s_hi[32][33];
  __shared__ float s_lo[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    float h = 0.0f, l = 0.0f;
    if (r < R && c < Cc) {
      const float x = src[(int64_t)r * lds + c];
      if (BF16) {
        h = x;
      } else {
        split_tf32(x, h, l);
      }
      if (hi) {
        if (BF16) {
          static_cast<__nv_bfloat16*>(hi)[(int64_t)r * ldo + c] = __float2bfloat16_rn(h);
        } else {
          static_cast<float*>(hi)[(int64_t)r * ldo + c] = h;
          static_cast<float*>(lo)[(int64_t)r * ldo + c] = l;
        }
      }
    }
    s_hi[i][threadIdx.x] = h;
    s_lo[i][threadIdx.x] = l;
  }
  if (!hiT) return;
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + threadIdx.x;  // output row = source column
    if (c < Cc && r < R) {
      if (BF16) {
        static_cast<__nv_bfloat16*>(hiT)[(int64_t)c * ldt + r] = __float2bfloat16_rn(s_hi[threadIdx.x][i]);
      } else {
        static_cast<float*>(hiT)[(int64_t)c * ldt + r] = s_hi[threadIdx.x][i];
        static_cast<float*>(loT)[(int64_t)c * ldt + r] = s_lo[threadIdx.x][i];
      }
    }
  }
}

// dlogits of one panel, written straight in tensor-core operand form:
//   dl[r][c] = scale_r * (exp(L[r][c] - lse[r]) - [c == target_r - v0])   (0 for ignored rows when masked)
// -> dl (hi, lo) [rows][ld_dl] and dl^T (hi, lo) [vc][ld_dlT].
template <bool BF16>
__global__ void __launch_bounds__(256)
dlogits_split_kernel(const float* __restrict__ L, int64_t ldl, int rows, int vc, int v0,
                     const int32_t* __restrict__ targets, const float* __restrict__ lse,
                     const float* __restrict__ row_scale, const float* __restrict__ dloss,
                     const float* __restrict__ denom, int V, int ignore_mode, void* __restrict__ dl_hi,
                     void* __restrict__ dl_lo, int64_t ld_dl, void* __restrict__ dlT_hi, void* __restrict__ dlT_lo,
                     int64_t ld_dlT) {
  __shared__ float s_hi[32][33];
  __shared__ float s_lo[32][33];
  __shared__ float s_lse[32], s_scale[32];
  __shared__ int s_tc[32];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  if (threadIdx.y == 0) {
    const int r = r0 + threadIdx.x;
    float sc = 0.0f, e = 0.0f;
    int tc = -1;
    if (r < rows) {
      const int t = targets[r];
      const bool valid = t >= 0 && t < V;
      sc = row_scale ? dloss[0] * row_scale[r] : dloss[0] / denom[0];
      if (!valid && ignore_mode == AG_CE_IGNORE_MASKED) sc = 0.0f;
      e = lse[r];
      tc = valid ? t - v0 : -1;
    }
    s_lse[threadIdx.x] = e;
    s_scale[threadIdx.x] = sc;
    s_tc[threadIdx.x] = tc;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    float h = 0.0f, l = 0.0f;
    if (r < rows && c < vc) {
      const float sc = s_scale[i];
      float d = 0.0f;
      if (sc != 0.0f) {
        float pr = expf(L[(int64_t)r * ldl + c] - s_lse[i]);
        if (c == s_tc[i]) pr -= 1.0f;
        d = pr * sc;
      }
      if (BF16) {
        h = d;
        static_cast<__nv_bfloat16*>(dl_hi)[(int64_t)r * ld_dl + c] = __float2bfloat16_rn(d);
      } else {
        split_tf32(d, h, l);
        static_cast<float*>(dl_hi)[(int64_t)r * ld_dl + c] = h;
        static_cast<float*>(dl_lo)[(int64_t)r * ld_dl + c] = l;
      }
    }
    s_hi[i][threadIdx.x] = h;
    s_lo[i][threadIdx.x] = l;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (c < vc && r < rows) {
      if (BF16) {
        static_cast<__nv_bfloat16*>(dlT_hi)[(int64_t)c * ld_dlT + r] = __float2bfloat16_rn(s_hi[threadIdx.x][i]);
      } else {
        static_cast<float*>(dlT_hi)[(int64_t)c * ld_dlT + r] = s_hi[threadIdx.x][i];
        static_cast<float*>(dlT_lo)[(int64_t)c * ld_dlT + r] = s_lo[threadIdx.x][i];
      }
    }
  }
}

// Folds the per-tile (max, sum exp) partials of one panel into the running row statistics, tiles
// in index order (fixed order, one thread per row).
__global__ void __launch_bounds__(256)
ce_merge_partials_kernel(const float2* __restrict__ part, int64_t part_ld, int tiles_n, int rows,
                         float* __restrict__ run_max, float* __restrict__ run_sum, int first_panel) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float m, s;
  int t0 = 0;
  if (first_panel) {
    const float2 v = part[r];
    m = v.x; s = v.y; t0 = 1;
  } else {
    m = run_max[r]; s = run_sum[r];
  }
  for (int t = t0; t < tiles_n; ++t) {
    const float2 v = part[(int64_t)t * part_ld + r];
    if (v.y == 0.0f) continue;  // an empty partial (max = -inf)
    const float nm = fmaxf(m, v.x);
    s = s * expf(m - nm) + v.y * expf(v.x - nm);
    m = nm;
  }
  run_max[r] = m;
  run_sum[r] = s;
}

// ---------------------------------------------------------------------------- workspace plan
struct TcPlan {
  int64_t rows_tile, vc, ldn;  // ldn: row stride of the [C][N] transposed activations
  size_t es;                   // operand element size
  size_t X_hi, X_lo, XT_hi, XT_lo, W_hi, W_lo, WT_hi, WT_lo, dl_hi, dl_lo, dlT_hi, dlT_lo, part, splitk, splitk_bytes,
      total;
  int64_t part_ld;
};

inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }
inline int64_t up8(int64_t x) { return (x + 7) & ~(int64_t)7; }

TcPlan tc_plan(const ag_flce_desc* d) {
  TcPlan p;
  const bool bf16 = d->precision == AG_CE_BF16;
  p.es = bf16 ? 2 : 4;
  p.rows_tile = d->N < 16384 ? d->N : 16384;
  p.vc = d->vocab_chunk < d->V ? d->vocab_chunk : d->V;
  p.ldn = up8(d->N);
  const int64_t ldv = up8(d->V), ldr = up8(p.rows_tile), ldc = up8(p.vc);
  size_t off = 0;
  auto take = [&](size_t elems) { size_t o = off; off += up256(elems * p.es); return o; };
  p.X_hi = take((size_t)d->N * d->C);
  p.X_lo = bf16 ? p.X_hi : take((size_t)d->N * d->C);
  p.W_hi = take((size_t)d->V * d->C);
  p.W_lo = bf16 ? p.W_hi : take((size_t)d->V * d->C);
  p.XT_hi = take((size_t)d->C * p.ldn);
  p.XT_lo = bf16 ? p.XT_hi : take((size_t)d->C * p.ldn);
  p.WT_hi = take((size_t)d->C * ldv);
  p.WT_lo = bf16 ? p.WT_hi : take((size_t)d->C * ldv);
  p.dl_hi = take((size_t)p.rows_tile * ldc);
  p.dl_lo = bf16 ? p.dl_hi : take((size_t)p.rows_tile * ldc);
  p.dlT_hi = take((size_t)p.vc * ldr);
  p.dlT_lo = bf16 ? p.dlT_hi : take((size_t)p.vc * ldr);
  // per (column tile, epilogue half, row) partial softmax statistics of one panel
  p.part_ld = ldr;
  p.part = off;
  off += up256((size_t)((p.vc + 127) / 128) * 2 * ldr * sizeof(float2));
  // split-K partial outputs of the dW panel GEMM (vc x C), up to 16 splits
  p.splitk = off;
  p.splitk_bytes = up256((size_t)16 * p.vc * d->C * sizeof(float));
  off += p.splitk_bytes;
  p.total = off;
  return p;
}

}  // namespace

// ---- entry points for other translation units (ag_flce.cuh) ---------------------------------
int ag_tc_gemm(ag_ctx* ctx, bool bf16, const AgTcOperand& A, const AgTcOperand& B, float* D, int64_t ldd, int M, int N,
               int K, bool accumulate, const float* bias, const float* resid, int64_t ld_resid, float* splitk_ws,
               size_t splitk_ws_bytes) {
  TcParams e = {};
  e.bias = bias;
  e.resid = resid;
  e.ld_resid = ld_resid;
  TcOperand a{A.hi, A.lo, A.ld}, b{B.hi, B.lo, B.ld};
  return tc_gemm(ctx, bf16, a, b, D, ldd, M, N, K, accumulate, EPI_STORE, &e, nullptr, splitk_ws, splitk_ws_bytes);
}

int ag_tc_split(ag_ctx* ctx, bool bf16, const float* src, int64_t lds, void* hi, void* lo, int64_t ldo, void* hiT,
                void* loT, int64_t ldt, int R, int Cc) {
  dim3 grid((Cc + 31) / 32, (R + 31) / 32);
  if (bf16)
    split_transpose_kernel<true><<<grid, dim3(32, 8), 0, ctx->stream>>>(src, lds, hi, lo, ldo, hiT, loT, ldt, R, Cc);
  else
    split_transpose_kernel<false><<<grid, dim3(32, 8), 0, ctx->stream>>>(src, lds, hi, lo, ldo, hiT, loT, ldt, R, Cc);
  AG_LAUNCHED(ctx, "split_transpose_kernel");
  return AG_OK;
}

// =========================================================================================
bool ag_flce_tc_supported(const ag_flce_desc* d) {
  if (d->precision != AG_CE_3XTF32 && d->precision != AG_CE_BF16) return false;
  // TMA needs 16-byte aligned row starts: rows of X / W are C elements long
  const int q = d->precision == AG_CE_BF16 ? 8 : 4;
  if (d->C % q != 0) return false;
  if (d->vocab_chunk % 8 != 0 && d->vocab_chunk < d->V) return false;
  if (d->C < 32 || d->V < 32 || d->N < 1) return false;
  return true;
}

size_t ag_flce_tc_scratch_bytes(const ag_flce_desc* d) { return tc_plan(d).total; }

int ag_flce_tc_prepare(ag_ctx* ctx, const ag_flce_desc* d, const float* X, const float* W, void* tc_scratch,
                       bool backward) {
  const TcPlan p = tc_plan(d);
  unsigned char* b = static_cast<unsigned char*>(tc_scratch);
  const bool bf16 = d->precision == AG_CE_BF16;
  const dim3 blk(32, 8);
  const int64_t ldv = up8(d->V);
  {
    dim3 grid((d->C + 31) / 32, (unsigned)((d->N + 31) / 32));
    void* hT = backward ? b + p.XT_hi : nullptr;
    void* lT = backward ? b + p.XT_lo : nullptr;
    if (bf16)
      split_transpose_kernel<true><<<grid, blk, 0, ctx->stream>>>(X, d->C, b + p.X_hi, b + p.X_lo, d->C, hT, lT, p.ldn,
                                                                   (int)d->N, d->C);
    else
      split_transpose_kernel<false><<<grid, blk, 0, ctx->stream>>>(X, d->C, b + p.X_hi, b + p.X_lo, d->C, hT, lT,
                                                                    p.ldn, (int)d->N, d->C);
    AG_LAUNCHED(ctx, "split_transpose_kernel(X)");
  }
  {
    dim3 grid((d->C + 31) / 32, (unsigned)((d->V + 31) / 32));
    void* hT = backward ? b + p.WT_hi : nullptr;
    void* lT = backward ? b + p.WT_lo : nullptr;
    if (bf16)
      split_transpose_kernel<true><<<grid, blk, 0, ctx->stream>>>(W, d->C, b + p.W_hi, b + p.W_lo, d->C, hT, lT, ldv,
                                                                   d->V, d->C);
    else
      split_transpose_kernel<false><<<grid, blk, 0, ctx->stream>>>(W, d->C, b + p.W_hi, b + p.W_lo, d->C, hT, lT, ldv,
                                                                    d->V, d->C);
    AG_LAUNCHED(ctx, "split_transpose_kernel(W)");
  }
  return AG_OK;
}

int ag_flce_tc_logits(ag_ctx* ctx, const ag_flce_desc* d, void* tc_scratch, int64_t r0, int rows, int v0, int vc,
                      float* panel, int64_t ld) {
  const TcPlan p = tc_plan(d);
  unsigned char* b = static_cast<unsigned char*>(tc_scratch);
  const bool bf16 = d->precision == AG_CE_BF16;
  const size_t row_bytes = (size_t)d->C * p.es;
  TcOperand A{b + p.X_hi + (size_t)r0 * row_bytes, b + p.X_lo + (size_t)r0 * row_bytes, d->C};
  TcOperand B{b + p.W_hi + (size_t)v0 * row_bytes, b + p.W_lo + (size_t)v0 * row_bytes, d->C};
  return tc_gemm(ctx, bf16, A, B, panel, ld, rows, vc, d->C, false);
}

int ag_flce_tc_forward_panel(ag_ctx* ctx, const ag_flce_desc* d, void* tc_scratch, int64_t r0, int rows, int v0,
                             int vc, const int32_t* targets, float* run_max, float* run_sum, float* tgt_logit,
                             bool first_panel) {
  const TcPlan p = tc_plan(d);
  unsigned char* b = static_cast<unsigned char*>(tc_scratch);
  const bool bf16 = d->precision == AG_CE_BF16;
  const size_t row_bytes = (size_t)d->C * p.es;
  TcOperand A{b + p.X_hi + (size_t)r0 * row_bytes, b + p.X_lo + (size_t)r0 * row_bytes, d->C};
  TcOperand B{b + p.W_hi + (size_t)v0 * row_bytes, b + p.W_lo + (size_t)v0 * row_bytes, d->C};
  TcParams e = {};
  e.targets = targets + r0;
  e.v0 = v0;
  e.V = d->V;
  e.part = reinterpret_cast<float2*>(b + p.part);
  e.part_ld = p.part_ld;
  e.tgt_logit = tgt_logit + r0;
  int tiles_n = 0;
  int rc = tc_gemm(ctx, bf16, A, B, nullptr, 0, rows, vc, d->C, false, EPI_STATS, &e, &tiles_n);
  if (rc) return rc;
  ce_merge_partials_kernel<<<(rows + 255) / 256, 256, 0, ctx->stream>>>(e.part, e.part_ld, tiles_n * 2, rows, run_max + r0,
                                                                      run_sum + r0, first_panel ? 1 : 0);
  AG_LAUNCHED(ctx, "ce_merge_partials_kernel");
  return AG_OK;
}

int ag_flce_tc_grads(ag_ctx* ctx, const ag_flce_desc* d, void* tc_scratch, int64_t r0, int rows, int v0, int vc,
                     const int32_t* targets, const float* lse, const float* row_scale, const float* dloss,
                     const float* denom, float* dX, float* dW) {
  const TcPlan p = tc_plan(d);
  unsigned char* b = static_cast<unsigned char*>(tc_scratch);
  const bool bf16 = d->precision == AG_CE_BF16;
  const int64_t ldc = up8(p.vc), ldr = up8(p.rows_tile), ldv = up8(d->V);
  const size_t row_bytes = (size_t)d->C * p.es;
  int rc;
  {
    // logits panel recomputed on the tensor cores; its epilogue writes dlogits in operand form
    TcOperand A{b + p.X_hi + (size_t)r0 * row_bytes, b + p.X_lo + (size_t)r0 * row_bytes, d->C};
    TcOperand B{b + p.W_hi + (size_t)v0 * row_bytes, b + p.W_lo + (size_t)v0 * row_bytes, d->C};
    TcParams e = {};
    e.targets = targets + r0;
    e.v0 = v0;
    e.V = d->V;
    e.lse = lse + r0;
    e.row_scale = row_scale ? row_scale + r0 : nullptr;
    e.dloss = dloss;
    e.denom = denom;
    e.ignore_mode = d->ignore_mode;
    e.dl_hi = b + p.dl_hi; e.dl_lo = b + p.dl_lo; e.ld_dl = ldc;
    e.dlT_hi = b + p.dlT_hi; e.dlT_lo = b + p.dlT_lo; e.ld_dlT = ldr;
    if ((rc = tc_gemm(ctx, bf16, A, B, nullptr, 0, rows, vc, d->C, false, EPI_DLOGITS, &e))) return rc;
  }
  if (dX) {
    // dX[r0:r0+rows, :] += dl [rows, vc] . (W^T [C, v0:v0+vc])^T
    TcOperand A{b + p.dl_hi, b + p.dl_lo, ldc};
    TcOperand B{b + p.WT_hi + (size_t)v0 * p.es, b + p.WT_lo + (size_t)v0 * p.es, ldv};
    if ((rc = tc_gemm(ctx, bf16, A, B, dX + r0 * d->C, d->C, rows, d->C, vc, true))) return rc;
  }
  if (dW) {
    // dW[v0:v0+vc, :] += dl^T [vc, rows] . (X^T [C, r0:r0+rows])^T
    TcOperand A{b + p.dlT_hi, b + p.dlT_lo, ldr};
    TcOperand B{b + p.XT_hi + (size_t)r0 * p.es, b + p.XT_lo + (size_t)r0 * p.es, p.ldn};
    if ((rc = tc_gemm(ctx, bf16, A, B, dW + (int64_t)v0 * d->C, d->C, vc, d->C, rows, true, EPI_STORE, nullptr, nullptr,
                      reinterpret_cast<float*>(b + p.splitk), p.splitk_bytes)))
      return rc;
  }
  return AG_OK;
}
